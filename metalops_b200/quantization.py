"""Host-side mirror of metalcore's quantization API for the q4_0 path, backed by sm_100a CUDA.

Same names, argument order, defaults, return shapes and dtypes as the reference's
``packages/metalcore/src/metalcore/quantization.py`` (q4_0 part: lines 288-454), so a caller
can switch ``from metalcore import ...`` to ``from metalops_b200 import ...``.  Differences, all
forced by "CUDA only, no fallback":

* tensors must live on a CUDA device of compute capability 10.x; a CPU tensor raises
  ``RuntimeError`` instead of taking the reference's pure-torch path (quantization.py:453-454);
* ``matmul_ggml_q4_0`` computes with fp32 accumulation from the packed weights and returns
  ``X.dtype`` (the reference's torch path dequantises to ``X.dtype`` and calls ``X @ W``);
  fp32 ``X`` is computed through fp16 like the reference's Metal entry does
  (``X.half()``, quantization.py:448) and returned as fp32;
* the packed weights are additionally kept in a streaming layout ("prepacked", see
  ``include/q4b200.h``).  ``quantize_ggml_q4_0`` writes it in the same kernel pass and attaches
  it to the returned tensor; a ``W_blocks`` tensor that arrives without one (e.g. loaded from a
  checkpoint) is repacked on first use and the result cached on the tensor object.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn as nn

from . import _cabi

QK4_0 = 32                       # quantization.py:303
BLOCK_Q4_0_SIZE = 2 + QK4_0 // 2  # quantization.py:304

GEMV_MAX_M = 16                  # M <= 16 -> decode kernel, else tcgen05 kernel


class Q4Prepacked:
    """Device buffer holding a weight in the streaming tile layout, plus its logical shape."""

    __slots__ = ("data", "K", "N")

    def __init__(self, data: torch.Tensor, K: int, N: int):
        self.data, self.K, self.N = data, K, N

    @property
    def device(self) -> torch.device:
        return self.data.device

    def nbytes(self) -> int:
        return self.data.numel()


def _alloc_prepacked(K: int, N: int, device: torch.device) -> torch.Tensor:
    nbytes = _cabi.load().q4b_prepacked_bytes(K, N)
    if nbytes == 0:
        raise AssertionError(f"K ({K}) must be divisible by {QK4_0}")
    return torch.empty(nbytes, dtype=torch.uint8, device=device)


def _quantize_impl(weight: torch.Tensor, want_blocks: bool, want_prepacked: bool):
    """Shared by quantize_ggml_q4_0 and Q4Prepacked.from_float; returns (blocks, Q4Prepacked)."""
    if weight.dim() != 2:
        raise ValueError("weight must be 2-D [K, N]")
    _cabi.require_device(weight, "weight")
    if weight.dtype not in _cabi.DTYPE_CODE:
        raise RuntimeError(f"unsupported weight dtype {weight.dtype}")
    K, N = weight.shape
    assert K % QK4_0 == 0, f"K ({K}) must be divisible by {QK4_0}"
    # A transposed view of a contiguous [N, K] tensor (nn.Linear.weight.T) is read in place.
    if weight.is_contiguous():
        layout, src = _cabi.LAYOUT_KN, weight
    elif weight.t().is_contiguous():
        layout, src = _cabi.LAYOUT_NK, weight.t()
    else:
        layout, src = _cabi.LAYOUT_KN, weight.contiguous()
    dev = weight.device
    blocks = torch.empty((K // QK4_0, N, BLOCK_Q4_0_SIZE), dtype=torch.uint8, device=dev) if want_blocks else None
    pre = _alloc_prepacked(K, N, dev) if want_prepacked else None
    with torch.cuda.device(dev):
        rc = _cabi.load().q4b_quantize(
            src.data_ptr(), _cabi.DTYPE_CODE[src.dtype], K, N, layout,
            blocks.data_ptr() if blocks is not None else None,
            pre.data_ptr() if pre is not None else None, _cabi.stream_ptr(dev))
    _cabi.check(rc, "quantize_ggml_q4_0")
    return blocks, (Q4Prepacked(pre, K, N) if pre is not None else None)


def quantize_ggml_q4_0(weight: torch.Tensor) -> torch.Tensor:
    """Quantize ``weight [K, N]`` to GGML block_q4_0: returns uint8 ``[K/32, N, 18]``.

    Bit-identical to the reference (quantization.py:307-371) for fp32, fp16 and bf16 weights.
    Note the reference's docstring says ``[num_blocks, 18]``; its code and this function return
    ``[K/32, N, 18]``.
    """
    blocks, pre = _quantize_impl(weight, True, True)
    blocks._q4b_prepacked = (blocks._version, pre)
    return blocks


def prepack_ggml_q4_0(W_blocks: torch.Tensor) -> Q4Prepacked:
    """Streaming-layout copy of ``W_blocks [K/32, N, 18]`` (cached on the tensor object)."""
    cached = getattr(W_blocks, "_q4b_prepacked", None)
    if cached is not None and cached[0] == W_blocks._version and cached[1].device == W_blocks.device:
        return cached[1]
    _cabi.require_device(W_blocks, "W_blocks")
    if W_blocks.dtype != torch.uint8 or W_blocks.dim() != 3 or W_blocks.shape[2] != BLOCK_Q4_0_SIZE:
        raise RuntimeError("W_blocks must be uint8 [K/32, N, 18]")           # core_mps.mm:5926,5938
    wb = W_blocks.contiguous()
    K, N = wb.shape[0] * QK4_0, wb.shape[1]
    pre = _alloc_prepacked(K, N, wb.device)
    with torch.cuda.device(wb.device):
        rc = _cabi.load().q4b_repack(wb.data_ptr(), K, N, pre.data_ptr(), _cabi.stream_ptr(wb.device))
    _cabi.check(rc, "prepack_ggml_q4_0")
    out = Q4Prepacked(pre, K, N)
    try:
        W_blocks._q4b_prepacked = (W_blocks._version, out)
    except AttributeError:
        pass
    return out


def unpack_ggml_q4_0(pre: Q4Prepacked) -> torch.Tensor:
    """Inverse of :func:`prepack_ggml_q4_0`: the interchange ``[K/32, N, 18]`` tensor."""
    blocks = torch.empty((pre.K // QK4_0, pre.N, BLOCK_Q4_0_SIZE), dtype=torch.uint8, device=pre.device)
    with torch.cuda.device(pre.device):
        rc = _cabi.load().q4b_unpack(pre.data.data_ptr(), pre.K, pre.N, blocks.data_ptr(),
                                     _cabi.stream_ptr(pre.device))
    _cabi.check(rc, "unpack_ggml_q4_0")
    return blocks


def dequantize_ggml_q4_0(blocks: torch.Tensor, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """Dequantize ``[K/32, N, 18]`` blocks to a dense ``[K, N]`` tensor (default fp16).

    ``W = (q - 8) * float(d)`` in fp32, then cast — quantization.py:374-419."""
    if dtype is None:
        dtype = torch.float16
    _cabi.require_device(blocks, "blocks")
    if blocks.dtype != torch.uint8 or blocks.dim() != 3 or blocks.shape[2] != BLOCK_Q4_0_SIZE:
        raise RuntimeError("blocks must be uint8 [K/32, N, 18]")
    if dtype not in _cabi.DTYPE_CODE:
        raise RuntimeError(f"unsupported output dtype {dtype}")
    b = blocks.contiguous()
    K, N = b.shape[0] * QK4_0, b.shape[1]
    W = torch.empty((K, N), dtype=dtype, device=b.device)
    with torch.cuda.device(b.device):
        rc = _cabi.load().q4b_dequantize(b.data_ptr(), K, N, W.data_ptr(), _cabi.DTYPE_CODE[dtype],
                                         _cabi.stream_ptr(b.device))
    _cabi.check(rc, "dequantize_ggml_q4_0")
    return W


def _matmul_prepacked(X: torch.Tensor, pre: Q4Prepacked, out: Optional[torch.Tensor] = None,
                      flags: int = _cabi.FLAG_NONE, kernel: str = "auto") -> torch.Tensor:
    _cabi.require_device(X, "X")
    if X.device != pre.device:
        raise RuntimeError(f"X is on {X.device} but the weights are on {pre.device}")
    assert X.shape[1] == pre.K, f"X K dim ({X.shape[1]}) must match weight K ({pre.K})"
    in_dtype = X.dtype
    if in_dtype == torch.float32:
        X = X.half()                         # the reference's native entry does the same (quantization.py:448)
    elif in_dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError(f"X must be float16, bfloat16 or float32 (got {in_dtype})")
    x = X if (X.stride(1) == 1 and X.stride(0) % 8 == 0 and X.data_ptr() % 16 == 0) else X.contiguous()
    if x.stride(0) % 8 or x.data_ptr() % 16:
        x = x.clone(memory_format=torch.contiguous_format)
    M = x.shape[0]
    if M == 0:
        return torch.empty((0, pre.N), dtype=in_dtype, device=X.device)
    y = out if (out is not None and in_dtype != torch.float32) else torch.empty((M, pre.N), dtype=x.dtype, device=x.device)
    if y.shape != (M, pre.N) or y.dtype != x.dtype or y.stride(1) != 1:
        raise RuntimeError("out must be [M, N], X's dtype, unit inner stride")
    lib = _cabi.load()
    fn = {"auto": lib.q4b_matmul, "gemv": lib.q4b_gemv, "gemm": lib.q4b_gemm}[kernel]
    with torch.cuda.device(x.device):
        rc = fn(x.data_ptr(), _cabi.DTYPE_CODE[x.dtype], M, x.stride(0), pre.data.data_ptr(), pre.K, pre.N,
                y.data_ptr(), y.stride(0), flags, _cabi.stream_ptr(x.device))
    _cabi.check(rc, "matmul_ggml_q4_0")
    return y.float() if in_dtype == torch.float32 else y


def wait_status(device=None) -> int:
    """Synchronise the current stream and return the prefill kernel's bounded-wait status:
    0 when every wait completed, else the code of the first wait that gave up (also raises)."""
    import ctypes
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    detail = ctypes.c_int(0)
    with torch.cuda.device(dev):
        rc = _cabi.load().q4b_wait_status(_cabi.stream_ptr(dev), ctypes.byref(detail))
    if rc == _cabi.ERR_TIMEOUT:
        raise RuntimeError(f"q4b_gemm: a bounded device-side wait gave up (code {detail.value})")
    _cabi.check(rc, "q4b_wait_status")
    return detail.value


def matmul_ggml_q4_0(X: torch.Tensor, W_blocks) -> torch.Tensor:
    """``Y = X @ dequant(W_blocks)`` — quantization.py:422-454.

    ``X`` is ``[M, K]`` (2-D only, like the reference); ``W_blocks`` is the uint8
    ``[K/32, N, 18]`` tensor from :func:`quantize_ggml_q4_0` (or a :class:`Q4Prepacked`).
    Returns ``[M, N]`` in ``X.dtype``.  M <= 16 runs the decode GEMV kernel, larger M the
    tcgen05 GEMM kernel.
    """
    if X.dim() != 2:
        raise RuntimeError("X must be 2-D [M, K]")
    pre = W_blocks if isinstance(W_blocks, Q4Prepacked) else prepack_ggml_q4_0(W_blocks)
    return _matmul_prepacked(X, pre)


# ---------------------------------------------------------------------------------------
# Group-wise asymmetric INT4 / INT8 entry points of the reference (quantization.py:26-286).
# Their native kernels are not part of this build yet; they raise rather than fall back.
# ---------------------------------------------------------------------------------------

def _not_built(name: str):
    raise NotImplementedError(
        f"{name}: the group-wise INT4/INT8 format has no sm_100a kernel in this build yet, and "
        "there is no CPU fallback by design; use the q4_0 entry points")


def quantize_int4(weight: torch.Tensor, group_size: int = 128) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    _not_built("quantize_int4")


def dequantize_int4(W_packed, scales, zeros, group_size: int = 128, dtype: Optional[torch.dtype] = None):
    _not_built("dequantize_int4")


def matmul_int4(X, W_packed, scales, zeros, group_size: int = 128):
    _not_built("matmul_int4")


def matmul_int8(X, W_packed, scales, zeros, group_size: int = 128):
    _not_built("matmul_int8")


class Int4Linear(nn.Module):
    """INT4 linear layer with the constructor, methods and ``extra_repr`` of the reference's
    ``Int4Linear`` (quantization.py:457-612), storing the weight as q4_0 blocks.

    Buffers: ``weight_blocks`` uint8 ``[in/32, out, 18]`` (serialised) and ``bias``.  The
    streaming copy used by the kernels is derived state, rebuilt after ``load_state_dict`` /
    ``.to()``.  ``group_size`` is accepted for signature compatibility; q4_0 fixes it at 32.
    ``dequant_on_load=True`` keeps a dense fp16 copy and uses a plain fp16 matmul exactly like
    the reference's "hybrid" mode (quantization.py:593-597); the default here is ``False``
    because the fused kernels are the point of this build.
    """

    def __init__(self, in_features: int, out_features: int, group_size: int = 128, bias: bool = True,
                 device: Optional[torch.device] = None, dtype: Optional[torch.dtype] = None,
                 dequant_on_load: bool = False):
        super().__init__()
        if in_features % QK4_0:
            raise AssertionError(f"in_features ({in_features}) must be divisible by {QK4_0}")
        self.in_features = in_features
        self.out_features = out_features
        self.group_size = group_size
        self._dequant_on_load = dequant_on_load
        blocks = torch.zeros((in_features // QK4_0, out_features, BLOCK_Q4_0_SIZE), dtype=torch.uint8, device=device)
        blocks[:, :, 1] = 0x3C
        blocks[:, :, 2:] = 0x88       # all-zero weight: d = 1.0, q = 8
        self.register_buffer("weight_blocks", blocks)
        self._weight_dequant: Optional[torch.Tensor] = None
        self._prepacked: Optional[Q4Prepacked] = None
        self._prepacked_key = None
        if bias:
            self.register_buffer("bias", torch.zeros(out_features, dtype=dtype or torch.float32, device=device))
        else:
            self.register_parameter("bias", None)

    def _weights(self) -> Q4Prepacked:
        wb = self.weight_blocks
        key = (wb.data_ptr(), wb._version, wb.device)
        if self._prepacked is None or self._prepacked_key != key:
            self._prepacked = prepack_ggml_q4_0(wb)
            self._prepacked_key = key
        return self._prepacked

    def dequantize(self, dtype: Optional[torch.dtype] = None) -> None:
        """Keep a dense copy (default fp16) and use a plain matmul (quantization.py:519-534)."""
        self._weight_dequant = dequantize_ggml_q4_0(self.weight_blocks, dtype or torch.float16)
        self._dequant_on_load = True

    def keep_quantized(self) -> None:
        """Drop the dense copy; forward uses the fused q4_0 kernels (quantization.py:536-544)."""
        self._weight_dequant = None
        self._dequant_on_load = False

    @classmethod
    def from_float(cls, module: nn.Linear, group_size: int = 128, dequant_on_load: bool = False) -> "Int4Linear":
        """Quantize an ``nn.Linear`` (quantization.py:546-589).  The ``[out, in]`` weight is read
        in place as the transposed ``[in, out]`` matrix; no transposed copy is made."""
        q = cls(module.in_features, module.out_features, group_size=group_size, bias=module.bias is not None,
                device=module.weight.device, dtype=module.weight.dtype, dequant_on_load=dequant_on_load)
        blocks, pre = _quantize_impl(module.weight.data.t(), True, True)
        q.weight_blocks = blocks
        q._prepacked = pre
        q._prepacked_key = (blocks.data_ptr(), blocks._version, blocks.device)
        if module.bias is not None:
            q.bias.copy_(module.bias.data)
        if dequant_on_load:
            q.dequantize()
        return q

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        if self._weight_dequant is not None:
            y = (x2.to(self._weight_dequant.dtype) @ self._weight_dequant).to(x.dtype)
        else:
            y = _matmul_prepacked(x2, self._weights())
        if self.bias is not None:
            y = y + self.bias
        return y.reshape(*lead, self.out_features)

    def extra_repr(self) -> str:
        mode = "fast_fp16" if self._weight_dequant is not None else "int4_kernel"
        return (f"in_features={self.in_features}, out_features={self.out_features}, "
                f"group_size={self.group_size}, bias={self.bias is not None}, mode={mode}")
