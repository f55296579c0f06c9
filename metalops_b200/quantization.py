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


def _version_of(t: torch.Tensor):
    """In-place modification counter used as a cache key.  Inference tensors keep no counter
    (reading it raises); they cannot be modified in place outside inference mode, so their
    storage address and shape stand in for it."""
    try:
        return t._version
    except RuntimeError:
        return ("inference", t.data_ptr(), tuple(t.shape))


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


def quantize_ggml_q4_0(weight: torch.Tensor, scale_mode: str = "metalcore") -> torch.Tensor:
    """Quantize ``weight [K, N]`` to GGML block_q4_0: returns uint8 ``[K/32, N, 18]``.

    Bit-identical to the reference (quantization.py:307-371) for fp32, fp16 and bf16 weights.
    Note the reference's docstring says ``[num_blocks, 18]``; its code and this function return
    ``[K/32, N, 18]``.

    ``scale_mode="ggml"`` (not in the reference) uses the scale rule of other GGML tools instead of
    the reference's ``amax / 7``: ``d = (value of largest magnitude) / -8``,
    ``q = clamp(round(w / d) + 8, 0, 15)``, an all-zero block gets ``d = 0, q = 8``."""
    if scale_mode == "metalcore":
        blocks, pre = _quantize_impl(weight, True, True)
    elif scale_mode == "ggml":
        blocks, pre = _quantize_ggml_rule(weight)
    else:
        raise ValueError(f"scale_mode must be 'metalcore' or 'ggml', not {scale_mode!r}")
    blocks._q4b_prepacked = (_version_of(blocks), pre)
    return blocks


def _quantize_ggml_rule(weight: torch.Tensor):
    if weight.dim() != 2:
        raise ValueError("weight must be 2-D [K, N]")
    _cabi.require_device(weight, "weight")
    if weight.dtype not in _cabi.DTYPE_CODE:
        raise RuntimeError(f"unsupported weight dtype {weight.dtype}")
    K, N = weight.shape
    assert K % QK4_0 == 0, f"K ({K}) must be divisible by {QK4_0}"
    if weight.is_contiguous():
        layout, src = _cabi.LAYOUT_KN, weight
    elif weight.t().is_contiguous():
        layout, src = _cabi.LAYOUT_NK, weight.t()
    else:
        layout, src = _cabi.LAYOUT_KN, weight.contiguous()
    blocks = torch.empty((K // QK4_0, N, BLOCK_Q4_0_SIZE), dtype=torch.uint8, device=weight.device)
    pre = _alloc_prepacked(K, N, weight.device)
    with torch.cuda.device(weight.device):
        rc = _cabi.load().q4b_quantize_ggml(src.data_ptr(), _cabi.DTYPE_CODE[src.dtype], K, N, layout, blocks.data_ptr(),
                                            pre.data_ptr(), _cabi.stream_ptr(weight.device))
    _cabi.check(rc, "quantize_ggml_q4_0")
    return blocks, Q4Prepacked(pre, K, N)


def prepack_ggml_q4_0(W_blocks: torch.Tensor) -> Q4Prepacked:
    """Streaming-layout copy of ``W_blocks [K/32, N, 18]`` (cached on the tensor object)."""
    cached = getattr(W_blocks, "_q4b_prepacked", None)
    if cached is not None and cached[0] == _version_of(W_blocks) and cached[1].device == W_blocks.device:
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
        W_blocks._q4b_prepacked = (_version_of(W_blocks), out)
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
                      flags: int = _cabi.FLAG_NONE, kernel: str = "auto",
                      addend: Optional[torch.Tensor] = None) -> torch.Tensor:
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
    fn = {"auto": lib.q4b_matmul_addend, "gemv": lib.q4b_gemv_addend, "gemm": lib.q4b_gemm_addend,
          "gemm_wt": lib.q4b_gemm_wt_addend}[kernel]
    ld_add = 0
    if addend is not None:
        if addend.dtype != torch.float32 or addend.device != x.device:
            raise RuntimeError("addend must be a float32 tensor on X's device")
        if addend.dim() == 1 and addend.numel() == pre.N and addend.is_contiguous():
            ld_add = 0                       # one row added to every row of the result (a bias)
        elif tuple(addend.shape) == (M, pre.N) and addend.stride(1) == 1:
            ld_add = addend.stride(0) if M > 1 else pre.N
        else:
            raise RuntimeError("addend must be [M, N] with unit inner stride, or a contiguous [N] row")
    with torch.cuda.device(x.device):
        rc = fn(x.data_ptr(), _cabi.DTYPE_CODE[x.dtype], M, x.stride(0), pre.data.data_ptr(), pre.K, pre.N,
                addend.data_ptr() if addend is not None else None, ld_add,
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
# Group-wise asymmetric INT4 (quantization.py:26-239 of the reference): weight_packed [K/2, N],
# scales / zeros [ceil(K/group), N], W = (q - zero) * scale.
# ---------------------------------------------------------------------------------------

def quantize_int4(weight: torch.Tensor, group_size: int = 128) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Quantize ``weight [K, N]`` to INT4 with per-group scale and zero point; returns
    ``(weight_packed uint8 [K/2, N], scales [groups, N], zeros [groups, N])``, scales and zeros in
    the weight's dtype.  Bit-identical to the reference's Python loop (quantization.py:26-93)."""
    if weight.dim() != 2:
        raise ValueError("weight must be 2-D [K, N]")
    _cabi.require_device(weight, "weight")
    if weight.dtype not in _cabi.DTYPE_CODE:
        raise RuntimeError(f"unsupported weight dtype {weight.dtype}")
    w = weight.contiguous()
    K, N = w.shape
    if K % 2 or group_size % 2 or group_size <= 0:
        raise RuntimeError("quantize_int4 needs an even K and an even, positive group_size")
    ng = (K + group_size - 1) // group_size
    packed = torch.empty((K // 2, N), dtype=torch.uint8, device=w.device)
    scales = torch.empty((ng, N), dtype=w.dtype, device=w.device)
    zeros = torch.empty((ng, N), dtype=w.dtype, device=w.device)
    with torch.cuda.device(w.device):
        rc = _cabi.load().q4b_int4g_quantize(w.data_ptr(), _cabi.DTYPE_CODE[w.dtype], K, N, group_size,
                                             packed.data_ptr(), scales.data_ptr(), zeros.data_ptr(),
                                             _cabi.stream_ptr(w.device))
    _cabi.check(rc, "quantize_int4")
    return packed, scales, zeros


def _check_int4g(W_packed, scales, zeros, group_size):
    _cabi.require_device(W_packed, "W_packed")
    if W_packed.dtype != torch.uint8 or W_packed.dim() != 2:
        raise RuntimeError("W_packed must be uint8 [K/2, N]")
    K, N = W_packed.shape[0] * 2, W_packed.shape[1]
    ng = (K + group_size - 1) // group_size
    if tuple(scales.shape) != (ng, N) or tuple(zeros.shape) != (ng, N) or scales.dtype != zeros.dtype:
        raise RuntimeError(f"scales and zeros must both be [{ng}, {N}] of one dtype")
    if scales.dtype not in _cabi.DTYPE_CODE:
        raise RuntimeError(f"unsupported scales dtype {scales.dtype}")
    if scales.device != W_packed.device or zeros.device != W_packed.device:
        raise RuntimeError("W_packed, scales and zeros must be on the same device")
    return K, N


def dequantize_int4(W_packed: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor, group_size: int = 128,
                    dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``W[k] = ((q - zero) * scale)`` in fp32, cast to ``dtype`` (default fp16) — quantization.py:96-153."""
    if dtype is None:
        dtype = torch.float16
    K, N = _check_int4g(W_packed, scales, zeros, group_size)
    if dtype not in _cabi.DTYPE_CODE:
        raise RuntimeError(f"unsupported output dtype {dtype}")
    p, s, z = W_packed.contiguous(), scales.contiguous(), zeros.contiguous()
    W = torch.empty((K, N), dtype=dtype, device=p.device)
    with torch.cuda.device(p.device):
        rc = _cabi.load().q4b_int4g_dequantize(p.data_ptr(), s.data_ptr(), z.data_ptr(), _cabi.DTYPE_CODE[s.dtype], K, N,
                                               group_size, W.data_ptr(), _cabi.DTYPE_CODE[dtype], _cabi.stream_ptr(p.device))
    _cabi.check(rc, "dequantize_int4")
    return W


class Int4GPrepacked:
    """A group-wise INT4 weight converted for the matmul kernels: streaming tiles (block scale =
    fp16 of the group scale) plus the fp32 per-group constant ``8*d - zero*scale``."""

    __slots__ = ("tiles", "corr", "group_size", "fold", "fold_ktiles")

    def __init__(self, tiles: Q4Prepacked, corr: torch.Tensor, group_size: int, fold: torch.Tensor, fold_ktiles: int):
        self.tiles, self.corr, self.group_size = tiles, corr, group_size
        # corr as the bf16 operand [N, 64 * fold_ktiles] of the extra k-tiles that carry the zero-point
        # term inside the prefill kernel's contraction (three-way bf16 split, six products)
        self.fold, self.fold_ktiles = fold, fold_ktiles


def prepack_int4(W_packed: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor, group_size: int = 128) -> Int4GPrepacked:
    """One-time conversion of a group-wise INT4 weight (cached on ``W_packed``).  Needs
    ``K % 32 == 0`` and ``group_size % 32 == 0``, and scales inside fp16's range (checked on the
    device; a scale beyond it raises instead of turning into ``inf``)."""
    key = (_version_of(W_packed), scales.data_ptr(), _version_of(scales), zeros.data_ptr(), _version_of(zeros), group_size)
    cached = getattr(W_packed, "_q4b_int4g", None)
    if cached is not None and cached[0] == key:
        return cached[1]
    K, N = _check_int4g(W_packed, scales, zeros, group_size)
    if K % QK4_0 or group_size % QK4_0:
        raise RuntimeError("the fused INT4 matmul needs K and group_size to be multiples of 32")
    p, s, z = W_packed.contiguous(), scales.contiguous(), zeros.contiguous()
    tiles = _alloc_prepacked(K, N, p.device)
    corr = torch.empty(s.shape, dtype=torch.float32, device=p.device)
    with torch.cuda.device(p.device):
        rc = _cabi.load().q4b_int4g_prepack(p.data_ptr(), s.data_ptr(), z.data_ptr(), _cabi.DTYPE_CODE[s.dtype], K, N,
                                            group_size, tiles.data_ptr(), corr.data_ptr(), _cabi.stream_ptr(p.device))
    _cabi.check(rc, "prepack_int4")
    import ctypes
    bad = ctypes.c_int(0)
    with torch.cuda.device(p.device):
        _cabi.check(_cabi.load().q4b_int4g_prepack_status(_cabi.stream_ptr(p.device), ctypes.byref(bad)), "prepack_int4")
    if bad.value:
        raise RuntimeError("prepack_int4: a group scale is outside float16's range (or NaN); the fused INT4 kernels "
                           "store block scales as float16")
    lib = _cabi.load()
    kx = lib.q4b_int4g_fold_ktiles(K, group_size)
    fold = torch.empty((N, 64 * kx), dtype=torch.bfloat16, device=p.device)
    with torch.cuda.device(p.device):
        _cabi.check(lib.q4b_int4g_fold_operand(corr.data_ptr(), K, N, group_size, fold.data_ptr(), _cabi.stream_ptr(p.device)),
                    "prepack_int4")
    out = Int4GPrepacked(Q4Prepacked(tiles, K, N), corr, group_size, fold, kx)
    try:
        W_packed._q4b_int4g = (key, out)
    except AttributeError:
        pass
    return out


_ACT_FLAGS = {None: 0, "none": 0, "silu": _cabi.FLAG_ACT_SILU, "gelu": _cabi.FLAG_ACT_GELU}
_FOLD_MIN_ROWS = 16         # above: the tensor-core kernels with the zero-point term folded into the contraction;
                            # up to it: the decode kernels, which form the term in their epilogue


def _matmul_int4_prepacked(X2: torch.Tensor, pre: Int4GPrepacked, bias: Optional[torch.Tensor] = None,
                           activation: Optional[str] = None) -> torch.Tensor:
    in_dtype = X2.dtype
    x = X2.half() if in_dtype == torch.float32 else X2
    if x.dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError(f"X must be float16, bfloat16 or float32 (got {in_dtype})")
    x = x.contiguous()
    M, K, N = x.shape[0], pre.tiles.K, pre.tiles.N
    assert x.shape[1] == K, f"X K dim ({x.shape[1]}) must match weight K ({K})"
    if M == 0:
        return torch.empty((0, N), dtype=in_dtype, device=x.device)
    lib = _cabi.load()
    b32 = None
    if bias is not None:
        b32 = bias.to(device=x.device, dtype=torch.float32).contiguous()
    # the same split between the decode and the tensor-core kernels as q4b_matmul makes
    if M > _FOLD_MIN_ROWS or (M > 8 and K * N >= (1 << 25)):
        # tensor-core kernels: the zero-point term rides in the contraction as extra k-tiles, no [M, N] addend
        rows = torch.empty((M, 64 * pre.fold_ktiles), dtype=torch.bfloat16, device=x.device)
        y = torch.empty((M, N), dtype=x.dtype, device=x.device)
        with torch.cuda.device(x.device):
            sp = _cabi.stream_ptr(x.device)
            rc = lib.q4b_int4g_fold_rows(x.data_ptr(), _cabi.DTYPE_CODE[x.dtype], M, x.stride(0), K, pre.group_size, rows.data_ptr(), sp)
            _cabi.check(rc, "matmul_int4")
            rc = lib.q4b_int4g_gemm_fold(x.data_ptr(), _cabi.DTYPE_CODE[x.dtype], M, x.stride(0), pre.tiles.data.data_ptr(), K, N,
                                         pre.fold.data_ptr(), rows.data_ptr(), pre.fold_ktiles,
                                         b32.data_ptr() if b32 is not None else None, y.data_ptr(), y.stride(0),
                                         _ACT_FLAGS[activation], sp)
        _cabi.check(rc, "matmul_int4")
        return y.float() if in_dtype == torch.float32 else y
    # decode kernels (up to 16 rows): the rows' group sums, then the product with the term formed in its epilogue
    rowsums = torch.empty(lib.q4b_int4g_rowsums_bytes(M, K, pre.group_size) // 4, dtype=torch.float32, device=x.device)
    y = torch.empty((M, N), dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        sp = _cabi.stream_ptr(x.device)
        rc = lib.q4b_int4g_rowsums(x.data_ptr(), _cabi.DTYPE_CODE[x.dtype], M, x.stride(0), K, pre.group_size, rowsums.data_ptr(), sp)
        _cabi.check(rc, "matmul_int4")
        rc = lib.q4b_int4g_gemv(x.data_ptr(), _cabi.DTYPE_CODE[x.dtype], M, x.stride(0), pre.tiles.data.data_ptr(), K, N,
                                pre.corr.data_ptr(), rowsums.data_ptr(), pre.group_size,
                                b32.data_ptr() if b32 is not None else None, y.data_ptr(), y.stride(0), _ACT_FLAGS[activation], sp)
    _cabi.check(rc, "matmul_int4")
    return y.float() if in_dtype == torch.float32 else y


def _matmul_int4_via_addend(x: torch.Tensor, pre: Int4GPrepacked, bias: Optional[torch.Tensor] = None,
                            activation: Optional[str] = None) -> torch.Tensor:
    """The same product with the zero-point term as an explicit fp32 ``[M, N]`` addend
    (``q4b_int4g_addend`` + ``q4b_matmul_addend``): the form every kernel accepts, kept for comparison."""
    M, K, N = x.shape[0], pre.tiles.K, pre.tiles.N
    lib = _cabi.load()
    addend = torch.empty((M, N), dtype=torch.float32, device=x.device)
    rowsums = torch.empty(lib.q4b_int4g_rowsums_bytes(M, K, pre.group_size) // 4, dtype=torch.float32, device=x.device)
    b32 = bias.to(device=x.device, dtype=torch.float32).contiguous() if bias is not None else None
    with torch.cuda.device(x.device):
        rc = lib.q4b_int4g_addend(x.data_ptr(), _cabi.DTYPE_CODE[x.dtype], M, x.stride(0), pre.corr.data_ptr(),
                                  b32.data_ptr() if b32 is not None else None, K, N, pre.group_size,
                                  rowsums.data_ptr(), addend.data_ptr(), _cabi.stream_ptr(x.device))
    _cabi.check(rc, "matmul_int4")
    return _matmul_prepacked(x, pre.tiles, addend=addend, flags=_ACT_FLAGS[activation])


def matmul_int4(X: torch.Tensor, W_packed: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor,
                group_size: int = 128, activation: Optional[str] = None) -> torch.Tensor:
    """``Y = X @ ((q - zero) * scale)`` for ``X [M, K]`` or ``[B, M, K]`` — quantization.py:156-239.

    Runs the fused kernels (decode GEMV for M <= 16, tcgen05 GEMM above) on a one-time
    conversion of the weight; the zero-point term enters as an fp32 addend before the single
    rounding.  Output dtype = ``X.dtype``."""
    _cabi.require_device(X, "X")
    batched = X.dim() == 3
    X2 = X.reshape(-1, X.shape[-1]) if batched else X
    if X2.dim() != 2:
        raise RuntimeError("X must be [M, K] or [B, M, K]")
    K = W_packed.shape[0] * 2
    if K % QK4_0 or group_size % QK4_0:
        Y = _matmul_int4_generic(X2, W_packed, scales, zeros, group_size, activation)
    else:
        Y = _matmul_int4_prepacked(X2, prepack_int4(W_packed, scales, zeros, group_size), activation=activation)
    return Y.view(X.shape[0], X.shape[1], -1) if batched else Y


def _matmul_int4_generic(X2: torch.Tensor, W_packed, scales, zeros, group_size: int, activation: Optional[str]) -> torch.Tensor:
    """Shapes the streaming tiles do not cover (K or group_size not a multiple of 32), which the
    reference's Python loop accepts (quantization.py:207-239): a CUDA-core kernel straight from the
    ``[K/2, N]`` format, fp32 accumulation.  The activation, if any, is applied afterwards."""
    K, N = _check_int4g(W_packed, scales, zeros, group_size)
    in_dtype = X2.dtype
    x = (X2.half() if in_dtype == torch.float32 else X2).contiguous()
    if x.dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError(f"X must be float16, bfloat16 or float32 (got {in_dtype})")
    assert x.shape[1] == K, f"X K dim ({x.shape[1]}) must match weight K ({K})"
    M = x.shape[0]
    y = torch.empty((M, N), dtype=x.dtype, device=x.device)
    if M:
        p, s, z = W_packed.contiguous(), scales.contiguous(), zeros.contiguous()
        with torch.cuda.device(x.device):
            rc = _cabi.load().q4b_int4g_matmul_generic(x.data_ptr(), _cabi.DTYPE_CODE[x.dtype], M, x.stride(0), p.data_ptr(),
                                                       s.data_ptr(), z.data_ptr(), _cabi.DTYPE_CODE[s.dtype], K, N, group_size,
                                                       y.data_ptr(), y.stride(0), _cabi.stream_ptr(x.device))
        _cabi.check(rc, "matmul_int4")
    if activation == "silu":
        y = torch.nn.functional.silu(y.float()).to(y.dtype)
    elif activation == "gelu":
        y = torch.nn.functional.gelu(y.float(), approximate="tanh").to(y.dtype)
    return y.float() if in_dtype == torch.float32 else y


def matmul_int4_silu(X, W_packed, scales, zeros, group_size: int = 128) -> torch.Tensor:
    """``silu(X @ dequant(W))`` with the activation fused into the matmul's epilogue (applied to the
    fp32 sum, one rounding) — the backend entry ``matmul_int4_silu`` of the reference
    (core_mps.mm:5784-5850, kernel quant_kernels.metal:880-1010)."""
    return matmul_int4(X, W_packed, scales, zeros, group_size, activation="silu")


def matmul_int4_gelu(X, W_packed, scales, zeros, group_size: int = 128) -> torch.Tensor:
    """``gelu(X @ dequant(W))``, tanh form, fused like :func:`matmul_int4_silu` — the reference's
    ``matmul_int4_gelu`` (core_mps.mm:5853-5914, kernel quant_kernels.metal:1015-1144)."""
    return matmul_int4(X, W_packed, scales, zeros, group_size, activation="gelu")


def rmsnorm(X: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """``X * rsqrt(mean(X^2, -1) + eps) * weight`` for fp16/bf16 ``X [M, K]``, sums in fp32, one
    rounding to ``X.dtype`` — the RMSNorm step of the reference's ``fused_rmsnorm_linear_int4``
    (training_kernels.metal:425-485)."""
    _cabi.require_device(X, "X")
    if X.dim() != 2 or X.dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError("X must be a float16 or bfloat16 [M, K] tensor")
    x = X if X.stride(1) == 1 else X.contiguous()
    w = weight.to(device=x.device, dtype=x.dtype).contiguous()
    if w.numel() != x.shape[1]:
        raise RuntimeError(f"weight has {w.numel()} elements, X has K = {x.shape[1]}")
    y = torch.empty((x.shape[0], x.shape[1]), dtype=x.dtype, device=x.device)
    if x.shape[0] == 0:
        return y
    with torch.cuda.device(x.device):
        rc = _cabi.load().q4b_rmsnorm(x.data_ptr(), _cabi.DTYPE_CODE[x.dtype], x.shape[0], x.shape[1], x.stride(0),
                                      w.data_ptr(), float(eps), y.data_ptr(), y.stride(0), _cabi.stream_ptr(x.device))
    _cabi.check(rc, "rmsnorm")
    return y


def fused_rmsnorm_linear_int4(X: torch.Tensor, W_norm: torch.Tensor, W_packed: torch.Tensor, scales: torch.Tensor,
                              zeros: torch.Tensor, eps: float, group_size: int) -> torch.Tensor:
    """RMSNorm followed by the group-wise INT4 linear layer, the reference's backend entry of the same
    name and argument order (core_mps.mm:3017-3103): like there, two kernels back to back on one
    stream with the normalised activations rounded to ``X.dtype`` in between."""
    return matmul_int4(rmsnorm(X, W_norm, eps), W_packed, scales, zeros, group_size)


def matmul_int8(X: torch.Tensor, W_packed: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor,
                group_size: int = 128) -> torch.Tensor:
    """``Y = X @ ((W_packed - zero) * scale)`` for int8 ``W_packed [K, N]`` and per-group
    ``scales`` / ``zeros [ceil(K/group_size), N]`` — quantization.py:242-286 (its Metal kernel:
    quant_kernels.metal:40-109).  fp32 accumulation, one rounding to ``X.dtype``; fp32 ``X`` is
    computed through fp16 like the other entry points."""
    _cabi.require_device(X, "X")
    _cabi.require_device(W_packed, "W_packed")
    if X.dim() != 2 or W_packed.dim() != 2 or W_packed.dtype != torch.int8:
        raise RuntimeError("X must be [M, K] and W_packed int8 [K, N]")
    K, N = W_packed.shape
    ng = (K + group_size - 1) // group_size
    if X.shape[1] != K or tuple(scales.shape) != (ng, N) or tuple(zeros.shape) != (ng, N) or scales.dtype != zeros.dtype:
        raise RuntimeError(f"shapes: X [M, {K}], scales and zeros [{ng}, {N}] of one dtype")
    if scales.dtype not in _cabi.DTYPE_CODE:
        raise RuntimeError(f"unsupported scales dtype {scales.dtype}")
    in_dtype = X.dtype
    x = X.half() if in_dtype == torch.float32 else X
    if x.dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError(f"X must be float16, bfloat16 or float32 (got {in_dtype})")
    x, w, s, z = x.contiguous(), W_packed.contiguous(), scales.contiguous(), zeros.contiguous()
    M = x.shape[0]
    y = torch.empty((M, N), dtype=x.dtype, device=x.device)
    if M == 0:
        return y.to(in_dtype)
    with torch.cuda.device(x.device):
        rc = _cabi.load().q4b_int8g_matmul(x.data_ptr(), _cabi.DTYPE_CODE[x.dtype], M, x.stride(0), w.data_ptr(), s.data_ptr(),
                                           z.data_ptr(), _cabi.DTYPE_CODE[s.dtype], K, N, group_size, y.data_ptr(), y.stride(0),
                                           _cabi.stream_ptr(x.device))
    _cabi.check(rc, "matmul_int8")
    return y.float() if in_dtype == torch.float32 else y


def import_ggml_q4_0(raw: torch.Tensor) -> torch.Tensor:
    """block_q4_0 data as other GGML tools store it — uint8 ``[N, K/32, 18]``, rows of blocks per
    output feature, byte j of a block = value j | value (j + 16) << 4 — converted to this package's
    ``[K/32, N, 18]`` (interleaved nibbles), ready for :func:`matmul_ggml_q4_0`."""
    _cabi.require_device(raw, "raw")
    if raw.dtype != torch.uint8 or raw.dim() != 3 or raw.shape[2] != BLOCK_Q4_0_SIZE:
        raise RuntimeError("raw must be uint8 [N, K/32, 18]")
    r = raw.contiguous()
    N, nb = r.shape[0], r.shape[1]
    blocks = torch.empty((nb, N, BLOCK_Q4_0_SIZE), dtype=torch.uint8, device=r.device)
    with torch.cuda.device(r.device):
        rc = _cabi.load().q4b_import_ggml(r.data_ptr(), nb * QK4_0, N, blocks.data_ptr(), _cabi.stream_ptr(r.device))
    _cabi.check(rc, "import_ggml_q4_0")
    return blocks


class Int4Linear(nn.Module):
    """INT4 quantized linear layer with the reference's constructor, buffers, methods and
    ``extra_repr`` (quantization.py:457-612): ``weight_packed [in/2, out]``, ``scales`` /
    ``zeros [groups, out]`` and ``bias`` are the serialised state, so checkpoints interchange.

    The fused kernels on the packed weight are the default here (the reference's ``int4_kernel``
    mode, bias included as an fp32 term before the output rounding): ``dequant_on_load`` is accepted
    for signature compatibility, but a dense fp16 copy (the reference's "hybrid" mode, four times the
    memory and a library GEMM) is made only by an explicit :meth:`dequantize` call."""

    def __init__(self, in_features: int, out_features: int, group_size: int = 128, bias: bool = True,
                 device: Optional[torch.device] = None, dtype: Optional[torch.dtype] = None,
                 dequant_on_load: bool = True):
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.group_size = group_size
        self._dequant_on_load = dequant_on_load
        self.register_buffer("weight_packed", torch.zeros((in_features // 2, out_features), dtype=torch.uint8, device=device))
        num_groups = (in_features + group_size - 1) // group_size
        self.register_buffer("scales", torch.ones((num_groups, out_features), dtype=dtype or torch.float32, device=device))
        self.register_buffer("zeros", torch.zeros((num_groups, out_features), dtype=dtype or torch.float32, device=device))
        self._weight_dequant: Optional[torch.Tensor] = None
        if bias:
            self.register_buffer("bias", torch.zeros(out_features, dtype=dtype or torch.float32, device=device))
        else:
            self.register_parameter("bias", None)

    def dequantize(self, dtype: Optional[torch.dtype] = None) -> None:
        """Keep a dense copy (default fp16) for a plain matmul; not serialised (quantization.py:519-534)."""
        self._weight_dequant = dequantize_int4(self.weight_packed, self.scales, self.zeros, self.group_size,
                                               dtype or torch.float16)
        self._dequant_on_load = True

    def keep_quantized(self) -> None:
        """Drop the dense copy and use the fused INT4 kernels (quantization.py:536-544)."""
        self._weight_dequant = None
        self._dequant_on_load = False

    @classmethod
    def from_float(cls, module: nn.Linear, group_size: int = 128, dequant_on_load: bool = True) -> "Int4Linear":
        """Quantize an ``nn.Linear`` (quantization.py:546-589)."""
        q = cls(module.in_features, module.out_features, group_size=group_size, bias=module.bias is not None,
                device=module.weight.device, dtype=module.weight.dtype, dequant_on_load=dequant_on_load)
        packed, scales, zeros = quantize_int4(module.weight.data.T.contiguous(), group_size)
        q.weight_packed.copy_(packed)
        q.scales.copy_(scales)
        q.zeros.copy_(zeros)
        if module.bias is not None:
            q.bias.copy_(module.bias.data)
        return q

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self._weight_dequant is not None:
            x_half = x.half() if x.dtype != torch.float16 else x
            y = (x_half @ self._weight_dequant).to(x.dtype)
            return y + self.bias if self.bias is not None else y
        lead = x.shape[:-1]
        if self.in_features % QK4_0 or self.group_size % QK4_0:
            y = _matmul_int4_generic(x.reshape(-1, x.shape[-1]), self.weight_packed, self.scales, self.zeros, self.group_size, None)
            if self.bias is not None:
                y = y + self.bias
            return y.reshape(*lead, self.out_features)
        pre = prepack_int4(self.weight_packed, self.scales, self.zeros, self.group_size)
        y = _matmul_int4_prepacked(x.reshape(-1, x.shape[-1]), pre, bias=self.bias)
        if self.bias is not None and self.bias.dtype != y.dtype:
            y = y.to(torch.promote_types(y.dtype, self.bias.dtype))     # the reference's `y + bias` promotes
        return y.reshape(*lead, self.out_features)

    def extra_repr(self) -> str:
        mode = "fast_fp16" if self._weight_dequant is not None else "int4_kernel"
        return (f"in_features={self.in_features}, out_features={self.out_features}, "
                f"group_size={self.group_size}, bias={self.bias is not None}, mode={mode}")


class Q4Linear(nn.Module):
    """Linear layer stored as GGML block_q4_0 (``weight_blocks`` uint8 ``[in/32, out, 18]`` + ``bias``),
    always computed by the fused q4_0 kernels.  Not in the reference (its ``Int4Linear`` uses the
    group-wise format above); this is the module form of ``matmul_ggml_q4_0``."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True,
                 device: Optional[torch.device] = None, dtype: Optional[torch.dtype] = None):
        super().__init__()
        if in_features % QK4_0:
            raise AssertionError(f"in_features ({in_features}) must be divisible by {QK4_0}")
        self.in_features, self.out_features = in_features, out_features
        blocks = torch.zeros((in_features // QK4_0, out_features, BLOCK_Q4_0_SIZE), dtype=torch.uint8, device=device)
        blocks[:, :, 1] = 0x3C
        blocks[:, :, 2:] = 0x88       # all-zero weight: d = 1.0, q = 8
        self.register_buffer("weight_blocks", blocks)
        if bias:
            self.register_buffer("bias", torch.zeros(out_features, dtype=dtype or torch.float32, device=device))
        else:
            self.register_parameter("bias", None)

    @classmethod
    def from_float(cls, module: nn.Linear) -> "Q4Linear":
        """The ``[out, in]`` weight is read in place as the transposed ``[in, out]`` matrix."""
        q = cls(module.in_features, module.out_features, bias=module.bias is not None,
                device=module.weight.device, dtype=module.weight.dtype)
        q.weight_blocks = quantize_ggml_q4_0(module.weight.data.t())
        if module.bias is not None:
            q.bias.copy_(module.bias.data)
        return q

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        addend = None
        if self.bias is not None and x2.shape[0] > 0:
            addend = self.bias.float().contiguous()           # one row, broadcast by the kernels' epilogues
        y = _matmul_prepacked(x2, prepack_ggml_q4_0(self.weight_blocks), addend=addend)
        return y.reshape(*lead, self.out_features)

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}, format=q4_0"
