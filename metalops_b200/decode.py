"""Single-row decode through the persistent stage-list kernel (``q4b_gemv_grouped``,
``q4b_chain_*`` of ``include/q4b200.h``).

The reference has nothing like it: ``matmul_ggml_q4_0`` (quantization.py:422-454) is called once
per projection.  Two entry points:

* :func:`matmul_ggml_q4_0_grouped` — several weights that share one input row (q|k|v, gate|up) in
  one launch;
* :class:`DecodeChain` — a whole list of such stages, where a stage may take its input from an
  earlier stage's output, built once and launched as ONE kernel per decode step.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence, Tuple, Union

import torch

from . import _cabi
from .quantization import Q4Prepacked, prepack_ggml_q4_0

ACT_FLAGS = {None: 0, "none": 0, "silu": _cabi.FLAG_ACT_SILU, "gelu": _cabi.FLAG_ACT_GELU}


def _as_prepacked(w: Union[torch.Tensor, Q4Prepacked]) -> Q4Prepacked:
    return w if isinstance(w, Q4Prepacked) else prepack_ggml_q4_0(w)


def _fill_product(dst: _cabi.ChainProduct, pre: Q4Prepacked, y: torch.Tensor, addend: Optional[torch.Tensor],
                  alpha: float, act: Optional[str]) -> None:
    if act not in ACT_FLAGS:
        raise ValueError(f"unknown activation {act!r}")
    if addend is not None:
        if addend.dtype != torch.float32 or addend.numel() != pre.N or not addend.is_contiguous():
            raise RuntimeError("addend must be a contiguous fp32 vector of N elements")
        _cabi.require_device(addend, "addend")
    dst.prepacked = pre.data.data_ptr()
    dst.y = y.data_ptr()
    dst.addend = addend.data_ptr() if addend is not None else None
    dst.N = pre.N
    dst.alpha = float(alpha)
    dst.flags = ACT_FLAGS[act]


def matmul_ggml_q4_0_grouped(x: torch.Tensor, weights: Sequence[Union[torch.Tensor, Q4Prepacked]], *,
                             alphas: Optional[Sequence[float]] = None,
                             addends: Optional[Sequence[Optional[torch.Tensor]]] = None,
                             acts: Optional[Sequence[Optional[str]]] = None, pdl: bool = False) -> List[torch.Tensor]:
    """``[act(alpha_p * (x @ dequant(W_p)) + addend_p) for p]`` for one row ``x [K]`` or ``[1, K]`` and
    up to four q4_0 weights ``[K/32, N_p, 18]`` (or their prepacked form), in one launch."""
    _cabi.require_device(x, "x")
    if x.dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError("x must be fp16 or bf16")
    if x.numel() != x.shape[-1]:
        raise RuntimeError("the grouped decode entry takes a single row")
    pres = [_as_prepacked(w) for w in weights]
    if not 1 <= len(pres) <= _cabi.CHAIN_MAX_PRODUCTS:
        raise ValueError(f"1..{_cabi.CHAIN_MAX_PRODUCTS} weights per call")
    K = x.shape[-1]
    xc = x.contiguous()
    outs = [torch.empty(x.shape[:-1] + (p.N,), dtype=x.dtype, device=x.device) for p in pres]
    arr = (_cabi.ChainProduct * len(pres))()
    for i, (p, y) in enumerate(zip(pres, outs)):
        if p.K != K:
            raise RuntimeError(f"weight {i} has K = {p.K}, x has {K}")
        _fill_product(arr[i], p, y, addends[i] if addends else None, alphas[i] if alphas else 1.0, acts[i] if acts else None)
    with torch.cuda.device(x.device):
        rc = _cabi.load().q4b_gemv_grouped(xc.data_ptr(), _cabi.DTYPE_CODE[x.dtype], K, arr, len(pres),
                                           _cabi.FLAG_PDL if pdl else 0, _cabi.stream_ptr(x.device))
    _cabi.check(rc, "matmul_ggml_q4_0_grouped")
    return outs


class DecodeChain:
    """A list of decode stages launched as one persistent kernel.

    >>> ch = DecodeChain(torch.float16, device)
    >>> s0 = ch.add_stage(x0, [wq, wk, wv])            # input in plain memory
    >>> s1 = ch.add_stage((s0, 2), [wo])               # input = output 2 of stage s0
    >>> s2 = ch.add_stage((s1, 0), [wgate, wup])
    >>> s3 = ch.add_stage(((s2, 0), (s2, 1)), [wdown], xform="silu_mul")   # x = silu(gate) * up
    >>> ch.build(); ch.run(); ch.outputs[s3][0]

    Outputs are allocated by the chain (``outputs[stage][product]``, shape ``[N]``) and overwritten by
    every :meth:`run`.  Runs of one chain must not overlap on the GPU.
    """

    def __init__(self, dtype: torch.dtype, device: torch.device, out_capacity: Optional[int] = None):
        """``out_capacity`` (elements): carve all outputs out of one flat buffer (``out_flat``) of
        that many elements, so that a caller can copy every result to the host in one transfer."""
        if dtype not in (torch.float16, torch.bfloat16):
            raise RuntimeError("chain dtype must be fp16 or bf16")
        self.dtype, self.device = dtype, torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("DecodeChain needs a CUDA device; this build has no CPU path")
        self._stages: List[dict] = []
        self.outputs: List[List[torch.Tensor]] = []
        self._workspace: Optional[torch.Tensor] = None
        self.out_flat = torch.empty(out_capacity, dtype=dtype, device=self.device) if out_capacity else None
        self._out_used = 0

    def add_stage(self, x, weights: Sequence[Union[torch.Tensor, Q4Prepacked]], *, alphas=None, addends=None, acts=None,
                  xform: Optional[str] = None) -> int:
        pres = [_as_prepacked(w) for w in weights]
        if not 1 <= len(pres) <= _cabi.CHAIN_MAX_PRODUCTS:
            raise ValueError(f"1..{_cabi.CHAIN_MAX_PRODUCTS} weights per stage")
        K = pres[0].K
        if any(p.K != K for p in pres):
            raise RuntimeError("the weights of a stage share the input row: same K")
        index = len(self._stages)
        st = {"pres": pres, "K": K, "alphas": alphas, "addends": addends, "acts": acts, "x": None, "src": None, "src2": None,
              "xform": _cabi.CHAIN_X_PLAIN}
        if isinstance(x, torch.Tensor):
            _cabi.require_device(x, "x")
            if x.dtype != self.dtype or x.numel() != K or not x.is_contiguous():
                raise RuntimeError("a stage input is a contiguous row of K elements in the chain's dtype")
            if xform is not None:
                raise ValueError("an input transform needs earlier outputs as operands")
            st["x"] = x
        elif xform == "silu_mul":
            (sa, pa), (sb, pb) = x
            st["src"], st["src2"], st["xform"] = (int(sa), int(pa)), (int(sb), int(pb)), _cabi.CHAIN_X_SILU_MUL
        elif xform is None:
            sa, pa = x
            st["src"] = (int(sa), int(pa))
        else:
            raise ValueError(f"unknown input transform {xform!r}")
        for src in (st["src"], st["src2"]):
            if src is not None:
                if not 0 <= src[0] < index or not 0 <= src[1] < len(self._stages[src[0]]["pres"]):
                    raise ValueError("a stage input must be an output of an earlier stage")
                if self._stages[src[0]]["pres"][src[1]].N != K:
                    raise RuntimeError("the earlier output's length is not this stage's K")
        self._stages.append(st)
        outs = []
        for p in pres:
            if self.out_flat is None:
                outs.append(torch.empty(p.N, dtype=self.dtype, device=self.device))
            else:
                if self._out_used + p.N > self.out_flat.numel():
                    raise RuntimeError("out_capacity is too small for the outputs of the stages added")
                outs.append(self.out_flat[self._out_used:self._out_used + p.N])
                self._out_used += p.N + (-p.N) % 8          # keep every output 16-byte aligned
        self.outputs.append(outs)
        self._workspace = None
        return index

    def _descriptors(self):
        arr = (_cabi.ChainStage * len(self._stages))()
        for i, st in enumerate(self._stages):
            d = arr[i]
            d.x = st["x"].data_ptr() if st["x"] is not None else None
            d.x_stage, d.x_product = st["src"] if st["src"] is not None else (-1, -1)
            d.x_stage2, d.x_product2 = st["src2"] if st["src2"] is not None else (-1, -1)
            d.xform = st["xform"]
            d.n_products = len(st["pres"])
            d.K = st["K"]
            for p, pre in enumerate(st["pres"]):
                _fill_product(d.products[p], pre, self.outputs[i][p], st["addends"][p] if st["addends"] else None,
                              st["alphas"][p] if st["alphas"] else 1.0, st["acts"][p] if st["acts"] else None)
        return arr

    def build(self) -> "DecodeChain":
        if not self._stages:
            raise RuntimeError("empty chain")
        lib = _cabi.load()
        arr = self._descriptors()
        nbytes = lib.q4b_chain_workspace_bytes(arr, len(self._stages))
        if nbytes == 0:
            raise RuntimeError("q4b_chain_workspace_bytes rejected the stage list")
        self._workspace = torch.empty(nbytes + 256, dtype=torch.uint8, device=self.device)
        off = (-self._workspace.data_ptr()) % 256
        self._ws_ptr = self._workspace.data_ptr() + off
        with torch.cuda.device(self.device):
            rc = lib.q4b_chain_build(arr, len(self._stages), self._ws_ptr, nbytes, _cabi.stream_ptr(self.device))
        _cabi.check(rc, "DecodeChain.build")
        self._max_k = max(st["K"] for st in self._stages)
        return self

    def run(self) -> List[List[torch.Tensor]]:
        if self._workspace is None:
            self.build()
        with torch.cuda.device(self.device):
            rc = _cabi.load().q4b_chain_run(self._ws_ptr, len(self._stages), _cabi.DTYPE_CODE[self.dtype], self._max_k, 0,
                                            _cabi.stream_ptr(self.device))
        _cabi.check(rc, "DecodeChain.run")
        return self.outputs

    @property
    def weight_bytes(self) -> int:
        return sum(p.K * p.N // 32 * 18 for st in self._stages for p in st["pres"])
