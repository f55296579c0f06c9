"""Column-parallel (and row-parallel) sharding of a q4_0 linear layer over the GPUs of one node.

The reference is single-device; this is the multi-GPU form its q4_0 matmul takes here.  Every
(k-block, n) quantization block is independent, so rank r of g owns the output columns
``[r*N/g, (r+1)*N/g)``: it quantizes and keeps only that slice of the weight, X is replicated,
and each rank computes ``Y_r [M, N/g]`` with no communication.  Only when the caller asks for
the full ``[M, N]`` is there an exchange: one NCCL all-gather of the column shards over NVLink.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from . import quantization as Q


def shard_bounds(N: int, world: int, rank: int, multiple: int = 16) -> Tuple[int, int]:
    """Columns ``[n0, n1)`` owned by ``rank``.  N must split evenly into slices that are a
    multiple of ``multiple`` columns (16 = one streaming tile), so every rank runs the same
    shapes and the all-gather needs no padding."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"bad rank/world {rank}/{world}")
    if N % world or (N // world) % multiple:
        raise ValueError(f"N={N} does not split into {world} column shards of a multiple of {multiple}")
    per = N // world
    return rank * per, (rank + 1) * per


def gather_columns(y_local: torch.Tensor, group=None, world: Optional[int] = None) -> torch.Tensor:
    """All-gather column shards ``[M, N/g]`` into ``[M, N]`` (rank-major column order).

    For M == 1 the gathered buffer already is ``[1, N]``; for M > 1 the collective lands as
    ``[g, M, N/g]`` and is permuted locally."""
    world = world if world is not None else dist.get_world_size(group)
    if world == 1:
        return y_local
    M, n_local = y_local.shape
    buf = torch.empty((world * M, n_local), dtype=y_local.dtype, device=y_local.device)   # rank-major rows
    dist.all_gather_into_tensor(buf, y_local.contiguous(), group=group)
    if M == 1:
        return buf.view(1, world * n_local)
    return buf.view(world, M, n_local).permute(1, 0, 2).reshape(M, world * n_local)


class ColumnParallelQ4Linear(nn.Module):
    """One rank's slice of a q4_0 linear layer, column-parallel over N.

    ``from_float`` takes the FULL floating-point weight ``[K, N]`` (or an ``nn.Linear``), keeps
    and quantizes only this rank's columns.  ``forward(x, gather_output=False)`` returns the
    local ``[M, N/g]`` slice; with ``gather_output=True`` the full ``[M, N]``.

    ``matmul`` is the local product; it defaults to the CUDA path and exists as a parameter so
    the host-side sharding logic can be exercised on CPU ranks in tests.
    """

    def __init__(self, K: int, N: int, rank: int, world: int, group=None,
                 matmul: Optional[Callable[[torch.Tensor, torch.Tensor], torch.Tensor]] = None):
        super().__init__()
        self.K, self.N, self.rank, self.world, self.group = K, N, rank, world, group
        self.n0, self.n1 = shard_bounds(N, world, rank)
        self._matmul = matmul or Q.matmul_ggml_q4_0
        self.register_buffer("weight_blocks", torch.zeros((K // Q.QK4_0, self.n1 - self.n0, Q.BLOCK_Q4_0_SIZE),
                                                          dtype=torch.uint8))

    @classmethod
    def from_float(cls, weight_kn: torch.Tensor, rank: int, world: int, group=None, matmul=None,
                   quantize: Optional[Callable[[torch.Tensor], torch.Tensor]] = None) -> "ColumnParallelQ4Linear":
        K, N = weight_kn.shape
        mod = cls(K, N, rank, world, group=group, matmul=matmul)
        shard = weight_kn[:, mod.n0:mod.n1].contiguous()
        mod.weight_blocks = (quantize or Q.quantize_ggml_q4_0)(shard)
        return mod

    def forward(self, x: torch.Tensor, gather_output: bool = False) -> torch.Tensor:
        y = self._matmul(x, self.weight_blocks)
        return gather_columns(y, self.group, self.world) if gather_output else y

    # ---- fused all-gather for decode (M <= 16): the kernel's epilogue stores into every rank's output ----
    def enable_fused_gather(self, max_rows: int = 16, dtype: torch.dtype = torch.float16) -> None:
        """Allocate the gathered output ``[max_rows, N]`` in symmetric memory (peer-mapped on every
        rank of the group) once.  Needs equal shards (N divisible by the world size) and CUDA."""
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        if self.N % self.world:
            raise RuntimeError("fused gather needs N divisible by the number of ranks")
        dev = self.weight_blocks.device
        group = self.group if self.group is not None else dist.group.WORLD
        self._gather_buf = symm_mem.empty((max_rows, self.N), dtype=dtype, device=dev)
        self._gather_hdl = symm_mem.rendezvous(self._gather_buf, group)
        self._gather_ptrs = [int(p) for p in self._gather_hdl.buffer_ptrs]

    def forward_fused_gather(self, x: torch.Tensor) -> torch.Tensor:
        """``[M, N]`` on every rank, M <= 16: each rank's decode kernel writes its columns into all
        ranks' outputs over NVLink; a symmetric-memory barrier on the stream orders the reads.  The
        returned tensor is a view of the shared buffer, valid until the next call."""
        import ctypes
        from . import _cabi
        if getattr(self, "_gather_hdl", None) is None:
            raise RuntimeError("call enable_fused_gather() first")
        M = x.shape[0]
        if M > self._gather_buf.shape[0] or M > 16 or x.dtype != self._gather_buf.dtype:
            raise RuntimeError("fused gather serves up to 16 rows of the dtype it was enabled for")
        pre = Q.prepack_ggml_q4_0(self.weight_blocks)
        xc = x.contiguous()
        self._gather_hdl.barrier()                      # nobody still reads the previous result
        ptrs = (ctypes.c_void_p * self.world)(*self._gather_ptrs)
        with torch.cuda.device(xc.device):
            rc = _cabi.load().q4b_gemv_gather(xc.data_ptr(), _cabi.DTYPE_CODE[xc.dtype], M, xc.stride(0), pre.data.data_ptr(),
                                              pre.K, pre.N, ptrs, self.world, self.n0, self.N, 0, _cabi.stream_ptr(xc.device))
        _cabi.check(rc, "q4b_gemv_gather")
        self._gather_hdl.barrier()                      # every rank's stores have landed
        return self._gather_buf[:M]


class FusedGatherBuffer:
    """The gathered output ``[max_rows, N]`` of a column-parallel decode product in symmetric memory
    (peer-mapped on every rank), and the launch that fills it: each rank's decode kernel stores its
    ``[M, N/g]`` columns into every rank's buffer over NVLink (plain peer stores), with a
    symmetric-memory barrier on the stream before (nobody still reads the previous result) and after
    (every rank's stores have landed).  Takes the weight per call, so one buffer serves many layers
    of the same width."""

    def __init__(self, N: int, rank: int, world: int, dtype: torch.dtype, device, group=None, max_rows: int = 16):
        import torch.distributed._symmetric_memory as symm_mem
        if N % world:
            raise RuntimeError("fused gather needs N divisible by the number of ranks")
        self.N, self.rank, self.world, self.n0 = N, rank, world, rank * (N // world)
        group = group if group is not None else dist.group.WORLD
        self.buf = symm_mem.empty((max_rows, N), dtype=dtype, device=device)
        self.hdl = symm_mem.rendezvous(self.buf, group)
        self.ptrs = [int(p) for p in self.hdl.buffer_ptrs]

    def gemv(self, x: torch.Tensor, pre: "Q.Q4Prepacked") -> torch.Tensor:
        import ctypes
        from . import _cabi
        M = x.shape[0]
        if M > self.buf.shape[0] or M > 16 or x.dtype != self.buf.dtype or pre.N != self.N // self.world:
            raise RuntimeError("fused gather: up to 16 rows of the buffer's dtype, weight shard of N / world columns")
        xc = x.contiguous()
        self.hdl.barrier()
        ptrs = (ctypes.c_void_p * self.world)(*self.ptrs)
        with torch.cuda.device(xc.device):
            rc = _cabi.load().q4b_gemv_gather(xc.data_ptr(), _cabi.DTYPE_CODE[xc.dtype], M, xc.stride(0), pre.data.data_ptr(),
                                              pre.K, pre.N, ptrs, self.world, self.n0, self.N, 0, _cabi.stream_ptr(xc.device))
        _cabi.check(rc, "q4b_gemv_gather")
        self.hdl.barrier()
        return self.buf[:M]


class RowParallelQ4Linear(nn.Module):
    """One rank's slice of a q4_0 linear layer, row-parallel over K (the down-projection that
    follows a column-parallel gate/up pair, whose sharded output it consumes as is).

    Quantization blocks are 32 consecutive k of one column, so rank r of g owns the k range
    ``[r*K/g, (r+1)*K/g)`` (a multiple of 64, one streaming tile) and the bits of its blocks are
    those of the full weight.  ``forward(x)`` takes either the full ``[M, K]`` activations or this
    rank's ``[M, K/g]`` slice, computes the partial product and sums the partials over the ranks:
    one NCCL all-reduce (in fp32), or for decode (M <= 16) the fused form in which every rank's
    kernel stores its partial into a slot of every rank's buffer and the sum is local.
    """

    def __init__(self, K: int, N: int, rank: int, world: int, group=None,
                 matmul: Optional[Callable[[torch.Tensor, torch.Tensor], torch.Tensor]] = None):
        super().__init__()
        self.K, self.N, self.rank, self.world, self.group = K, N, rank, world, group
        self.k0, self.k1 = shard_bounds(K, world, rank, multiple=64)
        self._matmul = matmul or Q.matmul_ggml_q4_0
        self.register_buffer("weight_blocks", torch.zeros(((self.k1 - self.k0) // Q.QK4_0, N, Q.BLOCK_Q4_0_SIZE),
                                                          dtype=torch.uint8))

    @classmethod
    def from_float(cls, weight_kn: torch.Tensor, rank: int, world: int, group=None, matmul=None,
                   quantize: Optional[Callable[[torch.Tensor], torch.Tensor]] = None) -> "RowParallelQ4Linear":
        K, N = weight_kn.shape
        mod = cls(K, N, rank, world, group=group, matmul=matmul)
        mod.weight_blocks = (quantize or Q.quantize_ggml_q4_0)(weight_kn[mod.k0:mod.k1].contiguous())
        return mod

    def _local_x(self, x: torch.Tensor) -> torch.Tensor:
        if x.shape[1] == self.K:
            return x[:, self.k0:self.k1]
        if x.shape[1] != self.k1 - self.k0:
            raise RuntimeError(f"x has {x.shape[1]} columns; expected {self.K} or this rank's {self.k1 - self.k0}")
        return x

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        part = self._matmul(self._local_x(x).contiguous(), self.weight_blocks)
        if self.world == 1:
            return part
        acc = part.float()
        dist.all_reduce(acc, group=self.group)
        return acc.to(part.dtype)

    # ---- fused reduction for decode (M <= 16) ----
    def enable_fused_reduce(self, max_rows: int = 16, dtype: torch.dtype = torch.float16) -> None:
        """Allocate ``[max_rows, world * N]`` in symmetric memory: slot r of every rank's buffer
        receives rank r's partial product."""
        import torch.distributed._symmetric_memory as symm_mem
        dev = self.weight_blocks.device
        group = self.group if self.group is not None else dist.group.WORLD
        self._red_buf = symm_mem.empty((max_rows, self.world * self.N), dtype=dtype, device=dev)
        self._red_hdl = symm_mem.rendezvous(self._red_buf, group)
        self._red_ptrs = [int(p) for p in self._red_hdl.buffer_ptrs]

    def forward_fused_reduce(self, x: torch.Tensor) -> torch.Tensor:
        """``[M, N]`` on every rank, M <= 16: the decode kernel of each rank writes its partial
        product into slot ``rank`` of all ranks' buffers over NVLink (q4b_gemv_gather); after a
        symmetric-memory barrier every rank adds the slots in rank order, in fp32."""
        import ctypes
        from . import _cabi
        if getattr(self, "_red_hdl", None) is None:
            raise RuntimeError("call enable_fused_reduce() first")
        xl = self._local_x(x).contiguous()
        M = xl.shape[0]
        if M > self._red_buf.shape[0] or M > 16 or xl.dtype != self._red_buf.dtype:
            raise RuntimeError("fused reduce serves up to 16 rows of the dtype it was enabled for")
        pre = Q.prepack_ggml_q4_0(self.weight_blocks)
        self._red_hdl.barrier()                         # nobody still reads the previous partials
        ptrs = (ctypes.c_void_p * self.world)(*self._red_ptrs)
        with torch.cuda.device(xl.device):
            rc = _cabi.load().q4b_gemv_gather(xl.data_ptr(), _cabi.DTYPE_CODE[xl.dtype], M, xl.stride(0), pre.data.data_ptr(),
                                              pre.K, pre.N, ptrs, self.world, self.rank * self.N, self.world * self.N, 0,
                                              _cabi.stream_ptr(xl.device))
        _cabi.check(rc, "q4b_gemv_gather")
        self._red_hdl.barrier()                         # every rank's partial has landed
        return self._red_buf[:M].view(M, self.world, self.N).float().sum(dim=1).to(xl.dtype)
