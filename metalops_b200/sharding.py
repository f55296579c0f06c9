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


class _PeerExchange:
    """Two ``[max_rows, width]`` uint32 buffers in symmetric memory (peer-mapped on every rank) and the
    device-resident call counter of the barrier-free exchange (q4b_gemv_exchange_dev): a decode kernel stores
    (value | epoch << 16) into every rank's buffer and each rank's unpack kernel waits, word by word and
    bounded, for the epoch, clears what it read and bumps the counter.  Calls alternate between the two
    buffers, so with every rank running its calls in stream order nobody can still be reading the buffer
    that a peer overwrites.  The one barrier is at set-up; nothing changes on the host between calls, so a
    call can be captured in a CUDA graph and replayed."""

    def __init__(self, max_rows: int, width: int, device, group=None):
        import ctypes
        import torch.distributed._symmetric_memory as symm_mem
        group = group if group is not None else dist.group.WORLD
        self.max_rows, self.width = max(16, max_rows), width
        self.buf = symm_mem.empty((2, self.max_rows, width), dtype=torch.int32, device=device)
        self.buf.zero_()                                     # no epoch anywhere
        self.ctl = torch.zeros(2, dtype=torch.int32, device=device)
        self.hdl = symm_mem.rendezvous(self.buf, group)
        torch.cuda.synchronize(device)
        self.hdl.barrier()                                   # every rank's buffers are cleared before anyone stores
        self.half_words = self.max_rows * width
        self.ptrs = (ctypes.c_void_p * len(self.hdl.buffer_ptrs))(*[int(p) for p in self.hdl.buffer_ptrs])
        self.local = self.buf.data_ptr()

    def run(self, x: torch.Tensor, pre: "Q.Q4Prepacked", world: int, col0: int, slots: int, out: torch.Tensor) -> None:
        """One exchange: the product of ``x`` with this rank's weight stored at column ``col0`` of every rank's
        buffer, then this rank's unpack into ``out`` (slots == 1: the gathered row; else the sum of the slots)."""
        from . import _cabi
        with torch.cuda.device(x.device):
            rc = _cabi.load().q4b_gemv_exchange_dev(x.data_ptr(), _cabi.DTYPE_CODE[x.dtype], x.shape[0], x.stride(0),
                                                    pre.data.data_ptr(), pre.K, pre.N, self.ptrs, world, col0, self.width,
                                                    self.local, self.half_words, slots, self.ctl.data_ptr(), out.data_ptr(),
                                                    out.stride(0), 0, _cabi.stream_ptr(x.device))
        _cabi.check(rc, "q4b_gemv_exchange_dev")


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
        """Allocate the exchange buffers ``2 x [max_rows, N]`` in symmetric memory (peer-mapped on every
        rank of the group) once.  Needs equal shards (N divisible by the world size) and CUDA."""
        if self.N % self.world:
            raise RuntimeError("fused gather needs N divisible by the number of ranks")
        self._gather = FusedGatherBuffer(self.N, self.rank, self.world, dtype, self.weight_blocks.device, self.group, max_rows)

    def forward_fused_gather(self, x: torch.Tensor) -> torch.Tensor:
        """``[M, N]`` on every rank, M <= 16: each rank's decode kernel writes its columns into all
        ranks' buffers over NVLink as self-validating words; no barrier, no collective."""
        if getattr(self, "_gather", None) is None:
            raise RuntimeError("call enable_fused_gather() first")
        return self._gather.gemv(x, Q.prepack_ggml_q4_0(self.weight_blocks))


class FusedGatherBuffer:
    """The gathered output of a column-parallel decode product without a collective: each rank's decode
    kernel stores its ``[M, N/g]`` columns into every rank's buffer over NVLink (plain peer stores of
    self-validating words, no TMA, no multicast) and a small kernel on each rank waits for them, bounded,
    and writes the plain ``[M, N]`` result.  Takes the weight per call, so one buffer serves many layers
    of the same width."""

    def __init__(self, N: int, rank: int, world: int, dtype: torch.dtype, device, group=None, max_rows: int = 16):
        if N % world:
            raise RuntimeError("fused gather needs N divisible by the number of ranks")
        self.N, self.rank, self.world, self.n0, self.dtype = N, rank, world, rank * (N // world), dtype
        self.ex = _PeerExchange(max_rows, N, device, group)

    def gemv(self, x: torch.Tensor, pre: "Q.Q4Prepacked") -> torch.Tensor:
        from . import _cabi
        M = x.shape[0]
        if M > self.ex.max_rows or M > 16 or x.dtype != self.dtype or pre.N != self.N // self.world:
            raise RuntimeError("fused gather: up to 16 rows of the buffer's dtype, weight shard of N / world columns")
        xc = x.contiguous()
        out = torch.empty((M, self.N), dtype=x.dtype, device=x.device)
        self.ex.run(xc, pre, self.world, self.n0, 1, out)
        return out


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
        """Allocate ``2 x [max_rows, world * N]`` in symmetric memory: slot r of every rank's buffer
        receives rank r's partial product."""
        self._red = _PeerExchange(max_rows, self.world * self.N, self.weight_blocks.device, self.group)
        self._red_dtype = dtype

    def forward_fused_reduce(self, x: torch.Tensor) -> torch.Tensor:
        """``[M, N]`` on every rank, M <= 16: the decode kernel of each rank writes its partial
        product into slot ``rank`` of all ranks' buffers over NVLink (self-validating words, no barrier);
        a small kernel on each rank waits for the ``world`` slots and adds them in rank order, in fp32."""
        from . import _cabi
        if getattr(self, "_red", None) is None:
            raise RuntimeError("call enable_fused_reduce() first")
        xl = self._local_x(x).contiguous()
        M = xl.shape[0]
        if M > self._red.max_rows or M > 16 or xl.dtype != self._red_dtype:
            raise RuntimeError("fused reduce serves up to 16 rows of the dtype it was enabled for")
        pre = Q.prepack_ggml_q4_0(self.weight_blocks)
        out = torch.empty((M, self.N), dtype=xl.dtype, device=xl.device)
        self._red.run(xl, pre, self.world, self.rank * self.N, self.world, out)
        return out
