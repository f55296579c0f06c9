"""Host-side logic of the column-parallel layer, on CPU ranks over gloo (world size 2).
The local product is replaced by the CPU oracle here; only index math and the gather are tested."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import q4_0_oracle as orc


def test_shard_bounds():
    from metalops_b200.sharding import shard_bounds
    assert shard_bounds(28672, 8, 3) == (3 * 3584, 4 * 3584)
    assert shard_bounds(8192, 8, 7) == (7168, 8192)
    assert shard_bounds(4096, 1, 0) == (0, 4096)
    covered = [shard_bounds(11008, 4, r) for r in range(4)]
    assert covered[0][0] == 0 and covered[-1][1] == 11008
    assert all(a[1] == b[0] for a, b in zip(covered, covered[1:]))
    with pytest.raises(ValueError):
        shard_bounds(1000, 3, 0)
    with pytest.raises(ValueError):
        shard_bounds(4096 + 8, 2, 0)       # shards would not be whole 16-column tiles
    with pytest.raises(ValueError):
        shard_bounds(4096, 2, 2)


def _worker(rank: int, world: int, port: int, M: int, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from metalops_b200.sharding import ColumnParallelQ4Linear
        g = torch.Generator().manual_seed(4)
        K, N = 128, 96
        w = torch.randn(K, N, generator=g) * 0.02
        x = torch.randn(M, K, generator=g)
        layer = ColumnParallelQ4Linear.from_float(
            w, rank, world, quantize=orc.quantize_q4_0,
            matmul=lambda xx, blocks: orc.matmul_q4_0_fp32(xx, blocks))
        assert tuple(layer.weight_blocks.shape) == (K // 32, N // world, 18)
        y_local = layer(x)
        assert tuple(y_local.shape) == (M, N // world)
        y_full = layer(x, gather_output=True)
        expect = orc.matmul_q4_0_fp32(x, orc.quantize_q4_0(w))
        # quantization blocks are per column, so sharding over N changes no bit of any block
        ok = torch.equal(y_full, expect) and torch.equal(y_local, expect[:, layer.n0:layer.n1])
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("M", [1, 5])
def test_column_parallel_gather_world2(M):
    world = 2
    port = 29500 + (os.getpid() % 500) + M
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, M, ret), nprocs=world, join=True)
    assert dict(ret) == {0: True, 1: True}


def _row_worker(rank: int, world: int, port: int, M: int, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from metalops_b200.sharding import RowParallelQ4Linear
        g = torch.Generator().manual_seed(5)
        K, N = 256, 48
        w = torch.randn(K, N, generator=g) * 0.02
        x = torch.randn(M, K, generator=g)
        layer = RowParallelQ4Linear.from_float(
            w, rank, world, quantize=orc.quantize_q4_0,
            matmul=lambda xx, blocks: orc.matmul_q4_0_fp32(xx, blocks))
        full_blocks = orc.quantize_q4_0(w)
        # blocks are 32 consecutive k of a column: a k shard's blocks are the full weight's
        ok = torch.equal(layer.weight_blocks, full_blocks[layer.k0 // 32:layer.k1 // 32])
        y = layer(x)                                    # full activations: the layer slices them
        y2 = layer(x[:, layer.k0:layer.k1])             # or this rank's slice
        expect = orc.matmul_q4_0_fp32(x, full_blocks)
        ok = ok and torch.equal(y, y2) and tuple(y.shape) == (M, N)
        ok = ok and bool(((y - expect).norm() / expect.norm()).item() < 1e-5)
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("M", [1, 5])
def test_row_parallel_allreduce_world2(M):
    world = 2
    port = 30100 + (os.getpid() % 500) + M
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_row_worker, args=(world, port, M, ret), nprocs=world, join=True)
    assert dict(ret) == {0: True, 1: True}
