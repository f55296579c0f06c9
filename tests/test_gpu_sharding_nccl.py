"""Column-parallel q4_0 layer on real GPUs over NCCL (needs >= 2 GPUs; skipped otherwise).
Each rank quantizes only its column shard; the gathered result must equal the single-GPU result
bit for bit (blocks are per column, so sharding over N changes no arithmetic)."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _worker(rank: int, world: int, port: int, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import metalops_b200 as mo
        g = torch.Generator().manual_seed(11)
        K, N = 1024, 2048
        w = (torch.randn(K, N, generator=g) * 0.02).to(dev)
        ok = True
        for M, dt in ((1, torch.float16), (5, torch.float16), (96, torch.bfloat16)):
            x = torch.randn(M, K, generator=g).to(dt).to(dev)
            layer = mo.ColumnParallelQ4Linear.from_float(w, rank, world)
            y_local = layer(x)
            y_full = layer(x, gather_output=True)
            ref = mo.matmul_ggml_q4_0(x, mo.quantize_ggml_q4_0(w))
            ok &= tuple(y_local.shape) == (M, N // world)
            ok &= bool(torch.equal(y_full, ref))
            ok &= bool(torch.equal(y_local, ref[:, layer.n0:layer.n1]))
        torch.cuda.synchronize()
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_column_parallel_nccl_world2():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, 29650 + os.getpid() % 200, ret), nprocs=world, join=True)
    assert dict(ret) == {0: True, 1: True}
