"""Column-parallel q4_0 layer on real GPUs over NCCL (2, 4 and 8 ranks; skipped where the box has fewer GPUs).
Each rank quantizes only its column shard (blocks are per column, so sharding over N changes no
packed bit); the gathered result must equal each rank's local slice bit for bit and the single-GPU
product within rounding (the launch plan, hence the order of the k-split sums, may depend on N).
The fused all-gather (decode kernels storing into every rank's output over NVLink) must equal the
NCCL gather bit for bit."""
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
            ref = mo.matmul_ggml_q4_0(x, mo.quantize_ggml_q4_0(w)).float()
            ok &= tuple(y_local.shape) == (M, N // world)
            ok &= bool(torch.equal(y_full[:, layer.n0:layer.n1], y_local))
            ok &= bool(((y_full.float() - ref).norm() / ref.norm()).item() <= 2e-3)
            if M <= 16:
                if M == 1:
                    layer.enable_fused_gather(max_rows=16, dtype=dt)
                    fused_layer = layer
                else:
                    layer._gather = fused_layer._gather          # one pair of exchange buffers serves layers of one width
                for it in range(9):                              # several calls: both buffers, advancing epochs
                    if it == 5:
                        ex = layer._gather.ex                    # the same on every rank: the 16-bit epoch starts over soon
                        c = int(ex.ctl[0].item())                # (keeping the alternation of the two buffers)
                        ex.ctl[0] = 65533 if c & 1 else 65534
                    y_fused = layer.forward_fused_gather(x)
                    ok &= bool(torch.equal(y_fused, y_full))
        # row-parallel (k-sharded) layer: NCCL all-reduce and the fused reduction against one GPU
        K2, N2 = 2048, 1000
        w2 = (torch.randn(K2, N2, generator=g) * 0.02).to(dev)
        row = mo.RowParallelQ4Linear.from_float(w2, rank, world)
        row.enable_fused_reduce(max_rows=16, dtype=torch.float16)
        for M in (1, 7):
            x2 = torch.randn(M, K2, generator=g).half().to(dev)
            ref2 = mo.matmul_ggml_q4_0(x2, mo.quantize_ggml_q4_0(w2)).float()
            for y2 in (row(x2), row.forward_fused_reduce(x2), row.forward_fused_reduce(x2), row.forward_fused_reduce(x2)):
                ok &= tuple(y2.shape) == (M, N2)
                ok &= bool(((y2.float() - ref2).norm() / ref2.norm()).item() <= 2e-3)
        # a captured exchange replays: the call counter lives on the device
        xg = torch.randn(1, K2, generator=g).half().to(dev)
        refg = row(xg)
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            row.forward_fused_reduce(xg)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                yg = row.forward_fused_reduce(xg)
            for _ in range(3):
                graph.replay()
        side.synchronize()
        ok &= bool(((yg.float() - refg.float()).norm() / refg.float().norm()).item() <= 2e-3)
        from metalops_b200 import quantization as Q
        ok &= Q.wait_status(dev) == 0
        torch.cuda.synchronize()
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_column_and_row_parallel_nccl(world):
    if not torch.cuda.is_available() or torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, 29650 + os.getpid() % 200, ret), nprocs=world, join=True)
    assert dict(ret) == {r: True for r in range(world)}


@pytest.mark.parametrize("M,dtype", [(1, torch.float16), (1, torch.bfloat16), (6, torch.float16), (13, torch.bfloat16)])
def test_fused_gather_kernel_on_one_gpu(M, dtype):
    """The gather epilogue itself, with two ranks' shards run as two launches on one GPU: every
    launch stores its columns into BOTH ranks' outputs, which must then equal the local products
    side by side, bit for bit."""
    import ctypes
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import metalops_b200 as mo
    from metalops_b200 import _cabi, quantization as Q
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(77)
    K, N, world = 1056, 2 * 1200, 2
    w = (torch.randn(K, N, generator=g) * 0.02).to(dev)
    x = torch.randn(M, K, generator=g).to(dtype).to(dev)
    outs = [torch.zeros(M, N, dtype=dtype, device=dev) for _ in range(world)]
    ptrs = (ctypes.c_void_p * world)(*[o.data_ptr() for o in outs])
    locals_ = []
    for r in range(world):
        n0, n1 = mo.shard_bounds(N, world, r)
        blocks = mo.quantize_ggml_q4_0(w[:, n0:n1].contiguous())
        pre = mo.prepack_ggml_q4_0(blocks)
        rc = _cabi.load().q4b_gemv_gather(x.data_ptr(), _cabi.DTYPE_CODE[dtype], M, x.stride(0), pre.data.data_ptr(), K, n1 - n0,
                                          ptrs, world, n0, N, 0, _cabi.stream_ptr(dev))
        assert rc == 0
        locals_.append(Q._matmul_prepacked(x, pre, kernel="gemv"))
    torch.cuda.synchronize()
    full = torch.cat(locals_, dim=1)
    for o in outs:
        assert torch.equal(o, full)
    # argument checks
    assert _cabi.load().q4b_gemv_gather(x.data_ptr(), _cabi.DTYPE_CODE[dtype], M, x.stride(0), pre.data.data_ptr(), K, 1200,
                                        ptrs, 9, 0, N, 0, _cabi.stream_ptr(dev)) != 0
    assert _cabi.load().q4b_gemv_gather(x.data_ptr(), _cabi.DTYPE_CODE[dtype], M, x.stride(0), pre.data.data_ptr(), K, 1200,
                                        ptrs, world, 1300, N, 0, _cabi.stream_ptr(dev)) != 0


@pytest.mark.parametrize("M,dtype", [(1, torch.float16), (9, torch.bfloat16)])
def test_barrier_free_gather_on_one_gpu(M, dtype):
    """The self-validating-word form of the gather with two ranks' shards run as launches on one GPU: both
    store (value | epoch) words into both ranks' buffers, the unpack kernel then finds every word of the
    epoch and returns the local products side by side, bit for bit; as partial sums (slots = 2) it adds
    them in fp32.  A buffer that never receives its epoch makes the bounded wait run out: status 700,
    zeros returned, and the next product is fine."""
    import ctypes
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import metalops_b200 as mo
    from metalops_b200 import _cabi, quantization as Q
    lib = _cabi.load()
    dev = torch.device("cuda:0")
    sp = _cabi.stream_ptr(dev)
    g = torch.Generator().manual_seed(78)
    K, N, world = 1056, 2 * 1200, 2
    w = (torch.randn(K, N, generator=g) * 0.02).to(dev)
    x = torch.randn(M, K, generator=g).to(dtype).to(dev)
    code = _cabi.DTYPE_CODE[dtype]
    lls = [torch.zeros(M, N, dtype=torch.int32, device=dev) for _ in range(world)]
    ptrs = (ctypes.c_void_p * world)(*[t.data_ptr() for t in lls])
    for epoch in (1, 2, 65535):
        locals_ = []
        for r in range(world):
            n0, n1 = mo.shard_bounds(N, world, r)
            pre = mo.prepack_ggml_q4_0(mo.quantize_ggml_q4_0(w[:, n0:n1].contiguous()))
            assert lib.q4b_gemv_gather_ll(x.data_ptr(), code, M, x.stride(0), pre.data.data_ptr(), K, n1 - n0, ptrs, world, n0, N,
                                          epoch, 0, sp) == 0
            locals_.append(Q._matmul_prepacked(x, pre, kernel="gemv"))
        full = torch.cat(locals_, dim=1)
        for t in lls:
            out = torch.empty(M, N, dtype=dtype, device=dev)
            assert lib.q4b_gather_ll_unpack(t.data_ptr(), M, N, N, 1, epoch, code, out.data_ptr(), N, sp) == 0
            assert torch.equal(out, full)
        # the two halves of a row as two partial results
        summed = torch.empty(M, N // 2, dtype=dtype, device=dev)
        assert lib.q4b_gather_ll_unpack(lls[0].data_ptr(), M, N // 2, N, 2, epoch, code, summed.data_ptr(), N // 2, sp) == 0
        assert torch.equal(summed, (locals_[0].float() + locals_[1].float()).to(dtype))
    assert Q.wait_status(dev) == 0
    # nobody stores epoch 7: the wait gives up after about two seconds
    out = torch.full((M, N), 3.0, dtype=dtype, device=dev)
    assert lib.q4b_gather_ll_unpack(lls[0].data_ptr(), M, 64, N, 1, 7, code, out.data_ptr(), N, sp) == 0
    detail = ctypes.c_int(0)
    assert lib.q4b_wait_status(sp, ctypes.byref(detail)) == _cabi.ERR_TIMEOUT and detail.value == 700
    assert float(out[:, :64].abs().max()) == 0.0
    assert Q.wait_status(dev) == 0
    assert torch.equal(Q._matmul_prepacked(x, pre, kernel="gemv"), locals_[1])
    assert lib.q4b_gemv_gather_ll(x.data_ptr(), code, M, x.stride(0), pre.data.data_ptr(), K, 1200, ptrs, world, 0, N, 0, 0, sp) != 0


def test_exchange_with_device_counter_on_one_gpu():
    """q4b_gemv_exchange_dev with one rank: the counter advances by one per call, the buffers alternate, the
    words that were read are cleared, and a captured call replays."""
    import ctypes
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import metalops_b200 as mo
    from metalops_b200 import _cabi, quantization as Q
    lib = _cabi.load()
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(79)
    K, N, M = 1056, 1200, 3
    pre = mo.prepack_ggml_q4_0(mo.quantize_ggml_q4_0((torch.randn(K, N, generator=g) * 0.02).to(dev)))
    x = torch.randn(M, K, generator=g).half().to(dev)
    ref = Q._matmul_prepacked(x, pre, kernel="gemv")
    ll = torch.zeros(2, 16, N, dtype=torch.int32, device=dev)
    ctl = torch.zeros(2, dtype=torch.int32, device=dev)
    ptrs = (ctypes.c_void_p * 1)(ll.data_ptr())
    out = torch.empty(M, N, dtype=torch.float16, device=dev)

    def call():
        rc = lib.q4b_gemv_exchange_dev(x.data_ptr(), _cabi.F16, M, K, pre.data.data_ptr(), K, N, ptrs, 1, 0, N, ll.data_ptr(), 16 * N, 1,
                                       ctl.data_ptr(), out.data_ptr(), N, 0, _cabi.stream_ptr(dev))
        assert rc == 0

    for i in range(5):
        out.zero_()
        call()
        assert torch.equal(out, ref)
        assert ctl.tolist() == [i + 1, 0]
        assert int(ll.abs().sum().item()) == 0                 # every word that was read is cleared again
    side = torch.cuda.Stream(dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            call()
        for _ in range(4):
            out.zero_()
            graph.replay()
    side.synchronize()
    assert torch.equal(out, ref) and ctl.tolist()[0] == 5 + 4 and Q.wait_status(dev) == 0
