"""The allocation-free host-buffer entry point, q4b_matmul_host_noalloc.

Some callers of this library may not allocate device memory at all (a plugin inside another
program's latency-critical loop, a host that owns every byte of the GPU in its own arena).  For
them the staging buffers live in a fixed array inside the library.  This test drives the entry
point through the C ABI with pinned host buffers, twice in a row with different data (the array
keeps the previous call's bytes, so the second call would show stale data if anything depended
on it), and requires bit-identical results to q4b_matmul_host with caller-allocated staging.
Collected last on purpose: a failure here must not hide the other tests' results.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _both(lib, cabi, x_host, pre, K, N, dev):
    M = x_host.shape[0]
    code = cabi.DTYPE_CODE[x_host.dtype]
    st = torch.cuda.current_stream(dev).cuda_stream
    y_new = torch.empty((M, N), dtype=x_host.dtype).pin_memory()
    rc = lib.q4b_matmul_host_noalloc(x_host.data_ptr(), code, M, pre.data.data_ptr(), K, N, y_new.data_ptr(), st)
    assert rc == 0, lib.q4b_strerror(rc)
    torch.cuda.synchronize(dev)
    y_old = torch.empty((M, N), dtype=x_host.dtype).pin_memory()
    x_dev = torch.empty((M, K), dtype=x_host.dtype, device=dev)
    y_dev = torch.empty((M, N), dtype=x_host.dtype, device=dev)
    rc = lib.q4b_matmul_host(x_host.data_ptr(), x_dev.data_ptr(), code, M, pre.data.data_ptr(), K, N,
                             y_dev.data_ptr(), y_old.data_ptr(), 0, st)
    assert rc == 0, lib.q4b_strerror(rc)
    torch.cuda.synchronize(dev)
    return y_new, y_old


def test_noalloc_matches_allocating_entry_twice(cuda_dev):
    import metalops_b200 as mo
    from metalops_b200 import _cabi
    from oracle import c_oracle
    from oracle import q4_0_oracle as orc
    lib = _cabi.load()
    _cabi.stream_ptr(cuda_dev)
    g = torch.Generator().manual_seed(4242)
    K, N = 1024, 2064
    w = torch.randn(K, N, generator=g) * 0.02
    blocks = mo.quantize_ggml_q4_0(w.to(cuda_dev))
    pre = mo.prepack_ggml_q4_0(blocks)
    with torch.cuda.device(cuda_dev):
        # first call: decode-sized (M = 3, fp16); second: a different shape, dtype and data
        for M, dt in ((3, torch.float16), (40, torch.bfloat16)):
            x = torch.randn(M, K, generator=g).to(dt).pin_memory()
            y_new, y_old = _both(lib, _cabi, x, pre, K, N, cuda_dev)
            assert torch.equal(y_new, y_old), f"M={M}: results differ from q4b_matmul_host"
            assert orc.rel_l2(y_new, c_oracle.matmul_f32(x, blocks.cpu())) <= 5e-3
        assert mo.quantization.wait_status(cuda_dev) == 0


def test_noalloc_rejects_sizes_beyond_the_fixed_array(cuda_dev):
    from metalops_b200 import _cabi
    lib = _cabi.load()
    buf = torch.empty(64, dtype=torch.uint8, device=cuda_dev)
    host = torch.empty(64, dtype=torch.uint8)
    # 128 x 8192 fp16 activations alone are 2 MiB, the [128, 28672] result another 7 MiB
    rc = lib.q4b_matmul_host_noalloc(host.data_ptr(), _cabi.F16, 128, buf.data_ptr(), 8192, 28672, host.data_ptr(), None)
    assert rc == _cabi.ERR_TOO_LARGE
    assert b"fixed internal buffer" in lib.q4b_strerror(rc)
