"""A bounded device-side wait that runs out: the kernel must return, report the code through
q4b_wait_status, and leave the GPU usable.  The wait is made to run out harmlessly: a tiny kernel
waits, with a limit of a few thousand cycles, on a shared-memory barrier nobody arrives at."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_wait_runs_out_and_is_reported(cuda_dev):
    import metalops_b200 as mo
    from metalops_b200 import _cabi
    from metalops_b200 import quantization as Q
    lib = _cabi.load()
    assert Q.wait_status(cuda_dev) == 0
    assert lib.q4b_selftest_wait_timeout(20000, _cabi.stream_ptr(cuda_dev)) == _cabi.OK
    detail = ctypes.c_int(0)
    rc = lib.q4b_wait_status(_cabi.stream_ptr(cuda_dev), ctypes.byref(detail))
    assert rc == _cabi.ERR_TIMEOUT and detail.value == 900
    # the status was cleared by reading it, and the next product launch is green
    assert Q.wait_status(cuda_dev) == 0
    g = torch.Generator().manual_seed(1)
    w = torch.randn(256, 64, generator=g) * 0.02
    x = torch.randn(200, 256, generator=g).bfloat16()
    blocks = mo.quantize_ggml_q4_0(w.to(cuda_dev))
    y = mo.matmul_ggml_q4_0(x.to(cuda_dev), blocks)
    ref = x.float() @ mo.dequantize_ggml_q4_0(blocks, torch.float32).cpu()
    assert float((y.float().cpu() - ref).norm() / ref.norm()) <= 5e-3
    assert Q.wait_status(cuda_dev) == 0
    with pytest.raises(RuntimeError):                 # the Python helper raises on a timeout
        lib.q4b_selftest_wait_timeout(20000, _cabi.stream_ptr(cuda_dev))
        Q.wait_status(cuda_dev)
