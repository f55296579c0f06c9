"""CPU-side checks of the C-ABI boundary: the library builds, loads without a GPU, exports every
symbol the header declares, and its argument checks answer without touching a device."""
import ctypes
import os
import re

import torch

from conftest import ROOT


def header_symbols():
    text = open(os.path.join(ROOT, "include", "q4b200.h")).read()
    return sorted(set(re.findall(r"Q4B_API\s+[\w\s\*]+?\b(q4b_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    import __graft_entry__
    __graft_entry__.build()
    from metalops_b200 import _cabi
    lib = ctypes.CDLL(_cabi.LIB_PATH)
    declared = header_symbols()
    assert len(declared) >= 14
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/q4b200.h but not exported"
    assert sorted(_cabi.SYMBOLS) == declared, "the ctypes table and the header disagree"


def test_status_strings_and_sizes():
    from metalops_b200 import _cabi
    lib = _cabi.load()
    assert lib.q4b_version() >= 100
    assert lib.q4b_strerror(0) == b"ok"
    for code in range(1, 9):
        assert len(lib.q4b_strerror(code)) > 5
    assert lib.q4b_prepacked_bytes(4096, 4096) == 4096 * 4096 // 32 * 18      # same 18 bytes per block
    assert lib.q4b_prepacked_bytes(96, 7) == 2 * 1 * 576                       # padded to 64 k x 16 n tiles
    assert lib.q4b_prepacked_bytes(48, 4) == 0


def test_argument_checks_without_a_device():
    from metalops_b200 import _cabi
    lib = _cabi.load()
    buf = (ctypes.c_uint8 * 64)()
    p = ctypes.addressof(buf)
    p16 = (p + 15) & ~15
    assert lib.q4b_quantize(None, _cabi.F32, 32, 4, 0, p16, None, None) == _cabi.ERR_ARG
    assert lib.q4b_quantize(p16, _cabi.F32, 48, 4, 0, p16, None, None) == _cabi.ERR_SHAPE
    assert lib.q4b_quantize(p16, 7, 32, 4, 0, p16, None, None) == _cabi.ERR_DTYPE
    assert lib.q4b_quantize(p16, _cabi.F32, 32, 4, 5, p16, None, None) == _cabi.ERR_ARG
    assert lib.q4b_gemv(p16, _cabi.F16, 17, 32, p16, 32, 16, p16, 16, 0, None) == _cabi.ERR_SHAPE
    assert lib.q4b_gemv(p16, _cabi.F32, 1, 32, p16, 32, 16, p16, 16, 0, None) == _cabi.ERR_DTYPE
    assert lib.q4b_gemv(p16 + 2, _cabi.F16, 1, 32, p16, 32, 16, p16, 16, 0, None) == _cabi.ERR_ALIGN
    assert lib.q4b_gemm(p16, _cabi.F16, 0, 32, p16, 32, 16, p16, 16, 0, None) == _cabi.ERR_ARG
    if not torch.cuda.is_available():
        assert lib.q4b_device_ok() != _cabi.OK


def test_package_has_no_cpu_fallback():
    import pytest

    import metalops_b200 as mo
    with pytest.raises(RuntimeError):
        mo.quantize_ggml_q4_0(torch.zeros(32, 4))
    with pytest.raises(RuntimeError):
        mo.dequantize_ggml_q4_0(torch.zeros(1, 4, 18, dtype=torch.uint8))
    with pytest.raises(RuntimeError):
        mo.matmul_ggml_q4_0(torch.zeros(1, 32, dtype=torch.float16), torch.zeros(1, 4, 18, dtype=torch.uint8))
    for name in ("quantize_ggml_q4_0", "dequantize_ggml_q4_0", "matmul_ggml_q4_0", "matmul_int4", "Int4Linear"):
        assert hasattr(mo, name)


def test_product_never_imports_the_oracle():
    """Nothing under the package may import, open or execute the oracle."""
    pkg = os.path.join(ROOT, "metalops_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.lower(), f"{f} mentions the oracle"
