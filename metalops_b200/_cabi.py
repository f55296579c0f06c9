"""ctypes binding of ``libq4b200.so`` (declared in ``include/q4b200.h``).

The library is the only compute path of this package.  If it is missing or fails to load the
import raises; there is no fallback of any kind.
"""
from __future__ import annotations

import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libq4b200.so")

F32, F16, BF16 = 0, 1, 2
LAYOUT_KN, LAYOUT_NK = 0, 1
FLAG_NONE, FLAG_PDL, FLAG_ACT_SILU, FLAG_ACT_GELU = 0, 1, 8, 16
OK, ERR_ARG, ERR_SHAPE, ERR_DTYPE, ERR_ALIGN, ERR_ARCH, ERR_CUDA, ERR_TIMEOUT, ERR_TOO_LARGE = range(9)

DTYPE_CODE = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}

_i64, _vp, _ci = ctypes.c_int64, ctypes.c_void_p, ctypes.c_int

CHAIN_MAX_PRODUCTS = 4
CHAIN_X_PLAIN, CHAIN_X_SILU_MUL = 0, 1


class ChainProduct(ctypes.Structure):
    """q4b_chain_product of include/q4b200.h."""
    _fields_ = [("prepacked", _vp), ("y", _vp), ("addend", _vp), ("N", _i64), ("alpha", ctypes.c_float), ("flags", _ci)]


class ChainStage(ctypes.Structure):
    """q4b_chain_stage of include/q4b200.h."""
    _fields_ = [("x", _vp), ("x_stage", _ci), ("x_product", _ci), ("x_stage2", _ci), ("x_product2", _ci),
                ("xform", _ci), ("n_products", _ci), ("K", _i64), ("products", ChainProduct * CHAIN_MAX_PRODUCTS)]


# every symbol include/q4b200.h declares: name -> (restype, argtypes)
SYMBOLS = {
    "q4b_strerror": (ctypes.c_char_p, [_ci]),
    "q4b_last_cuda_error": (ctypes.c_char_p, []),
    "q4b_version": (_ci, []),
    "q4b_device_ok": (_ci, []),
    "q4b_prepacked_bytes": (ctypes.c_size_t, [_i64, _i64]),
    "q4b_quantize": (_ci, [_vp, _ci, _i64, _i64, _ci, _vp, _vp, _vp]),
    "q4b_repack": (_ci, [_vp, _i64, _i64, _vp, _vp]),
    "q4b_unpack": (_ci, [_vp, _i64, _i64, _vp, _vp]),
    "q4b_dequantize": (_ci, [_vp, _i64, _i64, _vp, _ci, _vp]),
    "q4b_gemv": (_ci, [_vp, _ci, _i64, _i64, _vp, _i64, _i64, _vp, _i64, _ci, _vp]),
    "q4b_gemm": (_ci, [_vp, _ci, _i64, _i64, _vp, _i64, _i64, _vp, _i64, _ci, _vp]),
    "q4b_matmul": (_ci, [_vp, _ci, _i64, _i64, _vp, _i64, _i64, _vp, _i64, _ci, _vp]),
    "q4b_wait_status": (_ci, [_vp, ctypes.POINTER(_ci)]),
    "q4b_selftest_wait_timeout": (_ci, [_i64, _vp]),
    "q4b_gemv_gather": (_ci, [_vp, _ci, _i64, _i64, _vp, _i64, _i64, ctypes.POINTER(_vp), _ci, _i64, _i64, _ci, _vp]),
    "q4b_gemv_gather_ll": (_ci, [_vp, _ci, _i64, _i64, _vp, _i64, _i64, ctypes.POINTER(_vp), _ci, _i64, _i64, _ci, _ci, _vp]),
    "q4b_gather_ll_unpack": (_ci, [_vp, _i64, _i64, _i64, _ci, _ci, _ci, _vp, _i64, _vp]),
    "q4b_gemv_exchange_dev": (_ci, [_vp, _ci, _i64, _i64, _vp, _i64, _i64, ctypes.POINTER(_vp), _ci, _i64, _i64, _vp, _i64, _ci, _vp,
                                    _vp, _i64, _ci, _vp]),
    "q4b_gemv_exchange": (_ci, [_vp, _ci, _i64, _i64, _vp, _i64, _i64, ctypes.POINTER(_vp), _ci, _i64, _i64, _vp, _ci, _ci, _vp, _i64,
                                _ci, _vp]),
    "q4b_import_ggml": (_ci, [_vp, _i64, _i64, _vp, _vp]),
    "q4b_quantize_ggml": (_ci, [_vp, _ci, _i64, _i64, _ci, _vp, _vp, _vp]),
    "q4b_int8g_matmul": (_ci, [_vp, _ci, _i64, _i64, _vp, _vp, _vp, _ci, _i64, _i64, _i64, _vp, _i64, _vp]),
    "q4b_gemv_grouped": (_ci, [_vp, _ci, _i64, ctypes.POINTER(ChainProduct), _ci, _ci, _vp]),
    "q4b_chain_workspace_bytes": (ctypes.c_size_t, [ctypes.POINTER(ChainStage), _ci]),
    "q4b_chain_build": (_ci, [ctypes.POINTER(ChainStage), _ci, _vp, ctypes.c_size_t, _vp]),
    "q4b_chain_run": (_ci, [_vp, _ci, _ci, _i64, _ci, _vp]),
    "q4b_rmsnorm": (_ci, [_vp, _ci, _i64, _i64, _i64, _vp, ctypes.c_float, _vp, _i64, _vp]),
    "q4b_matmul_host": (_ci, [_vp, _vp, _ci, _i64, _vp, _i64, _i64, _vp, _vp, _ci, _vp]),
    "q4b_matmul_host_noalloc": (_ci, [_vp, _ci, _i64, _vp, _i64, _i64, _vp, _vp]),
    "q4b_gemv_addend": (_ci, [_vp, _ci, _i64, _i64, _vp, _i64, _i64, _vp, _i64, _vp, _i64, _ci, _vp]),
    "q4b_gemm_addend": (_ci, [_vp, _ci, _i64, _i64, _vp, _i64, _i64, _vp, _i64, _vp, _i64, _ci, _vp]),
    "q4b_gemm_wt_addend": (_ci, [_vp, _ci, _i64, _i64, _vp, _i64, _i64, _vp, _i64, _vp, _i64, _ci, _vp]),
    "q4b_matmul_addend": (_ci, [_vp, _ci, _i64, _i64, _vp, _i64, _i64, _vp, _i64, _vp, _i64, _ci, _vp]),
    "q4b_int4g_quantize": (_ci, [_vp, _ci, _i64, _i64, _i64, _vp, _vp, _vp, _vp]),
    "q4b_int4g_dequantize": (_ci, [_vp, _vp, _vp, _ci, _i64, _i64, _i64, _vp, _ci, _vp]),
    "q4b_int4g_prepack": (_ci, [_vp, _vp, _vp, _ci, _i64, _i64, _i64, _vp, _vp, _vp]),
    "q4b_int4g_rowsums_bytes": (ctypes.c_size_t, [_i64, _i64, _i64]),
    "q4b_int4g_rowsums": (_ci, [_vp, _ci, _i64, _i64, _i64, _i64, _vp, _vp]),
    "q4b_int4g_gemv": (_ci, [_vp, _ci, _i64, _i64, _vp, _i64, _i64, _vp, _vp, _i64, _vp, _vp, _i64, _ci, _vp]),
    "q4b_int4g_fold_ktiles": (_ci, [_i64, _i64]),
    "q4b_int4g_fold_operand": (_ci, [_vp, _i64, _i64, _i64, _vp, _vp]),
    "q4b_int4g_fold_rows": (_ci, [_vp, _ci, _i64, _i64, _i64, _i64, _vp, _vp]),
    "q4b_int4g_gemm_fold": (_ci, [_vp, _ci, _i64, _i64, _vp, _i64, _i64, _vp, _vp, _ci, _vp, _vp, _i64, _ci, _vp]),
    "q4b_int4g_addend": (_ci, [_vp, _ci, _i64, _i64, _vp, _vp, _i64, _i64, _i64, _vp, _vp, _vp]),
    "q4b_int4g_prepack_status": (_ci, [_vp, ctypes.POINTER(_ci)]),
    "q4b_int4g_matmul_generic": (_ci, [_vp, _ci, _i64, _i64, _vp, _vp, _vp, _ci, _i64, _i64, _i64, _vp, _i64, _vp]),
}

_lib = None


def load() -> ctypes.CDLL:
    """Load the shared library (once) and set the prototypes.  Raises if it is not built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python metalops_b200/build.py` "
                "(needs nvcc). This package has no CPU or PyTorch fallback.")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(lib, name)          # AttributeError if the library lacks a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(status: int, what: str) -> None:
    """Turn a non-zero status into the RuntimeError the reference's TORCH_CHECKs would raise
    (core_mps.mm:5923-5938), with the library's own message."""
    if status != OK:
        lib = load()
        msg = lib.q4b_strerror(status).decode()
        if status == ERR_CUDA:
            msg += ": " + lib.q4b_last_cuda_error().decode()
        raise RuntimeError(f"{what}: {msg}")


def require_device(t: torch.Tensor, name: str) -> None:
    if t.device.type != "cuda":
        raise RuntimeError(
            f"{name} must be a CUDA tensor (got {t.device}); this build is B200-only and has no CPU fallback")


_checked_devices: set[int] = set()


def stream_ptr(device: torch.device) -> int:
    """Current torch stream of ``device`` as a raw cudaStream_t; checks the architecture once."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _checked_devices:
        with torch.cuda.device(idx):
            check(load().q4b_device_ok(), "q4b200")
        _checked_devices.add(idx)
    return torch.cuda.current_stream(idx).cuda_stream
