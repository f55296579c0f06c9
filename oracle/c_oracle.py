"""ctypes binding of the plain-C oracle (``q4_0_oracle.c``).  TEST INFRASTRUCTURE ONLY."""
from __future__ import annotations

import ctypes
import os
import subprocess

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libq4oracle.so")
_DT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}
_lib = None


def build(force: bool = False) -> str:
    """Compile the C oracle with gcc if the library is missing or older than its source."""
    src = os.path.join(_HERE, "q4_0_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B"], check=True, capture_output=True)
    return _SO


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        i64, vp, ci = ctypes.c_int64, ctypes.c_void_p, ctypes.c_int
        _lib.q4o_quantize.argtypes = [vp, ci, i64, i64, vp]
        _lib.q4o_dequantize_f32.argtypes = [vp, i64, i64, vp]
        _lib.q4o_matmul_f32.argtypes = [vp, ci, i64, vp, i64, i64, vp]
        _lib.q4o_f32_to_f16_bits.argtypes = [ctypes.c_float]
        _lib.q4o_f32_to_f16_bits.restype = ctypes.c_uint16
        _lib.q4o_f16_bits_to_f32.argtypes = [ctypes.c_uint16]
        _lib.q4o_f16_bits_to_f32.restype = ctypes.c_float
        _lib.q4o_f32_to_bf16_bits.argtypes = [ctypes.c_float]
        _lib.q4o_f32_to_bf16_bits.restype = ctypes.c_uint16
    return _lib


def quantize(weight: torch.Tensor) -> torch.Tensor:
    w = weight.contiguous()
    K, N = w.shape
    out = torch.empty((K // 32, N, 18), dtype=torch.uint8)
    rc = lib().q4o_quantize(w.data_ptr(), _DT[w.dtype], K, N, out.data_ptr())
    if rc:
        raise ValueError("q4o_quantize: bad arguments")
    return out


def dequantize_f32(blocks: torch.Tensor) -> torch.Tensor:
    b = blocks.contiguous()
    K, N = b.shape[0] * 32, b.shape[1]
    out = torch.empty((K, N), dtype=torch.float32)
    if lib().q4o_dequantize_f32(b.data_ptr(), K, N, out.data_ptr()):
        raise ValueError("q4o_dequantize_f32: bad arguments")
    return out


def matmul_f32(X: torch.Tensor, blocks: torch.Tensor) -> torch.Tensor:
    x = X.contiguous()
    b = blocks.contiguous()
    K, N = b.shape[0] * 32, b.shape[1]
    out = torch.empty((x.shape[0], N), dtype=torch.float32)
    if lib().q4o_matmul_f32(x.data_ptr(), _DT[x.dtype], x.shape[0], b.data_ptr(), K, N, out.data_ptr()):
        raise ValueError("q4o_matmul_f32: bad arguments")
    return out
