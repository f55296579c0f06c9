"""metalops_b200 — B200-native (sm_100a) implementation of metalcore's block_q4_0 INT4 matmul path.

Exports the hot-path names of the reference package (``packages/metalcore/src/metalcore/
__init__.py:38-39,174-184``) with the same signatures.  All compute runs in hand-written CUDA
kernels behind the C ABI of ``include/q4b200.h``; importing this package loads that library and
raises if it has not been built (``python metalops_b200/build.py``).
"""
from . import _cabi

_cabi.load()  # fail loudly at import time when the CUDA library is missing

from .quantization import (  # noqa: E402
    BLOCK_Q4_0_SIZE,
    QK4_0,
    Int4Linear,
    Q4Linear,
    Q4Prepacked,
    dequantize_ggml_q4_0,
    dequantize_int4,
    matmul_ggml_q4_0,
    fused_rmsnorm_linear_int4,
    import_ggml_q4_0,
    matmul_int4,
    matmul_int4_gelu,
    matmul_int4_silu,
    matmul_int8,
    prepack_ggml_q4_0,
    prepack_int4,
    quantize_ggml_q4_0,
    quantize_int4,
    rmsnorm,
    unpack_ggml_q4_0,
)
from .decode import DecodeChain, matmul_ggml_q4_0_grouped  # noqa: E402
from .sharding import ColumnParallelQ4Linear, FusedGatherBuffer, RowParallelQ4Linear, shard_bounds  # noqa: E402

__version__ = "0.1.0"


def has_native_kernels() -> bool:
    """True when the current CUDA device can run the kernels (compute capability 10.x)."""
    import torch

    return torch.cuda.is_available() and _cabi.load().q4b_device_ok() == _cabi.OK


__all__ = [
    "quantize_ggml_q4_0", "dequantize_ggml_q4_0", "matmul_ggml_q4_0", "prepack_ggml_q4_0",
    "unpack_ggml_q4_0", "Q4Prepacked", "Int4Linear", "Q4Linear", "prepack_int4", "quantize_int4", "dequantize_int4", "matmul_int4", "matmul_int4_silu", "matmul_int4_gelu",
    "fused_rmsnorm_linear_int4", "rmsnorm",
    "matmul_int8", "import_ggml_q4_0", "DecodeChain", "matmul_ggml_q4_0_grouped", "FusedGatherBuffer", "ColumnParallelQ4Linear", "RowParallelQ4Linear", "shard_bounds", "has_native_kernels", "QK4_0",
    "BLOCK_Q4_0_SIZE",
]
