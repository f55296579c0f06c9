"""Generate the golden fixtures in this folder from the reference implementation itself.

Run once, in a container that has the reference checkout, as
    python tests/golden/make_golden.py /path/to/reference
It loads ``packages/metalcore/src/metalcore/quantization.py`` BY FILE PATH (the package
itself does not import off Apple hardware) and records, for seeded inputs, exactly what the
reference's CPU path returns.  The fixtures are small ``.npz`` files; bf16 tensors are
stored as their uint16 bit patterns, fp16 as numpy float16.

The tests never need the reference checkout: they read only the committed ``.npz`` files.
"""
from __future__ import annotations

import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference(root: str):
    path = os.path.join(root, "packages", "metalcore", "src", "metalcore", "quantization.py")
    sys.dont_write_bytecode = True
    spec = importlib.util.spec_from_file_location("ref_quantization", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    assert mod._HAS_METAL is False
    return mod


def to_np(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.bfloat16:
        return t.contiguous().view(torch.uint16).numpy().copy()
    return t.contiguous().numpy().copy()


def make_weight(seed: int, K: int, N: int, dtype: torch.dtype, std: float) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(K, N, generator=g) * std
    nb = K // 32
    # a few all-zero blocks, a few outliers, exact ties and a block of tiny values
    zero_mask = torch.rand(nb, N, generator=g) < 0.03
    w = w.view(nb, 32, N).masked_fill(zero_mask.unsqueeze(1), 0.0).reshape(K, N)
    idx = torch.randperm(K * N, generator=g)[: max(4, K * N // 500)]
    sign = torch.where(torch.rand(idx.numel(), generator=g) < 0.5, -1.0, 1.0)
    w.view(-1)[idx] = 0.5 * sign
    if K >= 64 and N >= 4:
        w[32:64, 0] = torch.linspace(-7.0, 7.0, 32) / 7.0 * 0.875      # exact multiples of d
        w[32:64, 1] = torch.linspace(-6.5, 6.5, 32) / 7.0 * 0.875      # lands on .5 ties
        w[0:32, 2] = 1e-7 * torch.randn(32, generator=g)                # subnormal fp16 scale
        w[0:32, 3] = -w[0:32, 3].abs()                                   # all-negative block
    return w.to(dtype)


def main() -> None:
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <path of the reference checkout>")
    root = sys.argv[1]
    ref = load_reference(root)
    torch.set_num_threads(1)

    # ---- q4_0 pack / unpack ---------------------------------------------------------
    cases = [
        ("f32_a", 1101, 128, 48, torch.float32, 0.02),
        ("f32_b", 1102, 32, 7, torch.float32, 1.0),
        ("f32_c", 1103, 320, 33, torch.float32, 0.015),
        ("f16_a", 1104, 128, 48, torch.float16, 0.02),
        ("f16_b", 1105, 96, 19, torch.float16, 1.0),
        ("bf16_a", 1106, 128, 48, torch.bfloat16, 0.02),
        ("bf16_b", 1107, 64, 5, torch.bfloat16, 3.0),
    ]
    out = {}
    for name, seed, K, N, dt, std in cases:
        w = make_weight(seed, K, N, dt, std)
        blocks = ref.quantize_ggml_q4_0(w)
        out[f"{name}.w"] = to_np(w)
        out[f"{name}.blocks"] = to_np(blocks)
        out[f"{name}.deq_f32"] = to_np(ref.dequantize_ggml_q4_0(blocks, torch.float32))
        out[f"{name}.deq_f16"] = to_np(ref.dequantize_ggml_q4_0(blocks))
    np.savez_compressed(os.path.join(HERE, "q4_0_pack.npz"), **out)

    # ---- q4_0 matmul (public path: dequantise to X.dtype, torch matmul) --------------
    out = {}
    for name, seed, M, K, N, xdt in [
        ("h_m1", 1201, 1, 256, 40, torch.float16),
        ("h_m5", 1202, 5, 128, 24, torch.float16),
        ("b_m16", 1203, 16, 128, 24, torch.bfloat16),
        ("b_m70", 1204, 70, 192, 136, torch.bfloat16),
        ("f_m3", 1205, 3, 64, 9, torch.float32),
    ]:
        g = torch.Generator().manual_seed(seed)
        w = torch.randn(K, N, generator=g) * 0.02
        x = torch.randn(M, K, generator=g).to(xdt)
        blocks = ref.quantize_ggml_q4_0(w)
        out[f"{name}.x"] = to_np(x)
        out[f"{name}.blocks"] = to_np(blocks)
        out[f"{name}.y_public"] = to_np(ref.matmul_ggml_q4_0(x, blocks))
        out[f"{name}.y_fp32"] = to_np(x.float() @ ref.dequantize_ggml_q4_0(blocks, torch.float32))
    np.savez_compressed(os.path.join(HERE, "q4_0_matmul.npz"), **out)

    # ---- group-wise asymmetric INT4 (quantize_int4 / dequantize_int4 / matmul_int4) ---
    out = {}
    for name, seed, K, N, gs, dt in [
        ("g128_f32", 1301, 256, 20, 128, torch.float32),
        ("g64_f32", 1302, 192, 12, 64, torch.float32),
        ("g128_f16", 1303, 256, 16, 128, torch.float16),
        ("g128_ragged", 1304, 160, 10, 128, torch.float32),
    ]:
        g = torch.Generator().manual_seed(seed)
        w = (torch.randn(K, N, generator=g) * 0.05).to(dt)
        if N > 2:
            w[: min(K, gs), 2] = 0.25          # constant group: scale clamps to 1e-8
        x = torch.randn(3, K, generator=g).to(dt)
        packed, scales, zeros = ref.quantize_int4(w, gs)
        out[f"{name}.w"] = to_np(w)
        out[f"{name}.x"] = to_np(x)
        out[f"{name}.packed"] = to_np(packed)
        out[f"{name}.scales"] = to_np(scales)
        out[f"{name}.zeros"] = to_np(zeros)
        out[f"{name}.deq_f32"] = to_np(ref.dequantize_int4(packed, scales, zeros, gs, torch.float32))
        out[f"{name}.y"] = to_np(ref.matmul_int4(x, packed, scales, zeros, gs))
    np.savez_compressed(os.path.join(HERE, "int4_groupwise.npz"), **out)

    # ---- group-wise INT8 matmul (matmul_int8, CPU path) --------------------------------
    out = {}
    for name, seed, M, K, N, gs, dt in [
        ("g128_h", 1501, 3, 256, 40, 128, torch.float16),
        ("g64_b", 1502, 9, 192, 130, 64, torch.bfloat16),
        ("g128_ragged_f", 1503, 2, 160, 7, 128, torch.float32),
    ]:
        g = torch.Generator().manual_seed(seed)
        w_q = torch.randint(-128, 128, (K, N), generator=g, dtype=torch.int16).to(torch.int8)
        ng = (K + gs - 1) // gs
        scales = (torch.rand(ng, N, generator=g) * 0.01 + 0.001).to(dt)
        zeros = (torch.randn(ng, N, generator=g) * 20.0).to(dt)
        x = torch.randn(M, K, generator=g).to(dt)
        out[f"{name}.x"] = to_np(x)
        out[f"{name}.w_q"] = to_np(w_q)
        out[f"{name}.scales"] = to_np(scales)
        out[f"{name}.zeros"] = to_np(zeros)
        out[f"{name}.y"] = to_np(ref.matmul_int8(x, w_q, scales, zeros, gs))
    np.savez_compressed(os.path.join(HERE, "int8_groupwise.npz"), **out)

    # ---- Int4Linear surface ----------------------------------------------------------
    torch.manual_seed(1401)
    lin = torch.nn.Linear(256, 24, bias=True)
    ql = ref.Int4Linear.from_float(lin, group_size=128, dequant_on_load=False)
    x = torch.randn(4, 256)
    out = {
        "lin.weight": to_np(lin.weight.data), "lin.bias": to_np(lin.bias.data), "x": to_np(x),
        "y_int4": to_np(ql(x)),
        "state_keys": np.array(sorted(ql.state_dict().keys())),
    }
    for k, v in ql.state_dict().items():
        out[f"sd.{k}"] = to_np(v)
    ql.dequantize()
    out["y_fp16cache"] = to_np(ql(x))
    out["repr_fast"] = np.array(ql.extra_repr())
    ql.keep_quantized()
    out["repr_int4"] = np.array(ql.extra_repr())
    np.savez_compressed(os.path.join(HERE, "int4_linear.npz"), **out)
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    main()
