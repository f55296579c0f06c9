"""GPU parity of the group-wise asymmetric INT4 path (quantize_int4, dequantize_int4,
matmul_int4, Int4Linear) against fixtures produced by the reference module and the CPU oracle."""
import numpy as np
import pytest
import torch

from conftest import golden_tensor, load_golden
from oracle import q4_0_oracle as orc

pytestmark = pytest.mark.gpu
TOL = 5e-3

CASES = [("g128_f32", 128), ("g64_f32", 64), ("g128_f16", 128), ("g128_ragged", 128)]


@pytest.fixture(scope="module")
def mo(cuda_dev):
    import metalops_b200
    assert metalops_b200.has_native_kernels()
    return metalops_b200


def same_bits(a: torch.Tensor, b: torch.Tensor) -> bool:
    """Equal including NaNs in the same places (a constant fp16 group yields NaN in the reference)."""
    a, b = a.cpu(), b.cpu()
    return a.dtype == b.dtype and a.shape == b.shape and bool(torch.allclose(a.float(), b.float(), rtol=0, atol=0, equal_nan=True))


@pytest.mark.parametrize("name,gs", CASES)
def test_golden_quantize_dequantize(mo, cuda_dev, name, gs):
    z = load_golden("int4_groupwise.npz")
    w = golden_tensor(z, f"{name}.w")
    packed, scales, zeros = mo.quantize_int4(w.to(cuda_dev), gs)
    assert scales.dtype == w.dtype and zeros.dtype == w.dtype and packed.dtype == torch.uint8
    assert same_bits(scales, golden_tensor(z, f"{name}.scales"))
    assert same_bits(zeros, golden_tensor(z, f"{name}.zeros"))
    gp = golden_tensor(z, f"{name}.packed")
    finite_cols = torch.isfinite(golden_tensor(z, f"{name}.zeros").float()).all(dim=0)
    # columns whose zero point is not finite go through an undefined NaN -> uint8 cast in the reference
    assert torch.equal(packed.cpu()[:, finite_cols], gp[:, finite_cols])
    deq = mo.dequantize_int4(gp.to(cuda_dev), golden_tensor(z, f"{name}.scales").to(cuda_dev),
                             golden_tensor(z, f"{name}.zeros").to(cuda_dev), gs, torch.float32)
    assert same_bits(deq, golden_tensor(z, f"{name}.deq_f32"))
    assert mo.dequantize_int4(packed, scales, zeros, gs).dtype == torch.float16


@pytest.mark.parametrize("name,gs", CASES)
def test_golden_matmul_int4(mo, cuda_dev, name, gs):
    z = load_golden("int4_groupwise.npz")
    x = golden_tensor(z, f"{name}.x")
    packed = golden_tensor(z, f"{name}.packed").to(cuda_dev)
    scales = golden_tensor(z, f"{name}.scales").to(cuda_dev)
    zeros = golden_tensor(z, f"{name}.zeros").to(cuda_dev)
    y = mo.matmul_int4(x.to(cuda_dev), packed, scales, zeros, gs)
    ref = golden_tensor(z, f"{name}.y")
    assert y.dtype == x.dtype and tuple(y.shape) == tuple(ref.shape)
    cols = torch.isfinite(ref.float()).all(dim=0)
    assert cols.sum() >= ref.shape[1] - 1
    assert orc.rel_l2(y.cpu()[:, cols], ref[:, cols]) <= TOL
    ref32 = x.float() @ golden_tensor(z, f"{name}.deq_f32")
    assert orc.rel_l2(y.cpu()[:, cols], ref32[:, cols]) <= TOL


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_seeded_quantize_vs_oracle(mo, cuda_dev, dtype):
    g = torch.Generator().manual_seed(21)
    w = (torch.randn(1024, 300, generator=g) * 0.05).to(dtype)
    packed, scales, zeros = mo.quantize_int4(w.to(cuda_dev), 128)
    op, os_, oz = orc.quantize_int4_groupwise(w, 128)
    assert torch.equal(packed.cpu(), op)
    assert same_bits(scales, os_) and same_bits(zeros, oz)
    assert same_bits(mo.dequantize_int4(packed, scales, zeros, 128, torch.float32),
                     orc.dequantize_int4_groupwise(op, os_, oz, 128, torch.float32))


@pytest.mark.parametrize("M,xdtype", [(1, torch.float16), (8, torch.float16), (16, torch.bfloat16), (70, torch.bfloat16),
                                      (200, torch.float16)])
def test_seeded_matmul_int4(mo, cuda_dev, M, xdtype):
    g = torch.Generator().manual_seed(50 + M)
    K, N = 2048, 1040
    w = torch.randn(K, N, generator=g) * 0.03 + 0.01            # non-zero mean: the zero-point term matters
    x = torch.randn(M, K, generator=g).to(xdtype)
    packed, scales, zeros = mo.quantize_int4(w.to(cuda_dev), 128)
    y = mo.matmul_int4(x.to(cuda_dev), packed, scales, zeros, 128)
    ref = x.float() @ orc.dequantize_int4_groupwise(packed.cpu(), scales.cpu(), zeros.cpu(), 128, torch.float32)
    err = orc.rel_l2(y, ref)
    assert err <= (1e-3 if xdtype == torch.float16 else TOL), f"rel-L2 {err:.3e}"
    # batched input [B, M, K] like the reference accepts
    yb = mo.matmul_int4(x.to(cuda_dev).unsqueeze(0).repeat(2, 1, 1), packed, scales, zeros, 128)
    assert tuple(yb.shape) == (2, M, N)
    assert orc.rel_l2(yb[1], ref) <= TOL and orc.rel_l2(yb[0], ref) <= TOL     # 2M rows may take another kernel
    assert mo.quantization.wait_status(cuda_dev) == 0


def test_int4_linear_matches_reference_module(mo, cuda_dev):
    z = load_golden("int4_linear.npz")
    lin = torch.nn.Linear(256, 24, bias=True)
    lin.weight.data.copy_(golden_tensor(z, "lin.weight"))
    lin.bias.data.copy_(golden_tensor(z, "lin.bias"))
    lin = lin.to(cuda_dev)
    ql = mo.Int4Linear.from_float(lin, group_size=128, dequant_on_load=False)
    sd = ql.state_dict()
    assert sorted(sd.keys()) == sorted(z["state_keys"].tolist())
    for k in sd:
        assert same_bits(sd[k], golden_tensor(z, f"sd.{k}")), k
    assert ql.extra_repr() == str(z["repr_int4"])
    x = golden_tensor(z, "x").to(cuda_dev)
    y = ql(x)
    assert y.dtype == torch.float32
    assert orc.rel_l2(y, golden_tensor(z, "y_int4")) <= TOL
    ql.dequantize()
    assert ql.extra_repr() == str(z["repr_fast"])
    assert orc.rel_l2(ql(x), golden_tensor(z, "y_fp16cache")) <= TOL
    ql.keep_quantized()
    assert torch.equal(ql(x), y)
    # a checkpoint written by the reference loads into a fresh module
    fresh = mo.Int4Linear(256, 24, group_size=128, dequant_on_load=False, device=cuda_dev)
    fresh.load_state_dict({k: golden_tensor(z, f"sd.{k}") for k in sd})
    assert torch.equal(fresh(x), y)


def test_int4_errors(mo, cuda_dev):
    w = torch.zeros(64, 8, device=cuda_dev)
    with pytest.raises(RuntimeError):
        mo.quantize_int4(torch.zeros(64, 8), 32)                       # CPU tensor: no fallback
    with pytest.raises(RuntimeError):
        mo.quantize_int4(w, 31)                                        # odd group
    big = torch.full((64, 8), 3.0e6, device=cuda_dev)
    big[::2] = -3.0e6
    p, s, zz = mo.quantize_int4(big, 32)                                  # scale 4e5: beyond fp16
    with pytest.raises(RuntimeError, match="float16"):
        mo.matmul_int4(torch.zeros(1, 64, device=cuda_dev, dtype=torch.float16), p, s, zz, 32)
    with pytest.raises(RuntimeError):                                  # CPU tensors: no fallback
        mo.matmul_int8(torch.zeros(1, 64), torch.zeros(64, 8, dtype=torch.int8), torch.ones(1, 8), torch.zeros(1, 8), 64)


@pytest.mark.parametrize("M", [1, 5, 16, 40, 300])
@pytest.mark.parametrize("act", ["silu", "gelu"])
def test_matmul_int4_fused_activation(mo, cuda_dev, M, act):
    """matmul_int4_silu / matmul_int4_gelu: the activation is applied to the fp32 sum in the
    kernels' epilogues (decode, prefill) — compared with activation(fp32 reference matmul)."""
    g = torch.Generator().manual_seed(7000 + M)
    K, N, gs = 512, 328, 128
    w = torch.randn(K, N, generator=g) * 0.05
    x = torch.randn(M, K, generator=g).half()
    packed, scales, zeros = mo.quantize_int4(w.to(cuda_dev), gs)
    wd = orc.dequantize_int4_groupwise(packed.cpu(), scales.cpu(), zeros.cpu(), gs, torch.float32)
    lin = x.float() @ wd
    ref = torch.nn.functional.silu(lin) if act == "silu" else torch.nn.functional.gelu(lin, approximate="tanh")
    fn = mo.matmul_int4_silu if act == "silu" else mo.matmul_int4_gelu
    y = fn(x.to(cuda_dev), packed, scales, zeros, gs)
    assert y.dtype == x.dtype and tuple(y.shape) == (M, N)
    assert orc.rel_l2(y, ref) <= TOL
    # the unfused composition agrees too
    y_lin = mo.matmul_int4(x.to(cuda_dev), packed, scales, zeros, gs).float().cpu()
    y_unfused = torch.nn.functional.silu(y_lin) if act == "silu" else torch.nn.functional.gelu(y_lin, approximate="tanh")
    assert orc.rel_l2(y, y_unfused) <= TOL


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("M", [1, 7, 33])
def test_rmsnorm_and_fused_rmsnorm_linear_int4(mo, cuda_dev, M, dtype):
    """rmsnorm against the fp32 formula with one rounding (bit-exact when the fp32 sums agree, so
    compared by tolerance of one ulp-scale), and fused_rmsnorm_linear_int4 against the composition
    the reference runs: rmsnorm rounded to X.dtype, then the INT4 matmul."""
    g = torch.Generator().manual_seed(8000 + M)
    K, N, gs, eps = 1024, 200, 128, 1e-5
    x = (torch.randn(M, K, generator=g) * 1.5).to(dtype)
    wn = (1.0 + 0.1 * torch.randn(K, generator=g)).to(dtype)
    w = torch.randn(K, N, generator=g) * 0.05
    xn = mo.rmsnorm(x.to(cuda_dev), wn.to(cuda_dev), eps)
    assert xn.dtype == dtype and tuple(xn.shape) == (M, K)
    xf = x.float()
    ref_n = (xf * torch.rsqrt(xf.pow(2).mean(dim=1, keepdim=True) + eps) * wn.float())
    assert orc.rel_l2(xn, ref_n) <= (2e-3 if dtype == torch.bfloat16 else 3e-4)      # one rounding to dtype
    assert torch.equal(xn, mo.rmsnorm(x.to(cuda_dev), wn.to(cuda_dev), eps)), "two runs differ bitwise"
    packed, scales, zeros = mo.quantize_int4(w.to(cuda_dev), gs)
    y = mo.fused_rmsnorm_linear_int4(x.to(cuda_dev), wn.to(cuda_dev), packed, scales, zeros, eps, gs)
    wd = mo.dequantize_int4(packed, scales, zeros, gs, torch.float32).cpu()
    ref = xn.float().cpu() @ wd
    assert y.dtype == dtype and tuple(y.shape) == (M, N)
    assert orc.rel_l2(y, ref) <= TOL


def test_activation_on_q4_0_kernels_all_paths(mo, cuda_dev):
    """The activation flag on every matmul kernel: single-row and multi-row decode, the
    small-batch tensor-memory kernel and the prefill kernel.  Reference weights come from the oracle."""
    from metalops_b200 import _cabi, quantization as Q
    g = torch.Generator().manual_seed(9001)
    K, N = 1024, 520
    w = torch.randn(K, N, generator=g) * 0.05
    blocks = mo.quantize_ggml_q4_0(w.to(cuda_dev))
    pre = mo.prepack_ggml_q4_0(blocks)
    wd = orc.dequantize_q4_0(blocks.cpu(), torch.float32)
    for M, kernel, extra in ((1, "gemv", 0), (6, "gemv", 0), (14, "gemv", 0), (70, "gemm", 0), (400, "gemm", 0)):
        x = torch.randn(M, K, generator=g).half()
        lin = x.float() @ wd
        for flag, ref in ((_cabi.FLAG_ACT_SILU, torch.nn.functional.silu(lin)),
                          (_cabi.FLAG_ACT_GELU, torch.nn.functional.gelu(lin, approximate="tanh"))):
            y = Q._matmul_prepacked(x.to(cuda_dev), pre, kernel=kernel, flags=flag | extra)
            assert orc.rel_l2(y, ref) <= TOL, (M, kernel, extra, flag)
    assert Q.wait_status(cuda_dev) == 0


@pytest.mark.parametrize("K,gs", [(64, 16), (96, 48), (130, 26), (256, 100)])
def test_matmul_int4_group_sizes_outside_the_tile_format(mo, cuda_dev, K, gs):
    """K or group_size not a multiple of 32: the reference's loop takes them (quantization.py:207-239);
    here a CUDA-core kernel reads the [K/2, N] format directly."""
    g = torch.Generator().manual_seed(K + gs)
    N = 37
    w = torch.randn(K, N, generator=g) * 0.05
    packed, scales, zeros = mo.quantize_int4(w.to(cuda_dev), gs)
    wd = orc.dequantize_int4_groupwise(packed.cpu(), scales.cpu(), zeros.cpu(), gs, torch.float32)
    for M in (1, 9):
        x = torch.randn(M, K, generator=g).half()
        y = mo.matmul_int4(x.to(cuda_dev), packed, scales, zeros, gs)
        assert y.dtype == x.dtype and tuple(y.shape) == (M, N)
        assert orc.rel_l2(y, x.float() @ wd) <= TOL
    lin = torch.nn.Linear(K, N).to(cuda_dev)
    ql = mo.Int4Linear.from_float(lin, group_size=gs)
    xl = torch.randn(3, K, generator=g).to(cuda_dev)
    assert orc.rel_l2(ql(xl), lin(xl)) <= 0.2                                  # the 4-bit quantisation error itself


def test_int4_linear_default_runs_the_fused_kernels(mo, cuda_dev):
    lin = torch.nn.Linear(256, 48).to(cuda_dev)
    ql = mo.Int4Linear.from_float(lin)                                         # reference defaults
    assert ql._weight_dequant is None and "int4_kernel" in ql.extra_repr()
    x = torch.randn(70000, 256, device=cuda_dev).half()                        # more rows than a grid dimension holds
    y = ql(x)
    assert tuple(y.shape) == (70000, 48)
    assert orc.rel_l2(y[:64], lin(x[:64].float())) <= 0.2
    ql.dequantize()
    assert "fast_fp16" in ql.extra_repr()


def test_addend_many_rows_and_ragged_tiles(mo, cuda_dev):
    """q4b_int4g_addend through the C ABI: more row tiles than a grid dimension holds (the entry point
    slices them), a last tile of few rows, odd N (scalar loads and stores), two passes over the groups."""
    from metalops_b200 import _cabi
    lib = _cabi.load()
    g = torch.Generator().manual_seed(77)
    for M, K, N, group in ((2_097_153, 64, 3, 32), (37, 2304, 515, 128), (1, 4096, 1000, 32)):
        G = K // group
        x = torch.randn(M, K, generator=g).half().to(cuda_dev)
        corr = torch.randn(G, N, generator=g).to(cuda_dev)
        bias = torch.randn(N, generator=g).to(cuda_dev)
        out = torch.empty((M, N), dtype=torch.float32, device=cuda_dev)
        ws = torch.empty(lib.q4b_int4g_rowsums_bytes(M, K, group) // 4, dtype=torch.float32, device=cuda_dev)
        assert ws.numel() == M * G
        rc = lib.q4b_int4g_addend(x.data_ptr(), _cabi.F16, M, K, corr.data_ptr(), bias.data_ptr(), K, N, group, ws.data_ptr(),
                                  out.data_ptr(), _cabi.stream_ptr(cuda_dev))
        assert rc == 0
        torch.cuda.synchronize()
        ref = x.float().view(M, G, group).sum(-1) @ corr + bias
        assert torch.allclose(out, ref, rtol=1e-4, atol=1e-4), (M, K, N, float((out - ref).abs().max()))
    assert lib.q4b_int4g_addend(x.data_ptr(), _cabi.F16, 1, 4096, corr.data_ptr(), None, 4096, 1000, 32, None, out.data_ptr(), None) == _cabi.ERR_ARG


@pytest.mark.parametrize("M,K,N,gs,xdtype,shift", [
    (1, 4096, 1000, 128, torch.float16, 0.05),           # the decode kernels: the term formed in the epilogue
    (7, 2080, 520, 32, torch.bfloat16, 0.08),
    (16, 256, 200, 128, torch.float16, 0.0),
    (17, 256, 200, 128, torch.float16, 0.0),
    (100, 8192, 520, 128, torch.bfloat16, 0.0),          # the small-batch kernel, clusters splitting the extended k range
    (128, 2080, 520, 32, torch.float16, 0.08),
    (300, 256, 200, 128, torch.float16, 0.0),
    (129, 4096, 1000, 128, torch.bfloat16, 0.05),       # zero points far from 8: the term is 15 x the main product
    (513, 2080, 520, 32, torch.float16, 0.08),          # odd number of k-tiles, seven fold tiles
    (2048, 4096, 264, 128, torch.bfloat16, 0.0),
])
def test_folded_zero_point_term_matches_the_addend_path(mo, cuda_dev, M, K, N, gs, xdtype, shift):
    """Above 16 rows matmul_int4 carries the zero-point term inside the contraction (extra k-tiles, bf16
    three-way splits; both tensor-core kernels); up to 16 rows the decode kernels form it in their epilogue.  It must agree with the fp32-addend path to a unit of the output type, and with
    the fp64 product of the dequantised weight like that path does; bias and activation included."""
    from metalops_b200 import quantization as Q
    g = torch.Generator().manual_seed(M + K)
    w = (torch.randn(K, N, generator=g) * 0.02 + shift).half().to(cuda_dev)
    x = (torch.randn(M, K, generator=g).abs() * 0.5 + 0.1).to(xdtype).to(cuda_dev)      # a positive mean: a large term
    bias = torch.randn(N, generator=g).to(cuda_dev)
    p, s, z = mo.quantize_int4(w, gs)
    ref = x.double() @ mo.dequantize_int4(p, s, z, gs).double()
    pre = Q.prepack_int4(p, s, z, gs)
    assert pre.fold_ktiles == (6 * (K // gs) + 63) // 64
    y_fold = Q._matmul_int4_prepacked(x, pre)
    yb_fold = Q._matmul_int4_prepacked(x, pre, bias=bias, activation="silu")
    assert Q.wait_status(cuda_dev) == 0
    y_add = Q._matmul_int4_via_addend(x, pre)
    yb_add = Q._matmul_int4_via_addend(x, pre, bias=bias, activation="silu")
    e_fold, e_add = orc.rel_l2(y_fold, ref.float()), orc.rel_l2(y_add, ref.float())
    assert e_fold <= max(1.05 * e_add, 1e-4), (e_fold, e_add)
    ulp = 2.0 ** (-7 if xdtype == torch.bfloat16 else -10)
    assert float(((y_fold.float() - y_add.float()).abs() / y_add.float().abs().clamp_min(1.0)).max()) <= 2 * ulp
    assert float(((yb_fold.float() - yb_add.float()).abs() / yb_add.float().abs().clamp_min(1.0)).max()) <= 2 * ulp
    assert torch.equal(y_fold, Q._matmul_int4_prepacked(x, pre)), "two runs differ bitwise"
