"""GPU parity of the q4_0 matmul (decode GEMV and prefill GEMM kernels, through the C ABI)
against the CPU oracle: relative L2 error <= 5e-3 versus dequantise-then-fp32-matmul."""
import pytest
import torch

from conftest import golden_tensor, load_golden
from oracle import c_oracle
from oracle import q4_0_oracle as orc

pytestmark = pytest.mark.gpu

TOL = 5e-3            # the stated tolerance of the path
TOL_F16 = 1e-3        # what fp16 activations should comfortably reach (fp32 accumulation)


@pytest.fixture(scope="module")
def mo(cuda_dev):
    import metalops_b200
    assert metalops_b200.has_native_kernels()
    return metalops_b200


def make_case(seed, M, K, N, xdtype, std=0.02, outliers=0.0):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(K, N, generator=g) * std
    if outliers:
        idx = torch.randperm(K * N, generator=g)[: int(K * N * outliers)]
        sign = torch.where(torch.rand(idx.numel(), generator=g) < 0.5, -1.0, 1.0)
        w.view(-1)[idx] = 0.5 * sign
    x = torch.randn(M, K, generator=g).to(xdtype)
    return w, x


def check(mo, dev, w, x, tol, kernel="auto"):
    from metalops_b200 import quantization as Q
    blocks = mo.quantize_ggml_q4_0(w.to(dev))
    pre = mo.prepack_ggml_q4_0(blocks)
    y = Q._matmul_prepacked(x.to(dev), pre, kernel=kernel)
    assert y.dtype == x.dtype and tuple(y.shape) == (x.shape[0], w.shape[1])
    ref = c_oracle.matmul_f32(x, blocks.cpu())
    err = orc.rel_l2(y, ref)
    assert torch.isfinite(y).all()
    assert err <= tol, f"rel-L2 {err:.3e} > {tol}"
    y2 = Q._matmul_prepacked(x.to(dev), pre, kernel=kernel)
    assert torch.equal(y, y2), "two runs differ bitwise"
    return err


@pytest.mark.parametrize("name", ["h_m1", "h_m5", "b_m16", "f_m3"])
def test_golden_matmul_decode(mo, cuda_dev, name):
    z = load_golden("q4_0_matmul.npz")
    x = golden_tensor(z, f"{name}.x")
    blocks = golden_tensor(z, f"{name}.blocks").to(cuda_dev)
    y = mo.matmul_ggml_q4_0(x.to(cuda_dev), blocks)
    assert y.dtype == x.dtype
    assert orc.rel_l2(y, golden_tensor(z, f"{name}.y_fp32")) <= TOL
    # and no further from the reference's own public result than that result is from fp32
    assert orc.rel_l2(y, golden_tensor(z, f"{name}.y_public")) <= 2 * TOL


@pytest.mark.parametrize("M", [1, 2, 3, 7, 8, 9, 15, 16])
@pytest.mark.parametrize("xdtype", [torch.float16, torch.bfloat16])
def test_decode_all_m(mo, cuda_dev, M, xdtype):
    w, x = make_case(100 + M, M, 512, 272, xdtype)
    check(mo, cuda_dev, w, x, TOL_F16 if xdtype == torch.float16 else TOL)


@pytest.mark.parametrize("K,N", [
    (32, 16), (32, 1), (96, 37), (64, 1000), (352, 130),        # ragged N, odd number of k blocks
    (256, 19008), (128, 40000), (64, 76000),                    # wide N: 4-, 2- and 1-way k split
])
def test_decode_ragged_shapes(mo, cuda_dev, K, N):
    w, x = make_case(K + N, 5, K, N, torch.float16)
    check(mo, cuda_dev, w, x, TOL_F16)


def test_config1(mo, cuda_dev):
    w, x = make_case(1001, 1, 4096, 4096, torch.float16)
    err = check(mo, cuda_dev, w, x, TOL_F16)
    print(f"config1 rel-L2 {err:.2e}")


@pytest.mark.parametrize("K,N", [(4096, 4096), (4096, 11008), (11008, 4096)])
@pytest.mark.parametrize("M", [1, 4, 16])
def test_config2_llama7b_decode(mo, cuda_dev, K, N, M):
    w, x = make_case(1002 + M, M, K, N, torch.float16)
    check(mo, cuda_dev, w, x, TOL_F16)


@pytest.mark.parametrize("M", [1, 128])
@pytest.mark.parametrize("K,N", [(8192, 28672), (28672, 8192)])
def test_config4_llama70b_column_sample(mo, cuda_dev, K, N, M):
    """Full-size 70B-shaped layer at M = 1 and 128; the oracle is evaluated on a seeded sample of
    columns (and rows), since the CPU product over everything would take minutes."""
    g = torch.Generator().manual_seed(1004)
    w = (torch.randn(K, N, generator=g) * 0.015).half()
    x = torch.randn(M, K, generator=g).half()
    blocks = mo.quantize_ggml_q4_0(w.to(cuda_dev))
    y = mo.matmul_ggml_q4_0(x.to(cuda_dev), blocks)
    cols = torch.randperm(N, generator=g)[:1024 if M == 1 else 256].sort().values
    rows = torch.arange(M) if M == 1 else torch.randperm(M, generator=g)[:16].sort().values
    ref = c_oracle.matmul_f32(x[rows].contiguous(), blocks[:, cols.to(cuda_dev)].cpu().contiguous())
    assert orc.rel_l2(y[rows.to(cuda_dev)][:, cols.to(cuda_dev)], ref) <= TOL_F16
    if M > 1:
        # checksum over the full output: column sums commute with the product
        wd = mo.dequantize_ggml_q4_0(blocks, torch.float32)
        assert orc.rel_l2(y.float().sum(0, keepdim=True), x.to(cuda_dev).float().sum(0, keepdim=True) @ wd) <= TOL
        return
    # linearity, a size-independent property of the full output: Y(2x) = 2 Y(x) up to output rounding
    y2 = mo.matmul_ggml_q4_0((2 * x).to(cuda_dev), blocks)
    assert orc.rel_l2(y2, 2 * y) <= 5e-4


def test_pdl_launch_matches_plain(mo, cuda_dev):
    from metalops_b200 import _cabi
    from metalops_b200 import quantization as Q
    w, x = make_case(7, 1, 4096, 4096, torch.float16)
    pre = mo.prepack_ggml_q4_0(mo.quantize_ggml_q4_0(w.to(cuda_dev)))
    xd = x.to(cuda_dev)
    torch.cuda.synchronize()
    plain = Q._matmul_prepacked(xd, pre)
    outs = [Q._matmul_prepacked(xd, pre, flags=_cabi.FLAG_PDL) for _ in range(8)]
    torch.cuda.synchronize()
    for o in outs:
        assert torch.equal(o, plain)


def test_fp32_activations_and_errors(mo, cuda_dev):
    w, x = make_case(11, 3, 128, 48, torch.float32)
    blocks = mo.quantize_ggml_q4_0(w.to(cuda_dev))
    y = mo.matmul_ggml_q4_0(x.to(cuda_dev), blocks)
    assert y.dtype == torch.float32
    assert orc.rel_l2(y, c_oracle.matmul_f32(x, blocks.cpu())) <= TOL
    with pytest.raises(AssertionError):
        mo.matmul_ggml_q4_0(torch.zeros(1, 96, dtype=torch.float16, device=cuda_dev), blocks)
    with pytest.raises(RuntimeError):
        mo.matmul_ggml_q4_0(torch.zeros(1, 128, dtype=torch.float16), blocks)          # CPU X
    with pytest.raises(RuntimeError):
        mo.matmul_ggml_q4_0(torch.zeros(2, 1, 128, dtype=torch.float16, device=cuda_dev), blocks)


def test_q4_linear_module(mo, cuda_dev):
    torch.manual_seed(3)
    lin = torch.nn.Linear(256, 48, bias=True).to(cuda_dev).half()
    ql = mo.Q4Linear.from_float(lin)
    assert sorted(ql.state_dict().keys()) == ["bias", "weight_blocks"]
    x = torch.randn(2, 5, 256, device=cuda_dev, dtype=torch.float16)
    y = ql(x)
    assert tuple(y.shape) == (2, 5, 48) and y.dtype == torch.float16
    blocks = ql.weight_blocks.cpu()
    ref = c_oracle.matmul_f32(x.reshape(-1, 256).cpu(), blocks) + lin.bias.float().cpu()
    assert orc.rel_l2(y.reshape(-1, 48), ref) <= TOL_F16          # bias enters before the single rounding
    assert torch.equal(blocks, c_oracle.quantize(lin.weight.data.t().contiguous().cpu()))
    # checkpoint round trip: a fresh module loads the state dict and gives the same output
    fresh = mo.Q4Linear(256, 48, dtype=torch.float16, device=cuda_dev)
    fresh.load_state_dict(ql.state_dict())
    assert torch.equal(fresh(x), y)
    # prefill-sized batch through the tcgen05 kernel, bias included
    xb = torch.randn(70, 256, device=cuda_dev, dtype=torch.bfloat16)
    refb = c_oracle.matmul_f32(xb.cpu(), blocks) + lin.bias.float().cpu()
    assert orc.rel_l2(ql(xb), refb) <= TOL


# ---------------------------------------------------------------------------------------
# prefill kernel (tcgen05 / TMEM)
# ---------------------------------------------------------------------------------------

def check_gemm(mo, dev, w, x, tol):
    from metalops_b200 import quantization as Q
    err = check(mo, dev, w, x, tol, kernel="gemm")
    assert Q.wait_status(dev) == 0
    return err


@pytest.mark.parametrize("M", [17, 63, 64, 65, 128, 129, 300])
@pytest.mark.parametrize("xdtype", [torch.float16, torch.bfloat16])
def test_gemm_m_edges(mo, cuda_dev, M, xdtype):
    w, x = make_case(200 + M, M, 512, 512, xdtype)
    check_gemm(mo, cuda_dev, w, x, TOL_F16 if xdtype == torch.float16 else TOL)


@pytest.mark.parametrize("K,N", [(32, 8), (64, 256), (96, 40), (352, 1000), (4096, 264), (128, 37)])
def test_gemm_ragged_shapes(mo, cuda_dev, K, N):
    w, x = make_case(K * 3 + N, 70, K, N, torch.bfloat16)
    check_gemm(mo, cuda_dev, w, x, TOL)


def test_gemm_single_row_through_prefill_kernel(mo, cuda_dev):
    w, x = make_case(31, 1, 256, 512, torch.float16)
    check_gemm(mo, cuda_dev, w, x, TOL_F16)


@pytest.mark.parametrize("xdtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("M,K,N", [
    (1, 64, 16), (17, 32, 8), (129, 96, 48),          # one k-tile, half a k-tile, an odd number of k-tiles
    (256, 448, 520), (257, 192, 130), (300, 1056, 1000),   # row-tile boundaries: 256, 2 x 144, 2 x 160 rows
    (513, 2080, 272), (1000, 320, 4112), (2048, 4096, 384),
    (200, 28672, 256),                                     # 224 stages per item
])
def test_persistent_prefill_kernel_forced(mo, cuda_dev, M, K, N, xdtype):
    """The persistent kernel (items of 128 columns x up to 256 rows) at any M: stages of one and two
    k-tiles, partial panels, partial row tiles; bitwise equal to what the dispatching entry gives."""
    from metalops_b200 import quantization as Q
    w, x = make_case(M + K + N, M, K, N, xdtype)
    tol = TOL_F16 if xdtype == torch.float16 else TOL
    check(mo, cuda_dev, w, x, tol, kernel="gemm_wt")
    assert Q.wait_status(cuda_dev) == 0
    blocks = mo.quantize_ggml_q4_0(w.to(cuda_dev))
    pre = mo.prepack_ggml_q4_0(blocks)
    g = torch.Generator().manual_seed(M)
    add = torch.randn(M, N, generator=g).to(cuda_dev)
    ya = Q._matmul_prepacked(x.to(cuda_dev), pre, kernel="gemm_wt", addend=add, flags=_cabi_flags().FLAG_ACT_SILU)
    v = c_oracle.matmul_f32(x, blocks.cpu()) + add.cpu()
    assert orc.rel_l2(ya, v / (1.0 + torch.exp(-v))) <= 2 * tol
    yb = Q._matmul_prepacked(x.to(cuda_dev), pre, kernel="gemm_wt", addend=add[0].contiguous())
    assert orc.rel_l2(yb, c_oracle.matmul_f32(x, blocks.cpu()) + add[0].cpu()) <= tol
    assert Q.wait_status(cuda_dev) == 0


def _cabi_flags():
    from metalops_b200 import _cabi
    return _cabi


def test_golden_matmul_prefill(mo, cuda_dev):
    z = load_golden("q4_0_matmul.npz")
    x = golden_tensor(z, "b_m70.x")
    blocks = golden_tensor(z, "b_m70.blocks").to(cuda_dev)
    y = mo.matmul_ggml_q4_0(x.to(cuda_dev), blocks)
    assert orc.rel_l2(y, golden_tensor(z, "b_m70.y_fp32")) <= TOL
    assert orc.rel_l2(y, golden_tensor(z, "b_m70.y_public")) <= 2 * TOL


@pytest.mark.parametrize("M", [512, 2048])
def test_config3_prefill_with_outliers(mo, cuda_dev, M):
    """K=4096, N=14336, bf16 activations, 0.1 % outliers at +-0.5.  The oracle is evaluated on a
    seeded sample of 256 rows x 1024 columns; the full product is checked by a checksum
    identity: (1^T X) W must equal 1^T (X W) (column sums commute with the product)."""
    from metalops_b200 import quantization as Q
    w, x = make_case(1003, M, 4096, 14336, torch.bfloat16, outliers=0.001)
    blocks = mo.quantize_ggml_q4_0(w.to(cuda_dev))
    xd = x.to(cuda_dev)
    y = mo.matmul_ggml_q4_0(xd, blocks)
    assert Q.wait_status(cuda_dev) == 0
    g = torch.Generator().manual_seed(9)
    rows = torch.randperm(M, generator=g)[:256].sort().values
    cols = torch.randperm(14336, generator=g)[:1024].sort().values
    ref = c_oracle.matmul_f32(x[rows].contiguous(), blocks[:, cols.to(cuda_dev)].cpu().contiguous())
    err = orc.rel_l2(y[rows.to(cuda_dev)][:, cols.to(cuda_dev)], ref)
    assert err <= TOL, f"rel-L2 {err:.3e}"
    wd = mo.dequantize_ggml_q4_0(blocks, torch.float32)
    lhs = xd.float().sum(0, keepdim=True) @ wd            # [1, N] in fp32
    rhs = y.float().sum(0, keepdim=True)
    assert orc.rel_l2(rhs, lhs) <= TOL
    print(f"config3 M={M} rel-L2 {err:.2e}")


@pytest.mark.parametrize("M", [1, 2, 8, 32, 128, 512, 4096])
def test_config5_gemm_sweep(mo, cuda_dev, M):
    from metalops_b200 import quantization as Q
    w, x = make_case(1005 + M, M, 4096, 14336, torch.float16)
    blocks = mo.quantize_ggml_q4_0(w.half().to(cuda_dev))
    y = mo.matmul_ggml_q4_0(x.to(cuda_dev), blocks)
    assert Q.wait_status(cuda_dev) == 0
    g = torch.Generator().manual_seed(M)
    rows = torch.randperm(M, generator=g)[:min(M, 32)].sort().values
    cols = torch.randperm(14336, generator=g)[:2048].sort().values
    ref = c_oracle.matmul_f32(x[rows].contiguous(), blocks[:, cols.to(cuda_dev)].cpu().contiguous())
    assert orc.rel_l2(y[rows.to(cuda_dev)][:, cols.to(cuda_dev)], ref) <= TOL_F16


@pytest.mark.parametrize("xdtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("M,K,N", [(17, 512, 128), (33, 96, 48), (64, 4096, 1000), (100, 1056, 200), (128, 2048, 4112),
                                   (20, 4096, 4096), (128, 11008, 4096)])
def test_small_batch_tensor_memory_kernel(mo, cuda_dev, M, K, N, xdtype):
    """17..128 rows run on the tensor-memory kernel (weights as the tcgen05 A operand, k split over a
    thread-block cluster): tolerance, bitwise repeatability, no bounded wait gave up.  Covers row
    counts that are not multiples of 16, column tails, an odd number of 32-k blocks, cluster sizes
    1..8 and agreement with the decode kernel on the first 16 rows."""
    from metalops_b200 import quantization as Q
    w, x = make_case(6000 + M + K + N, M, K, N, xdtype)
    blocks = mo.quantize_ggml_q4_0(w.to(cuda_dev))
    pre = mo.prepack_ggml_q4_0(blocks)
    y = Q._matmul_prepacked(x.to(cuda_dev), pre, kernel="gemm")
    assert Q.wait_status(cuda_dev) == 0
    ref = c_oracle.matmul_f32(x, blocks.cpu())
    assert torch.isfinite(y).all()
    assert orc.rel_l2(y, ref) <= TOL
    y2 = Q._matmul_prepacked(x.to(cuda_dev), pre, kernel="gemm")
    assert torch.equal(y, y2), "two runs differ bitwise"
    y16 = Q._matmul_prepacked(x[:16].to(cuda_dev), pre, kernel="gemv")
    assert orc.rel_l2(y[:16], y16.float().cpu()) <= TOL


def test_quantize_and_matmul_under_inference_mode(mo, cuda_dev):
    """Inference tensors keep no version counter; the cache of the streaming-layout copy must not
    depend on one."""
    w, x = make_case(77, 3, 256, 80, torch.float16)
    with torch.inference_mode():
        blocks = mo.quantize_ggml_q4_0(w.to(cuda_dev))
        y = mo.matmul_ggml_q4_0(x.to(cuda_dev), blocks)
        lin = mo.Q4Linear.from_float(torch.nn.Linear(256, 80).to(cuda_dev))
        lin(x.to(cuda_dev).float())
    assert orc.rel_l2(y, c_oracle.matmul_f32(x, blocks.cpu())) <= TOL_F16
    # a blocks tensor that arrives without a cached copy (e.g. from a checkpoint), created in inference mode
    with torch.inference_mode():
        fresh = blocks.clone()
        assert torch.equal(mo.matmul_ggml_q4_0(x.to(cuda_dev), fresh), y)


def test_both_activation_flags_are_rejected(mo, cuda_dev):
    from metalops_b200 import _cabi
    lib = _cabi.load()
    w, x = make_case(5, 1, 64, 32, torch.float16)
    pre = mo.prepack_ggml_q4_0(mo.quantize_ggml_q4_0(w.to(cuda_dev)))
    xd, y = x.to(cuda_dev), torch.empty(1, 32, dtype=torch.float16, device=cuda_dev)
    both = _cabi.FLAG_ACT_SILU | _cabi.FLAG_ACT_GELU
    for fn in (lib.q4b_gemv, lib.q4b_gemm, lib.q4b_matmul):
        assert fn(xd.data_ptr(), _cabi.F16, 1, 64, pre.data.data_ptr(), 64, 32, y.data_ptr(), 32, both, None) == _cabi.ERR_ARG


def test_bias_row_vector_addend_all_kernels(mo, cuda_dev):
    """A bias enters the epilogues as one fp32 row (leading dimension 0), not as an [M, N] tensor."""
    from metalops_b200 import quantization as Q
    g = torch.Generator().manual_seed(12)
    K, N = 512, 272
    w = torch.randn(K, N, generator=g) * 0.05
    bias = torch.randn(N, generator=g)
    blocks = mo.quantize_ggml_q4_0(w.to(cuda_dev))
    pre = mo.prepack_ggml_q4_0(blocks)
    for M in (1, 5, 12, 40, 200):
        x = torch.randn(M, K, generator=g).half()
        y = Q._matmul_prepacked(x.to(cuda_dev), pre, addend=bias.to(cuda_dev))
        ref = c_oracle.matmul_f32(x, blocks.cpu()) + bias
        assert orc.rel_l2(y, ref) <= TOL_F16, M
