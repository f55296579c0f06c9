"""GPU parity of the two side entrances of the INT4 path: the group-wise INT8 matmul (against
reference-generated fixtures and the oracle) and the GGML-tool conventions (scale rule and
split-half storage order, bit for bit against the oracle; products through the ordinary kernels)."""
import pytest
import torch

from conftest import golden_tensor, load_golden
from oracle import q4_0_oracle as orc

pytestmark = pytest.mark.gpu
TOL = 5e-3


@pytest.fixture(scope="module")
def mo(cuda_dev):
    import metalops_b200
    assert metalops_b200.has_native_kernels()
    return metalops_b200


@pytest.mark.parametrize("name,gs", [("g128_h", 128), ("g64_b", 64), ("g128_ragged_f", 128)])
def test_matmul_int8_against_reference_fixture(mo, cuda_dev, name, gs):
    z = load_golden("int8_groupwise.npz")
    x, w_q = golden_tensor(z, f"{name}.x"), golden_tensor(z, f"{name}.w_q")
    scales, zeros, y_ref = golden_tensor(z, f"{name}.scales"), golden_tensor(z, f"{name}.zeros"), golden_tensor(z, f"{name}.y")
    y = mo.matmul_int8(x.to(cuda_dev), w_q.to(cuda_dev), scales.to(cuda_dev), zeros.to(cuda_dev), gs)
    assert y.dtype == x.dtype and tuple(y.shape) == tuple(y_ref.shape)
    fp32 = orc.matmul_int8_fp32(x, w_q, scales, zeros, gs)
    assert orc.rel_l2(y, fp32) <= TOL
    # and no further from the reference's own result than that result is from fp32
    assert orc.rel_l2(y, y_ref) <= max(2 * orc.rel_l2(y_ref, fp32), 1e-3)


@pytest.mark.parametrize("M,K,N,gs,dt", [(1, 4096, 4096, 128, torch.float16), (7, 1000, 333, 100, torch.bfloat16),
                                         (33, 512, 130, 64, torch.float16), (1, 96, 5, 32, torch.float16)])
def test_matmul_int8_shapes(mo, cuda_dev, M, K, N, gs, dt):
    g = torch.Generator().manual_seed(M + K + N)
    w_q = torch.randint(-128, 128, (K, N), generator=g, dtype=torch.int16).to(torch.int8)
    ng = (K + gs - 1) // gs
    scales = (torch.rand(ng, N, generator=g) * 0.01 + 0.001).to(dt)
    zeros = (torch.randn(ng, N, generator=g) * 10.0).to(dt)
    x = torch.randn(M, K, generator=g).to(dt)
    y = mo.matmul_int8(x.to(cuda_dev), w_q.to(cuda_dev), scales.to(cuda_dev), zeros.to(cuda_dev), gs)
    assert orc.rel_l2(y, orc.matmul_int8_fp32(x, w_q, scales, zeros, gs)) <= TOL
    assert torch.equal(y, mo.matmul_int8(x.to(cuda_dev), w_q.to(cuda_dev), scales.to(cuda_dev), zeros.to(cuda_dev), gs))


@pytest.mark.parametrize("dt", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("layout", ["kn", "nk"])
def test_ggml_scale_rule_bit_exact(mo, cuda_dev, dt, layout):
    g = torch.Generator().manual_seed(31)
    K, N = 256, 77
    w = (torch.randn(K, N, generator=g) * 0.02).to(dt)
    w[32:64, 3] = 0                                        # an all-zero block: d = 0, q = 8
    w[0:32, 5] = -w[0:32, 5].abs()                         # the extreme value is negative: d > 0
    w[64, 7], w[65, 7] = 0.5, -0.5                         # equal magnitudes: the first one sets the sign
    wd = w.to(cuda_dev)
    src = wd if layout == "kn" else wd.t().contiguous().t()
    blocks = mo.quantize_ggml_q4_0(src, scale_mode="ggml")
    want = orc.quantize_q4_0_ggml_rule(w)
    assert torch.equal(blocks.cpu(), want)
    assert blocks[1, 3].cpu().tolist() == [0, 0] + [0x88] * 16
    # the ordinary kernels multiply with it (negative d included)
    x = torch.randn(3, K, generator=g).half()
    y = mo.matmul_ggml_q4_0(x.to(cuda_dev), blocks)
    assert orc.rel_l2(y, orc.matmul_q4_0_fp32(x, want)) <= 1e-3
    # the rule quantizes about as well as the reference's own
    err = orc.rel_l2(orc.dequantize_q4_0(want, torch.float32), w.float())
    assert err < 0.15


def test_import_split_half_storage(mo, cuda_dev):
    g = torch.Generator().manual_seed(32)
    K, N = 160, 19
    w = torch.randn(K, N, generator=g) * 0.02
    blocks = orc.quantize_q4_0(w)
    raw = orc.ggml_split_half_from_blocks(blocks)             # as another tool would have stored it
    assert tuple(raw.shape) == (N, K // 32, 18)
    assert torch.equal(orc.blocks_from_ggml_split_half(raw), blocks)
    got = mo.import_ggml_q4_0(raw.to(cuda_dev))
    assert torch.equal(got.cpu(), blocks)
    x = torch.randn(1, K, generator=g).half()
    assert orc.rel_l2(mo.matmul_ggml_q4_0(x.to(cuda_dev), got), orc.matmul_q4_0_fp32(x, blocks)) <= 1e-3
