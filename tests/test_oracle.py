"""Pins both CPU oracles (torch restatement and plain C) to fixtures produced by the reference
module itself (tests/golden/make_golden.py).  Everything here is bit-exact unless noted."""
import numpy as np
import pytest
import torch

from conftest import golden_tensor, load_golden
from oracle import c_oracle
from oracle import q4_0_oracle as orc

PACK_CASES = ["f32_a", "f32_b", "f32_c", "f16_a", "f16_b", "bf16_a", "bf16_b"]


@pytest.fixture(scope="module")
def pack():
    return load_golden("q4_0_pack.npz")


@pytest.mark.parametrize("name", PACK_CASES)
def test_pack_bit_exact_torch(pack, name):
    w = golden_tensor(pack, f"{name}.w")
    assert torch.equal(orc.quantize_q4_0(w), golden_tensor(pack, f"{name}.blocks"))


@pytest.mark.parametrize("name", PACK_CASES)
def test_pack_bit_exact_c(pack, name):
    w = golden_tensor(pack, f"{name}.w")
    assert torch.equal(c_oracle.quantize(w), golden_tensor(pack, f"{name}.blocks"))


@pytest.mark.parametrize("name", PACK_CASES)
def test_unpack_bit_exact(pack, name):
    blocks = golden_tensor(pack, f"{name}.blocks")
    ref32 = golden_tensor(pack, f"{name}.deq_f32")
    assert torch.equal(orc.dequantize_q4_0(blocks, torch.float32), ref32)
    assert torch.equal(c_oracle.dequantize_f32(blocks), ref32)
    assert torch.equal(orc.dequantize_q4_0(blocks), golden_tensor(pack, f"{name}.deq_f16"))


def test_zero_block_bytes():
    blocks = orc.quantize_q4_0(torch.zeros(32, 3))
    expect = torch.tensor([0x00, 0x3C] + [0x88] * 16, dtype=torch.uint8)
    assert torch.equal(blocks[0, 1], expect)
    assert torch.equal(c_oracle.quantize(torch.zeros(32, 3))[0, 2], expect)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_c_equals_torch_on_larger_seeded(dtype):
    g = torch.Generator().manual_seed(77)
    w = (torch.randn(512, 257, generator=g) * 0.02).to(dtype)
    w[64:96, 5] = 0
    a, b = orc.quantize_q4_0(w), c_oracle.quantize(w)
    assert torch.equal(a, b)
    q = orc.unpack_q4_0(a)[1]
    assert int(q.min()) >= 1 and int(q.max()) <= 15          # the reference never emits q=0


def test_roundtrip_bound():
    g = torch.Generator().manual_seed(5)
    w = torch.randn(256, 64, generator=g) * 0.02
    blocks = orc.quantize_q4_0(w)
    d, _ = orc.unpack_q4_0(blocks)
    err = (orc.dequantize_q4_0(blocks, torch.float32) - w).abs().view(8, 32, 64)
    bound = d.float().unsqueeze(1) * 0.5 * 1.002 + 1e-9        # |w - w^| <= d/2 (+ fp16 scale rounding)
    assert bool((err <= bound).all())


def test_k_must_be_multiple_of_32():
    with pytest.raises(AssertionError):
        orc.quantize_q4_0(torch.zeros(48, 4))


MM_CASES = ["h_m1", "h_m5", "b_m16", "b_m70", "f_m3"]


@pytest.mark.parametrize("name", MM_CASES)
def test_matmul_against_reference_outputs(name):
    z = load_golden("q4_0_matmul.npz")
    x = golden_tensor(z, f"{name}.x")
    blocks = golden_tensor(z, f"{name}.blocks")
    y32 = golden_tensor(z, f"{name}.y_fp32")
    # same ops, same order -> bit-exact for the fp32 oracle; the public path goes through a
    # reduced-precision matmul whose blocking may differ, so it is compared by rel-L2
    assert torch.allclose(orc.matmul_q4_0_fp32(x, blocks), y32, rtol=1e-5, atol=1e-6)
    assert orc.rel_l2(c_oracle.matmul_f32(x, blocks), y32) < 1e-6
    assert orc.rel_l2(orc.matmul_q4_0_public(x, blocks), golden_tensor(z, f"{name}.y_public")) < 1e-6 \
        or x.dtype != torch.float32
    assert orc.rel_l2(golden_tensor(z, f"{name}.y_public"), y32) < 5e-3


@pytest.mark.parametrize("name", ["g128_f32", "g64_f32", "g128_f16", "g128_ragged"])
def test_groupwise_int4(name):
    z = load_golden("int4_groupwise.npz")
    gs = 64 if name.startswith("g64") else 128
    w = golden_tensor(z, f"{name}.w")
    packed, scales, zeros = orc.quantize_int4_groupwise(w, gs)
    assert torch.equal(packed, golden_tensor(z, f"{name}.packed"))
    assert torch.equal(scales, golden_tensor(z, f"{name}.scales"))
    assert torch.equal(zeros, golden_tensor(z, f"{name}.zeros"))
    deq = orc.dequantize_int4_groupwise(packed, scales, zeros, gs, torch.float32)
    # a constant fp16 group has scale clamp(0, 1e-8) -> 0 in fp16 and the reference yields NaN there
    assert torch.allclose(deq, golden_tensor(z, f"{name}.deq_f32"), rtol=0, atol=0, equal_nan=True)


def test_half_conversion_helpers_exhaustive():
    lib = c_oracle.lib()
    bits = torch.arange(0, 65536, dtype=torch.int32).to(torch.int16).view(torch.float16)
    f = bits.float()
    finite = torch.isfinite(f)
    for i in range(0, 65536, 97):
        if bool(finite[i]):
            assert lib.q4o_f32_to_f16_bits(float(f[i])) == (i & 0xFFFF)
            assert lib.q4o_f16_bits_to_f32(i) == float(f[i])
    g = torch.Generator().manual_seed(3)
    x = torch.randn(2000, generator=g) * torch.logspace(-9, 5, 2000)
    for v in x.tolist():
        vf = float(np.float32(v))
        assert lib.q4o_f32_to_f16_bits(vf) == int(np.float32(vf).astype(np.float16).view(np.uint16))
        assert lib.q4o_f32_to_bf16_bits(vf) == int(torch.tensor(vf).bfloat16().view(torch.int16)) & 0xFFFF


def test_int8_oracle_matches_reference_fixture():
    z = load_golden("int8_groupwise.npz")
    for name, gs in (("g128_h", 128), ("g64_b", 64), ("g128_ragged_f", 128)):
        x, w_q = golden_tensor(z, f"{name}.x"), golden_tensor(z, f"{name}.w_q")
        scales, zeros, y_ref = golden_tensor(z, f"{name}.scales"), golden_tensor(z, f"{name}.zeros"), golden_tensor(z, f"{name}.y")
        fp32 = orc.matmul_int8_fp32(x, w_q, scales, zeros, gs)
        assert orc.rel_l2(y_ref, fp32) <= 5e-3, name


def test_ggml_rule_and_split_half_order():
    """Known answers of the scale rule stated for configuration 1 and of the storage order the
    reference's own helper reads (quant_kernels.metal:1714-1731)."""
    w = torch.zeros(64, 2)
    w[:32, 0] = torch.arange(32, dtype=torch.float32) - 16.0        # extreme value -16 -> d = 2
    b = orc.quantize_q4_0_ggml_rule(w)
    assert b[0, 0, :2].view(torch.float16).item() == 2.0
    q = torch.stack([b[0, 0, 2:] & 0xF, b[0, 0, 2:] >> 4], dim=1).reshape(-1)
    assert q.tolist() == [min(15, max(0, int(torch.tensor((k - 16) / 2.0).round().item()) + 8)) for k in range(32)]
    assert b[1, 0].tolist() == [0, 0] + [0x88] * 16                  # all-zero block
    raw = orc.ggml_split_half_from_blocks(b)
    assert tuple(raw.shape) == (2, 2, 18)
    assert (raw[0, 0, 2] & 0xF) == q[0] and (raw[0, 0, 2] >> 4) == q[16]
    assert torch.equal(orc.blocks_from_ggml_split_half(raw), b)
