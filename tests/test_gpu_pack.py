"""GPU parity of the quantize / repack / unpack / dequantize kernels (through the C ABI) against
the golden fixtures and both CPU oracles.  Everything here is bit-exact."""
import pytest
import torch

from conftest import golden_tensor, load_golden
from oracle import c_oracle
from oracle import q4_0_oracle as orc

pytestmark = pytest.mark.gpu

PACK_CASES = ["f32_a", "f32_b", "f32_c", "f16_a", "f16_b", "bf16_a", "bf16_b"]


@pytest.fixture(scope="module")
def mo(cuda_dev):
    import metalops_b200
    assert metalops_b200.has_native_kernels()
    return metalops_b200


def seeded_weight(seed, K, N, dtype, std=0.02, zero_frac=0.01):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(K, N, generator=g) * std
    if zero_frac:
        mask = torch.rand(K // 32, N, generator=g) < zero_frac
        w = w.view(K // 32, 32, N).masked_fill(mask.unsqueeze(1), 0.0).reshape(K, N)
    return w.to(dtype)


@pytest.mark.parametrize("name", PACK_CASES)
@pytest.mark.parametrize("layout", ["kn", "nk"])
def test_golden_pack(mo, cuda_dev, name, layout):
    z = load_golden("q4_0_pack.npz")
    w = golden_tensor(z, f"{name}.w")
    expect = golden_tensor(z, f"{name}.blocks")
    wd = w.to(cuda_dev)
    if layout == "nk":
        wd = wd.t().contiguous().t()          # same values, stored [N, K]
        assert not wd.is_contiguous()
    blocks = mo.quantize_ggml_q4_0(wd)
    assert blocks.dtype == torch.uint8 and tuple(blocks.shape) == tuple(expect.shape)
    assert torch.equal(blocks.cpu(), expect)
    # the streaming copy written by the same kernel holds the same information
    pre = mo.prepack_ggml_q4_0(blocks)
    assert torch.equal(mo.unpack_ggml_q4_0(pre).cpu(), expect)
    fresh = blocks.clone()                   # no cached prepack on the clone -> repack kernel runs
    pre2 = mo.prepack_ggml_q4_0(fresh)
    assert pre2 is not pre
    assert torch.equal(pre2.data.cpu(), pre.data.cpu())


@pytest.mark.parametrize("name", PACK_CASES)
def test_golden_dequantize(mo, cuda_dev, name):
    z = load_golden("q4_0_pack.npz")
    blocks = golden_tensor(z, f"{name}.blocks").to(cuda_dev)
    assert torch.equal(mo.dequantize_ggml_q4_0(blocks, torch.float32).cpu(), golden_tensor(z, f"{name}.deq_f32"))
    out16 = mo.dequantize_ggml_q4_0(blocks)
    assert out16.dtype == torch.float16
    assert torch.equal(out16.cpu(), golden_tensor(z, f"{name}.deq_f16"))
    assert torch.equal(mo.dequantize_ggml_q4_0(blocks, torch.bfloat16).cpu(),
                       orc.dequantize_q4_0(blocks.cpu(), torch.bfloat16))


@pytest.mark.parametrize("K,N,dtype", [
    (4096, 4096, torch.float32),       # config 1
    (4096, 1000, torch.float16),       # N not a multiple of the 128-column CTA tile
    (96, 7, torch.bfloat16),           # odd N, odd number of k blocks
    (32, 1, torch.float32),
    (352, 130, torch.float16),
    (11008, 512, torch.bfloat16),      # 344 blocks along k
    (256, 4099, torch.float32),        # odd N -> scalar loads, unaligned block rows
])
def test_seeded_pack_vs_c_oracle(mo, cuda_dev, K, N, dtype):
    w = seeded_weight(K * 7 + N, K, N, dtype)
    expect = c_oracle.quantize(w)
    for wd in (w.to(cuda_dev), w.to(cuda_dev).t().contiguous().t()):
        blocks = mo.quantize_ggml_q4_0(wd)
        assert torch.equal(blocks.cpu(), expect)
        assert torch.equal(mo.unpack_ggml_q4_0(mo.prepack_ggml_q4_0(blocks)).cpu(), expect)
    assert torch.equal(mo.dequantize_ggml_q4_0(blocks, torch.float32).cpu(), c_oracle.dequantize_f32(expect))


def test_config5_full_size_pack(mo, cuda_dev):
    """fp16 nn.Linear-layout weight 14336 x 4096 with 1 % all-zero blocks, packed in place from
    the [N, K] storage; must equal packing the transposed contiguous copy, and the C oracle."""
    g = torch.Generator().manual_seed(1005)
    N, K = 14336, 4096
    wl = (torch.randn(N, K, generator=g) * 0.02).half()
    mask = torch.rand(N, K // 32, generator=g) < 0.01
    wl = wl.view(N, K // 32, 32).masked_fill(mask.unsqueeze(2), 0.0).reshape(N, K)
    wl_d = wl.to(cuda_dev)
    a = mo.quantize_ggml_q4_0(wl_d.t())                   # read in place, [N, K] kernel
    b = mo.quantize_ggml_q4_0(wl_d.t().contiguous())      # [K, N] kernel
    assert torch.equal(a, b)
    assert torch.equal(mo.prepack_ggml_q4_0(a).data, mo.prepack_ggml_q4_0(b).data)
    expect = c_oracle.quantize(wl.t().contiguous())
    assert torch.equal(a.cpu(), expect)
    zero_block = torch.tensor([0x00, 0x3C] + [0x88] * 16, dtype=torch.uint8)
    kb, n = torch.nonzero(mask.t())[0].tolist()
    assert torch.equal(a[kb, n].cpu(), zero_block)
    # size-independent property: re-quantizing the dequantized weight reproduces the nibbles
    deq = mo.dequantize_ggml_q4_0(a, torch.float32)
    again = mo.quantize_ggml_q4_0(deq)
    assert torch.equal(again[:, :, 2:], a[:, :, 2:])


def test_errors(mo, cuda_dev):
    with pytest.raises(AssertionError):
        mo.quantize_ggml_q4_0(torch.zeros(48, 4, device=cuda_dev))
    with pytest.raises(RuntimeError):
        mo.quantize_ggml_q4_0(torch.zeros(32, 4))                        # CPU tensor: no fallback
    with pytest.raises(RuntimeError):
        mo.dequantize_ggml_q4_0(torch.zeros(1, 4, 17, dtype=torch.uint8, device=cuda_dev))
    with pytest.raises(RuntimeError):
        mo.quantize_ggml_q4_0(torch.zeros(32, 4, dtype=torch.float64, device=cuda_dev))
