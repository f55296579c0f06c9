"""GPU parity of the single-row persistent decode kernel (q4b_gemv_grouped, q4b_chain_* through
ctypes) against the CPU oracle: every product within 5e-3 rel-L2 of dequantise-then-fp32-matmul on
the input the stage really saw, bitwise repeatable, hand-over between stages included."""
import ctypes
import math

import pytest
import torch

from oracle import c_oracle
from oracle import q4_0_oracle as orc

pytestmark = pytest.mark.gpu

TOL = 5e-3
TOL_F16 = 1e-3


@pytest.fixture(scope="module")
def mo(cuda_dev):
    import metalops_b200
    assert metalops_b200.has_native_kernels()
    return metalops_b200


def quantized(mo, dev, seed, K, N, std=0.02):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(K, N, generator=g) * std
    blocks = mo.quantize_ggml_q4_0(w.to(dev))
    return blocks, mo.prepack_ggml_q4_0(blocks)


def oracle_row(x_row, blocks, alpha=1.0, addend=None, act=None):
    """fp32 oracle of one product of a stage: act(alpha * (x . dequant(W)) + addend)."""
    y = c_oracle.matmul_f32(x_row.view(1, -1).cpu(), blocks.cpu()).view(-1).double() * alpha
    if addend is not None:
        y = y + addend.cpu().double()
    if act == "silu":
        y = y / (1.0 + torch.exp(-y))
    elif act == "gelu":
        y = y * 0.5 * (1.0 + torch.tanh(0.7978845608028654 * (y + 0.044715 * y ** 3)))
    return y.float()


@pytest.mark.parametrize("xdtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("K,Ns", [
    (4096, (4096, 4096, 4096)),          # q | k | v
    (4096, (11008, 11008)),              # gate | up
    (11008, (4096,)),                    # down: 172 k tiles, not a multiple of the 8-way split
    (96, (40,)),                         # odd number of 32-k blocks, ragged N
    (4128, (100, 16, 17, 1)),            # four products, odd k tiles, single column
    (32, (5,)),                          # one block: seven of the eight k-split warps have no share
])
def test_grouped_matches_oracle(mo, cuda_dev, K, Ns, xdtype):
    from metalops_b200 import decode as D
    from metalops_b200 import quantization as Q
    g = torch.Generator().manual_seed(K + len(Ns))
    x = torch.randn(K, generator=g).to(xdtype)
    ws = [quantized(mo, cuda_dev, 17 * K + i, K, N) for i, N in enumerate(Ns)]
    ys = D.matmul_ggml_q4_0_grouped(x.to(cuda_dev), [p for _, p in ws])
    assert Q.wait_status(cuda_dev) == 0
    tol = TOL_F16 if xdtype == torch.float16 else TOL
    for y, (blocks, _), N in zip(ys, ws, Ns):
        assert y.dtype == xdtype and tuple(y.shape) == (N,)
        assert torch.isfinite(y).all()
        err = orc.rel_l2(y, oracle_row(x, blocks))
        assert err <= tol, f"N={N}: rel-L2 {err:.3e}"
    again = D.matmul_ggml_q4_0_grouped(x.to(cuda_dev), [p for _, p in ws])
    assert all(torch.equal(a, b) for a, b in zip(ys, again)), "two runs differ bitwise"


def test_grouped_equals_separate_calls_bitwise(mo, cuda_dev):
    """The summation order depends on K only, so one launch over three weights and three launches
    over one weight each give the same bits."""
    from metalops_b200 import decode as D
    g = torch.Generator().manual_seed(5)
    x = torch.randn(4096, generator=g).half().to(cuda_dev)
    pres = [quantized(mo, cuda_dev, 900 + i, 4096, N)[1] for i, N in enumerate((4096, 1024, 11008))]
    together = D.matmul_ggml_q4_0_grouped(x, pres)
    for y, p in zip(together, pres):
        assert torch.equal(y, D.matmul_ggml_q4_0_grouped(x, [p])[0])


def test_grouped_epilogue_alpha_addend_activation(mo, cuda_dev):
    from metalops_b200 import decode as D
    g = torch.Generator().manual_seed(6)
    K = 1024
    x = torch.randn(K, generator=g).half()
    ws = [quantized(mo, cuda_dev, 40 + i, K, 272) for i in range(3)]
    bias = [torch.randn(272, generator=g), None, torch.randn(272, generator=g)]
    acts = ["silu", "gelu", None]
    alphas = [0.5, 2.0, -1.25]
    ys = D.matmul_ggml_q4_0_grouped(x.to(cuda_dev), [p for _, p in ws], alphas=alphas,
                                    addends=[b.to(cuda_dev) if b is not None else None for b in bias], acts=acts)
    for y, (blocks, _), b, a, al in zip(ys, ws, bias, acts, alphas):
        assert orc.rel_l2(y, oracle_row(x, blocks, al, b, a)) <= 2e-3


def build_layers(mo, dev, layers, xdtype, shapes, seed=77):
    """A chain shaped like decoder layers: q|k|v (x) -> o (v) -> gate|up (o) -> down (gate), the next
    layer reading `down`; alpha keeps the activations near unit variance."""
    from metalops_b200 import decode as D
    H, F = shapes
    g = torch.Generator().manual_seed(seed)
    x0 = torch.randn(H, generator=g).to(xdtype).to(dev)
    aH, aF = 1.0 / (0.02 * math.sqrt(H)), 1.0 / (0.02 * math.sqrt(F))
    ch = D.DecodeChain(xdtype, dev)
    graph, prev = [], x0                 # graph: (stage index, source, [(blocks, alpha)])
    for layer in range(layers):
        mk = lambda i, K, N: quantized(mo, dev, seed + 100 * layer + i, K, N)
        q, k, v, o, ga, up, dn = mk(0, H, H), mk(1, H, H), mk(2, H, H), mk(3, H, H), mk(4, H, F), mk(5, H, F), mk(6, F, H)
        s0 = ch.add_stage(prev, [q[1], k[1], v[1]], alphas=[aH] * 3)
        graph.append((s0, prev, [(q[0], aH), (k[0], aH), (v[0], aH)]))
        s1 = ch.add_stage((s0, 2), [o[1]], alphas=[aH])
        graph.append((s1, (s0, 2), [(o[0], aH)]))
        s2 = ch.add_stage((s1, 0), [ga[1], up[1]], alphas=[aH] * 2)
        graph.append((s2, (s1, 0), [(ga[0], aH), (up[0], aH)]))
        s3 = ch.add_stage((s2, 0), [dn[1]], alphas=[aF])
        graph.append((s3, (s2, 0), [(dn[0], aF)]))
        prev = (s3, 0)
    return ch.build(), x0, graph


@pytest.mark.parametrize("xdtype,shapes,layers", [
    (torch.float16, (512, 1376), 3),         # small: many stages have fewer tiles than workers
    (torch.bfloat16, (512, 1376), 2),
    (torch.float16, (4096, 11008), 2),       # the Llama-2-7B layer shapes
])
def test_chain_matches_oracle_stage_by_stage(mo, cuda_dev, xdtype, shapes, layers):
    from metalops_b200 import quantization as Q
    ch, x0, graph = build_layers(mo, cuda_dev, layers, xdtype, shapes)
    tol = TOL_F16 if xdtype == torch.float16 else TOL
    first = None
    for rep in range(3):                     # replays: the epoch of the hand-over words moves on
        outs = ch.run()
        assert Q.wait_status(cuda_dev) == 0
        flat = [t.clone() for st in outs for t in st]
        if first is None:
            first = flat
        else:
            assert all(torch.equal(a, b) for a, b in zip(first, flat)), "replay differs bitwise"
    for stage, src, prods in graph:
        x = x0 if isinstance(src, torch.Tensor) else outs[src[0]][src[1]]
        for p, (blocks, alpha) in enumerate(prods):
            y = outs[stage][p]
            assert torch.isfinite(y).all()
            err = orc.rel_l2(y, oracle_row(x, blocks, alpha))
            assert err <= tol, f"stage {stage} product {p}: rel-L2 {err:.3e}"


def test_chain_gated_mlp_input_transform(mo, cuda_dev):
    """down(silu(gate) * up): the product of two earlier outputs is formed while the input is loaded."""
    from metalops_b200 import decode as D
    from metalops_b200 import quantization as Q
    H, F = 768, 2048
    g = torch.Generator().manual_seed(3)
    x = torch.randn(H, generator=g).half().to(cuda_dev)
    ga, up, dn = quantized(mo, cuda_dev, 1, H, F), quantized(mo, cuda_dev, 2, H, F), quantized(mo, cuda_dev, 3, F, H)
    aH = 1.0 / (0.02 * math.sqrt(H))
    ch = D.DecodeChain(torch.float16, cuda_dev)
    s0 = ch.add_stage(x, [ga[1], up[1]], alphas=[aH, aH])
    s1 = ch.add_stage(((s0, 0), (s0, 1)), [dn[1]], xform="silu_mul")
    outs = ch.build().run()
    assert Q.wait_status(cuda_dev) == 0
    gate, upv = outs[s0][0].float().cpu(), outs[s0][1].float().cpu()
    h = gate / (1.0 + torch.exp(-gate)) * upv
    ref = c_oracle.matmul_f32(h.view(1, -1), dn[0].cpu()).view(-1)
    assert orc.rel_l2(outs[s1][0], ref) <= TOL_F16


def test_chain_argument_checks(mo, cuda_dev):
    from metalops_b200 import _cabi
    from metalops_b200 import decode as D
    lib = _cabi.load()
    pre = quantized(mo, cuda_dev, 9, 64, 32)[1]
    x = torch.zeros(64, dtype=torch.float16, device=cuda_dev)
    ch = D.DecodeChain(torch.float16, cuda_dev)
    s0 = ch.add_stage(x, [pre])
    with pytest.raises(RuntimeError):
        ch.add_stage((s0, 0), [pre])                      # output has 32 elements, K is 64
    with pytest.raises(ValueError):
        ch.add_stage((5, 0), [quantized(mo, cuda_dev, 10, 32, 32)[1]])
    st = (_cabi.ChainStage * 1)()
    assert lib.q4b_chain_workspace_bytes(st, 0) == 0
    assert lib.q4b_chain_build(st, 1, None, 0, None) == _cabi.ERR_ARG
    prod = (_cabi.ChainProduct * 1)()
    assert lib.q4b_gemv_grouped(x.data_ptr(), _cabi.F16, 64, prod, 1, 0, None) == _cabi.ERR_ARG     # null weights
    assert lib.q4b_gemv_grouped(x.data_ptr(), _cabi.F32, 64, prod, 1, 0, None) == _cabi.ERR_DTYPE
    assert lib.q4b_gemv_grouped(x.data_ptr(), _cabi.F16, 64, prod, 5, 0, None) == _cabi.ERR_ARG
