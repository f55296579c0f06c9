"""CPU oracle for metalcore's block_q4_0 INT4 path.  TEST INFRASTRUCTURE, NOT PRODUCT.

This module restates, on the CPU and with plain torch tensor ops, what the reference's
``packages/metalcore/src/metalcore/quantization.py`` computes for the q4_0 path.  It is
imported only by the tests, by the smoke check and by the CPU-baseline / reference arm of
the benchmark.  The shipped package never imports it: the product path is CUDA only.

Parity status: the reference ships no golden vector or known-answer test for any
quantization function (its test-suite never imports them), so parity is pinned instead
against outputs of the reference module itself: ``tests/golden/make_golden.py`` loads the
reference file by path, runs it on seeded inputs and stores the results as the committed
fixtures ``tests/golden/*.npz``; ``tests/test_oracle.py`` checks this restatement (and the
independent C restatement in ``q4_0_oracle.c``) against those fixtures bit for bit.

Block format (quantization.py:303-304, quant_kernels.metal:1703-1710): a block covers 32
consecutive k of one output column n and occupies 18 bytes: a little-endian fp16 scale d
followed by 16 bytes, byte j = q[2j] | q[2j+1] << 4.  The tensor layout is
``[K/32, N, 18]`` uint8.
"""
from __future__ import annotations

import torch

QK = 32          # weights per block           (quantization.py:303)
BLOCK_BYTES = 18  # 2-byte scale + 16 nibble bytes (quantization.py:304)


def quantize_q4_0(weight: torch.Tensor) -> torch.Tensor:
    """Pack ``weight [K, N]`` (fp32 / fp16 / bf16) into ``[K/32, N, 18]`` uint8.

    Follows quantization.py:328-371.  Every arithmetic step below is a separate torch op in
    the weight's own dtype, exactly as in the reference, so that fp16 and bf16 inputs round
    after each step (amax/7, w/d, +8) the way the reference does:
      d  = amax(|w|) / 7          ; d = 1 wherever ``d > 0`` is false (zero block, NaN)
      q  = clamp(round_half_even(w / d + 8), 0, 15)   with the UNROUNDED d of that dtype
      stored scale = fp16(d)      (quantization.py:355, taken after q was computed)
      byte j = q[2j] | q[2j+1] << 4   (quantization.py:364-369)
    """
    if weight.dim() != 2:
        raise ValueError("weight must be [K, N]")
    K, N = weight.shape
    if K % QK:
        raise AssertionError(f"K ({K}) must be divisible by {QK}")
    nb = K // QK
    w = weight.contiguous().view(nb, QK, N)
    amax = w.abs().amax(dim=1)
    d = amax / 7.0
    d = torch.where(d > 0, d, torch.ones_like(d))
    q = (w / d.unsqueeze(1) + 8.0).round().clamp(0, 15).to(torch.uint8)      # [nb, 32, N]
    out = torch.empty((nb, N, BLOCK_BYTES), dtype=torch.uint8)
    out[:, :, 0:2] = d.to(torch.float16).contiguous().view(torch.uint8).view(nb, N, 2)
    qn = q.transpose(1, 2)                                                    # [nb, N, 32]
    out[:, :, 2:] = qn[:, :, 0::2] | (qn[:, :, 1::2] << 4)
    return out


def unpack_q4_0(blocks: torch.Tensor):
    """Split ``[K/32, N, 18]`` blocks into (d fp16 ``[K/32, N]``, q int8 ``[K/32, N, 32]``)."""
    nb, N, bb = blocks.shape
    if bb != BLOCK_BYTES:
        raise ValueError("last dim of blocks must be 18")
    d = blocks[:, :, 0:2].contiguous().view(torch.float16).view(nb, N)
    qs = blocks[:, :, 2:]
    q = torch.empty((nb, N, QK), dtype=torch.int8)
    q[:, :, 0::2] = (qs & 0x0F).to(torch.int8)
    q[:, :, 1::2] = (qs >> 4).to(torch.int8)
    return d, q


def dequantize_q4_0(blocks: torch.Tensor, dtype: torch.dtype | None = None) -> torch.Tensor:
    """``W[k, n] = (q - 8) * float(d)`` in fp32, then cast (quantization.py:391-419)."""
    if dtype is None:
        dtype = torch.float16
    d, q = unpack_q4_0(blocks)
    nb, N = d.shape
    w = (q.float() - 8.0) * d.float().unsqueeze(2)            # [nb, N, 32]
    return w.permute(0, 2, 1).reshape(nb * QK, N).to(dtype)


def matmul_q4_0_public(X: torch.Tensor, blocks: torch.Tensor) -> torch.Tensor:
    """What the reference's public entry returns off-MPS (quantization.py:440-454):
    dequantise to X's dtype, then a torch matmul in that dtype."""
    K = blocks.shape[0] * QK
    assert X.shape[1] == K, f"X K dim ({X.shape[1]}) must match weight K ({K})"
    return X @ dequantize_q4_0(blocks, X.dtype)


def matmul_q4_0_fp32(X: torch.Tensor, blocks: torch.Tensor, n_chunk: int = 4096) -> torch.Tensor:
    """The accuracy oracle: dequantise to fp32 and multiply in fp32.  Chunked over N so the
    70B-shaped layers do not need the whole fp32 weight at once."""
    N = blocks.shape[1]
    Xf = X.float()
    out = torch.empty((X.shape[0], N), dtype=torch.float32)
    for n0 in range(0, N, n_chunk):
        n1 = min(N, n0 + n_chunk)
        out[:, n0:n1] = Xf @ dequantize_q4_0(blocks[:, n0:n1].contiguous(), torch.float32)
    return out


def rel_l2(y: torch.Tensor, ref: torch.Tensor) -> float:
    """Relative L2 error ||y - ref|| / ||ref|| in fp64."""
    y = y.double().cpu()
    ref = ref.double().cpu()
    den = ref.norm().item()
    return (y - ref).norm().item() / (den if den > 0 else 1.0)


# ---------------------------------------------------------------------------------------
# Group-wise asymmetric INT4 format (quantization.py:26-239): weight_packed [K/2, N],
# scales / zeros [ceil(K/group), N].  Byte r of column n holds k=2r (low) and k=2r+1 (high).
# ---------------------------------------------------------------------------------------

def quantize_int4_groupwise(weight: torch.Tensor, group_size: int = 128):
    """Vectorised restatement of the double loop at quantization.py:61-90."""
    K, N = weight.shape
    ng = (K + group_size - 1) // group_size
    packed = torch.zeros((K // 2, N), dtype=torch.uint8)
    scales = torch.zeros((ng, N), dtype=weight.dtype)
    zeros = torch.zeros((ng, N), dtype=weight.dtype)
    for g in range(ng):
        k0, k1 = g * group_size, min((g + 1) * group_size, K)
        grp = weight[k0:k1]
        lo = grp.min(dim=0).values
        hi = grp.max(dim=0).values
        scale = ((hi - lo) / 15.0).clamp(min=1e-8)
        zero = -lo / scale
        scales[g], zeros[g] = scale, zero
        q = (grp / scale + zero).round().clamp(0, 15).to(torch.uint8)        # [k1-k0, N]
        even = q[0::2]
        odd = q[1::2]
        r0 = k0 // 2
        packed[r0:r0 + even.shape[0]] = even
        packed[r0:r0 + odd.shape[0]] |= odd << 4
    return packed, scales, zeros


def dequantize_int4_groupwise(packed, scales, zeros, group_size: int = 128, dtype=None):
    """``W[k] = ((q - zero) * scale)`` in fp32, cast per row (quantization.py:131-153)."""
    if dtype is None:
        dtype = torch.float16
    K = packed.shape[0] * 2
    q = torch.empty((K, packed.shape[1]), dtype=torch.float32)
    q[0::2] = (packed & 0x0F).float()
    q[1::2] = (packed >> 4).float()
    gi = torch.arange(K) // group_size
    return ((q - zeros[gi]) * scales[gi]).to(dtype)


# ---------------------------------------------------------------------------------------
# Group-wise INT8 weights (quantization.py:242-286): w_q int8 [K, N], scales / zeros
# [ceil(K/group), N]; W = (w_q - zero) * scale, Y = X @ W.
# ---------------------------------------------------------------------------------------

def dequantize_int8_groupwise(w_q: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor, group_size: int = 128) -> torch.Tensor:
    """fp32 W of the loop at quantization.py:277-284 (before its cast to X.dtype)."""
    gi = torch.arange(w_q.shape[0]) // group_size
    return (w_q.float() - zeros.float()[gi]) * scales.float()[gi]


def matmul_int8_fp32(X: torch.Tensor, w_q, scales, zeros, group_size: int = 128) -> torch.Tensor:
    return X.float() @ dequantize_int8_groupwise(w_q, scales, zeros, group_size)


# ---------------------------------------------------------------------------------------
# GGML-tool conventions (format provenance: quantization.py:292-304).  Scale rule as the build's
# configuration 1 states it: d = (value of largest magnitude) / -8, q = clamp(round(w / d) + 8, 0, 15);
# an all-zero block has d = 0 and q = 8.  fp32 arithmetic, ties to even (torch.round), the first
# value wins among equal magnitudes.  Original storage order (the one the reference's helper at
# quant_kernels.metal:1714-1731 reads): rows of K/32 blocks per output feature, byte j of a block =
# value j | value (j + 16) << 4.
# ---------------------------------------------------------------------------------------

def quantize_q4_0_ggml_rule(weight: torch.Tensor) -> torch.Tensor:
    """[K, N] -> uint8 [K/32, N, 18] in this build's (interleaved-nibble) layout."""
    K, N = weight.shape
    nb = K // QK
    w = weight.float().view(nb, QK, N)
    idx = w.abs().argmax(dim=1, keepdim=True)                 # first index of the maximum
    vmax = torch.gather(w, 1, idx)                            # [nb, 1, N]
    d = torch.where(vmax == 0, torch.zeros_like(vmax), vmax / -8.0)     # +0 for an all-zero block
    safe = torch.where(d == 0, torch.ones_like(d), d)
    q = torch.where(d == 0, torch.full_like(w, 8.0), ((w / safe).round() + 8.0).clamp(0, 15))
    q = q.to(torch.uint8).permute(0, 2, 1).contiguous()       # [nb, N, 32]
    out = torch.zeros((nb, N, BLOCK_BYTES), dtype=torch.uint8)
    out[:, :, 0:2] = d.squeeze(1).to(torch.float16).contiguous().view(torch.uint8).view(nb, N, 2)
    out[:, :, 2:] = q[:, :, 0::2] | (q[:, :, 1::2] << 4)
    return out


def ggml_split_half_from_blocks(blocks: torch.Tensor) -> torch.Tensor:
    """This build's [K/32, N, 18] -> the original storage [N, K/32, 18] (byte j = v[j] | v[j+16] << 4)."""
    nb, N, _ = blocks.shape
    qs = blocks[:, :, 2:]
    v = torch.empty((nb, N, QK), dtype=torch.uint8)
    v[:, :, 0::2] = qs & 0x0F
    v[:, :, 1::2] = qs >> 4
    raw = torch.empty((nb, N, BLOCK_BYTES), dtype=torch.uint8)
    raw[:, :, 0:2] = blocks[:, :, 0:2]
    raw[:, :, 2:] = v[:, :, :16] | (v[:, :, 16:] << 4)
    return raw.permute(1, 0, 2).contiguous()


def blocks_from_ggml_split_half(raw: torch.Tensor) -> torch.Tensor:
    """The inverse: original storage [N, K/32, 18] -> this build's [K/32, N, 18]."""
    N, nb, _ = raw.shape
    qs = raw[:, :, 2:]
    v = torch.cat([qs & 0x0F, qs >> 4], dim=2)                # values 0..15 then 16..31
    out = torch.empty((N, nb, BLOCK_BYTES), dtype=torch.uint8)
    out[:, :, 0:2] = raw[:, :, 0:2]
    out[:, :, 2:] = v[:, :, 0::2] | (v[:, :, 1::2] << 4)
    return out.permute(1, 0, 2).contiguous()
