// Shared definitions for the q4b200 kernels: the prepacked tile geometry, nibble helpers and
// the host-side checking macros.  Device code here is sm_100a only.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/q4b200.h"

namespace q4b {

constexpr int QK = 32;             // weights per q4_0 block
constexpr int BLOCK_BYTES = 18;    // interchange bytes per block
constexpr int TILE_N = 16;         // output columns per prepacked tile
constexpr int TILE_KB = 2;         // q4_0 blocks along k per prepacked tile (64 k)
constexpr int TILE_K = TILE_KB * QK;
constexpr int TILE_QS_BYTES = 512; // 32 slots x 16 bytes
constexpr int TILE_BYTES = 576;    // + 8 rows x 4 fp16 scales

__host__ __device__ inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
__host__ __device__ inline int64_t tiles_k(int64_t K) { return ceil_div(K, TILE_K); }
__host__ __device__ inline int64_t tiles_n(int64_t N) { return ceil_div(N, TILE_N); }

// Tiles are stored column-tile-major: all k tiles of 16 output columns are contiguous, so the
// decode kernel streams one long run per column tile.
__host__ __device__ inline size_t tile_offset(int64_t nt, int64_t ku, int64_t KU) {
    return (size_t)(nt * KU + ku) * TILE_BYTES;
}
// Position (16-byte slot index) inside a tile of the words belonging to column-in-octet g
// (0..7) and k-octet c (0..3).  The XOR makes both access patterns bank-conflict free when the
// tile sits in shared memory: the decode kernel's lane 4g+c, and the prefill kernel's lane
// 8c+g, each touch eight distinct 16-byte bank groups per quarter warp.
__host__ __device__ inline int slot_of(int g, int c) { return (g >> 1) * 8 + (g & 1) * 4 + (c ^ (g >> 1)); }
__host__ __device__ inline void slot_inverse(int p, int &g, int &c) {
    g = (p >> 3) * 2 + ((p >> 2) & 1);
    c = (p & 3) ^ (p >> 3);
}

// ---- nibble order ---------------------------------------------------------------------
// Interchange word (4 consecutive nibble bytes of a block): byte j = q[2j] | q[2j+1] << 4.
// Prepacked word: q0 | q2<<4 | q4<<8 | q6<<12 | q1<<16 | q3<<20 | q5<<24 | q7<<28, so that
// (word >> 4s) & 0x000F000F yields the consecutive pair (q[2s], q[2s+1]) in the two halves.
__host__ __device__ inline uint32_t interchange_to_prepacked_word(uint32_t w) {
    uint32_t lo = w & 0x0F0F0F0Fu;          // q0, q2, q4, q6 one per byte
    uint32_t hi = (w >> 4) & 0x0F0F0F0Fu;   // q1, q3, q5, q7 one per byte
    lo = (lo | (lo >> 4)) & 0x00FF00FFu;
    lo = (lo | (lo >> 8)) & 0x0000FFFFu;
    hi = (hi | (hi >> 4)) & 0x00FF00FFu;
    hi = (hi | (hi >> 8)) & 0x0000FFFFu;
    return lo | (hi << 16);
}
__host__ __device__ inline uint32_t prepacked_to_interchange_word(uint32_t p) {
    uint32_t lo = p & 0xFFFFu, hi = p >> 16;
    lo = (lo | (lo << 8)) & 0x00FF00FFu;
    lo = (lo | (lo << 4)) & 0x0F0F0F0Fu;
    hi = (hi | (hi << 8)) & 0x00FF00FFu;
    hi = (hi | (hi << 4)) & 0x0F0F0F0Fu;
    return lo | (hi << 4);
}
// eight q values (0..15), q[i] for k offset i, into a prepacked word
__device__ inline uint32_t pack_prepacked_word(const int *q) {
    return (uint32_t)q[0] | ((uint32_t)q[2] << 4) | ((uint32_t)q[4] << 8) | ((uint32_t)q[6] << 12) |
           ((uint32_t)q[1] << 16) | ((uint32_t)q[3] << 20) | ((uint32_t)q[5] << 24) |
           ((uint32_t)q[7] << 28);
}

// ---- register dequantisation ------------------------------------------------------------
// One prepacked word -> four packed pairs (q-8) as fp16x2 / bf16x2 bit patterns, pair s =
// (k offset 2s, 2s+1).  fp16 uses the "1024+q" and "64+q" mantissa tricks (one shift per
// word); bf16 has 7 mantissa bits so every pair but the first needs its own shift.
__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t orv) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));   // (a & b) | c
    return r;
}
__device__ __forceinline__ uint32_t hsub2_bits(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("sub.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t hmul2_bits(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("mul.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t bsub2_bits(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("sub.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t bmul2_bits(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("mul.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}

template <bool BF16>
__device__ __forceinline__ void dequant_word(uint32_t w, uint32_t (&h)[4]) {
    if constexpr (!BF16) {
        const uint32_t w8 = w >> 8;
        h[0] = hsub2_bits(lop3_and_or(w, 0x000F000Fu, 0x64006400u), 0x64086408u);    // 1024+q - 1032
        h[1] = hsub2_bits(lop3_and_or(w, 0x00F000F0u, 0x54005400u), 0x54805480u);    // 64+q   - 72
        h[2] = hsub2_bits(lop3_and_or(w8, 0x000F000Fu, 0x64006400u), 0x64086408u);
        h[3] = hsub2_bits(lop3_and_or(w8, 0x00F000F0u, 0x54005400u), 0x54805480u);
    } else {
        h[0] = bsub2_bits(lop3_and_or(w, 0x000F000Fu, 0x43004300u), 0x43084308u);    // 128+q - 136
        h[1] = bsub2_bits(lop3_and_or(w >> 4, 0x000F000Fu, 0x43004300u), 0x43084308u);
        h[2] = bsub2_bits(lop3_and_or(w >> 8, 0x000F000Fu, 0x43004300u), 0x43084308u);
        h[3] = bsub2_bits(lop3_and_or(w >> 12, 0x000F000Fu, 0x43004300u), 0x43084308u);
    }
}

// The same without the subtraction: pair s holds (OFF + q) with OFF = 1024 for pairs 0 and 2 and
// 64 for pairs 1 and 3 (fp16), or 128 for every pair (bf16).  The single-row decode kernel
// removes sum((OFF + 8) * x) once per 32-k block instead of subtracting per pair.
template <bool BF16>
__device__ __forceinline__ void dequant_word_biased(uint32_t w, uint32_t (&h)[4]) {
    if constexpr (!BF16) {
        const uint32_t w8 = w >> 8;
        h[0] = lop3_and_or(w, 0x000F000Fu, 0x64006400u);
        h[1] = lop3_and_or(w, 0x00F000F0u, 0x54005400u);
        h[2] = lop3_and_or(w8, 0x000F000Fu, 0x64006400u);
        h[3] = lop3_and_or(w8, 0x00F000F0u, 0x54005400u);
    } else {
        h[0] = lop3_and_or(w, 0x000F000Fu, 0x43004300u);
        h[1] = lop3_and_or(w >> 4, 0x000F000Fu, 0x43004300u);
        h[2] = lop3_and_or(w >> 8, 0x000F000Fu, 0x43004300u);
        h[3] = lop3_and_or(w >> 12, 0x000F000Fu, 0x43004300u);
    }
}

// A block's fp16 scale as a pair in the activations' type (bf16: rounded once from fp16).
template <bool BF16> __device__ __forceinline__ uint32_t scale_pair(uint16_t dbits) {
    if constexpr (BF16) {
        __nv_bfloat16 b = __float2bfloat16_rn(__half2float(__ushort_as_half(dbits)));
        uint32_t u = __bfloat16_as_ushort(b);
        return u | (u << 16);
    } else {
        return (uint32_t)dbits | ((uint32_t)dbits << 16);
    }
}

// ---- epilogue activation (flags Q4B_FLAG_ACT_*: 0 none, 1 SiLU, 2 tanh-GELU), applied to the fp32 sum ----
// Formulas of the reference's fused kernels (quant_kernels.metal:997, 1125-1131).
__host__ __device__ inline int act_of_flags(int flags) { return (flags >> 3) & 3; }
__device__ __forceinline__ float apply_act(float v, int act) {
    if (act == 1) return v / (1.0f + __expf(-v));
    if (act == 2) return v * 0.5f * (1.0f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
    return v;
}

// ---- host-side helpers ---------------------------------------------------------------
void set_cuda_error(cudaError_t e);
inline bool aligned(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

#define Q4B_CUDA_TRY(expr)                         \
    do {                                           \
        cudaError_t _e = (expr);                   \
        if (_e != cudaSuccess) {                   \
            ::q4b::set_cuda_error(_e);             \
            return Q4B_ERR_CUDA;                   \
        }                                          \
    } while (0)

// launch-time check of the last kernel launch (configuration errors only; never synchronises)
#define Q4B_LAUNCH_CHECK() Q4B_CUDA_TRY(cudaGetLastError())

}  // namespace q4b
