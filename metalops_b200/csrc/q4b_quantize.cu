// q4_0 quantize / pack, repack, unpack and dequantize kernels (HBM-bound byte work).
//
// quantize: replaces the torch pipeline of quantize_ggml_q4_0
// (packages/metalcore/src/metalcore/quantization.py:328-371).  The reference evaluates
// amax/7, w/d, +8 and round as separate tensor ops in the weight's dtype; for fp16 / bf16
// each op computes in fp32 and rounds to the narrow type.  RoundTo<T> reproduces exactly that,
// with IEEE division (or an equivalent proven on every operand pair, see BlockDivider) and ties-to-even
// rounding, so the bytes are identical.
#include "q4b_common.cuh"

namespace q4b {

template <typename T> struct RoundTo;
template <> struct RoundTo<float> {
    static __device__ __forceinline__ float r(float v) { return v; }
    static __device__ __forceinline__ float ld(const float *p) { return *p; }
};
template <> struct RoundTo<__half> {
    static __device__ __forceinline__ float r(float v) { return __half2float(__float2half_rn(v)); }
    static __device__ __forceinline__ float ld(const __half *p) { return __half2float(*p); }
};
template <> struct RoundTo<__nv_bfloat16> {
    static __device__ __forceinline__ float r(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
    static __device__ __forceinline__ float ld(const __nv_bfloat16 *p) { return __bfloat162float(*p); }
};

// Two values rounded to T and widened again.  The packed conversions (two floats -> half2 / bf16x2)
// and the widening add issue at full rate, where one-at-a-time float<->half conversions queue on the
// quarter-rate conversion unit, which bounded the 16-bit packers.
template <typename T> __device__ __forceinline__ void round_pair(float &a, float &b);
template <> __device__ __forceinline__ void round_pair<float>(float &, float &) {}
template <> __device__ __forceinline__ void round_pair<__half>(float &a, float &b) {
    const float2 f = __half22float2(__floats2half2_rn(a, b));
    a = f.x;
    b = f.y;
}
template <> __device__ __forceinline__ void round_pair<__nv_bfloat16>(float &a, float &b) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    const uint32_t u = *reinterpret_cast<const uint32_t *>(&h);
    a = __uint_as_float(u << 16);
    b = __uint_as_float(u & 0xFFFF0000u);
}
// round-half-to-even of t (|t| < 2^22) and clamp to [0, 15], as an integer: adding 1.5 * 2^23 leaves
// the rounded integer in the low mantissa bits (the same result as rintf + clamp + convert; NaN -> 0)
__device__ __forceinline__ int round_clamp_q(float t) {
    t = fminf(fmaxf(t, -1.0f), 16.0f);                 // keeps the sum in range; NaN becomes -1 -> 0 below
    const int q = __float_as_int(__fadd_rn(t, 12582912.0f)) - 0x4B400000;
    return min(max(q, 0), 15);
}

// v / d as the reference's division gives it (IEEE, round to nearest), for the many values of one block.
// For fp32 weights that is the division instruction sequence.  For fp16 / bf16 weights, whose d has at
// most 11 significant bits, the quotient comes from the correctly rounded reciprocal of d, computed once
// per block, and one fused correction step: q = v * r, e = fma(-q, d, v) (the exact remainder),
// q + e * r.  The 4-bit result of the whole pipeline (round to T, + 8, round to T, round half to even,
// clamp) is identical to the one through IEEE division for EVERY pair of fp16 and of bf16 operands with
// 1e-30 <= d <= 1e30 and |v| <= 16.5 d: tests/exact_division_check.c enumerates them.  Outside that range
// of d (bf16 scales near the fp32 denormals, an infinite block maximum) the division is used.
template <typename T> struct BlockDivider {
    float d, r;
    bool fast;
    __device__ __forceinline__ explicit BlockDivider(float d_) : d(d_), r(0.0f), fast(false) {
        if constexpr (sizeof(T) == 2) {
            fast = d_ >= 1e-30f && d_ <= 1e30f;
            r = __frcp_rn(fast ? d_ : 1.0f);
        }
    }
    __device__ __forceinline__ float operator()(float v) const {
        if constexpr (sizeof(T) == 2) {
            if (fast) {
                const float q = __fmul_rn(v, r);
                return __fmaf_rn(__fmaf_rn(-q, d, v), r, q);
            }
        }
        return __fdiv_rn(v, d);
    }
};

// Quantise the 32 values of one block.  Returns the fp16 scale bits and fills q[32].
template <typename T>
__device__ __forceinline__ uint16_t quantize_block(const float (&v)[QK], int (&q)[QK]) {
    float amax = 0.0f;
    bool nan = false;
#pragma unroll
    for (int i = 0; i < QK; ++i) {
        float a = fabsf(v[i]);
        nan |= (a != a);
        amax = fmaxf(amax, a);
    }
    float d = RoundTo<T>::r(__fdiv_rn(amax, 7.0f));   // quantization.py:341
    if (nan || !(d > 0.0f)) d = 1.0f;                 // quantization.py:342 (NaN amax fails d > 0)
    const BlockDivider<T> div(d);
#pragma unroll
    for (int i = 0; i < QK; i += 2) {
        float t0 = div(v[i]), t1 = div(v[i + 1]);     // quantization.py:347, one rounding per op
        round_pair<T>(t0, t1);
        t0 = __fadd_rn(t0, 8.0f);
        t1 = __fadd_rn(t1, 8.0f);
        round_pair<T>(t0, t1);
        q[i] = round_clamp_q(t0);                      // ties to even, as torch.round; NaN -> 0 (the
        q[i + 1] = round_clamp_q(t1);                  // reference's result is undefined there)
    }
    return __half_as_ushort(__float2half_rn(d));      // quantization.py:355
}

constexpr int QT_N = 128;        // columns per CTA
constexpr int QT_THREADS = 128;  // 2 blocks along k x 64 column pairs

// Copy `bytes` (even) from shared memory to global memory where both addresses are congruent
// modulo 16: 2-byte stores up to the first 16-byte boundary, 16-byte stores for the body.
__device__ __forceinline__ void copy_out_congruent(uint8_t *dst, const uint8_t *src, int bytes, int tid,
                                                   int nthreads) {
    int head = (int)((16 - (reinterpret_cast<uintptr_t>(dst) & 15)) & 15);
    if (head > bytes) head = bytes;
    const int body = (bytes - head) & ~15;
    const int tail = bytes - head - body;
    for (int i = tid * 2; i < head; i += nthreads * 2)
        *reinterpret_cast<uint16_t *>(dst + i) = *reinterpret_cast<const uint16_t *>(src + i);
    for (int i = tid * 16; i < body; i += nthreads * 16)
        *reinterpret_cast<uint4 *>(dst + head + i) = *reinterpret_cast<const uint4 *>(src + head + i);
    for (int i = tid * 2; i < tail; i += nthreads * 2)
        *reinterpret_cast<uint16_t *>(dst + head + body + i) =
            *reinterpret_cast<const uint16_t *>(src + head + body + i);
}

// Weight [K, N] (N contiguous).  CTA = one 64-k tile row (2 blocks) x 128 columns; each thread
// owns two adjacent columns of one block, reading 32 rows with one (vector) load per row.
template <typename T, bool VEC2>
__global__ void __launch_bounds__(QT_THREADS)
quantize_kn_kernel(const T *__restrict__ w, int64_t K, int64_t N, uint8_t *__restrict__ blocks,
                   uint8_t *__restrict__ prepacked) {
    __shared__ __align__(16) uint8_t s_blk[TILE_KB][QT_N * BLOCK_BYTES + 16];
    __shared__ __align__(16) uint8_t s_tile[QT_N / TILE_N][TILE_BYTES];

    const int tid = threadIdx.x;
    const int kbl = tid >> 6;
    const int nl = (tid & 63) * 2;
    const int64_t KB = K / QK;
    const int64_t NT = tiles_n(N);
    const int64_t ku = blockIdx.y;
    const int64_t kb = ku * TILE_KB + kbl;
    const int64_t n0 = (int64_t)blockIdx.x * QT_N;
    const int64_t n = n0 + nl;

    float v[2][QK];
    const bool kb_ok = kb < KB;
    const bool ok0 = kb_ok && n < N, ok1 = kb_ok && (n + 1) < N;
    if (VEC2 && ok1) {
        // N even here, so (k*N + n) is even and the pair load is aligned
#pragma unroll
        for (int i = 0; i < QK; ++i) {
            const T *p = w + (kb * QK + i) * N + n;
            if constexpr (sizeof(T) == 4) {
                float2 x = __ldg(reinterpret_cast<const float2 *>(p));
                v[0][i] = x.x;
                v[1][i] = x.y;
            } else {
                uint32_t x = __ldg(reinterpret_cast<const uint32_t *>(p));
                T lo, hi;
                *reinterpret_cast<uint16_t *>(&lo) = (uint16_t)(x & 0xFFFF);
                *reinterpret_cast<uint16_t *>(&hi) = (uint16_t)(x >> 16);
                v[0][i] = RoundTo<T>::ld(&lo);
                v[1][i] = RoundTo<T>::ld(&hi);
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < QK; ++i) {
            const T *p = w + (kb * QK + i) * N + n;
            v[0][i] = ok0 ? RoundTo<T>::ld(p) : 0.0f;
            v[1][i] = ok1 ? RoundTo<T>::ld(p + 1) : 0.0f;
        }
    }

    // where this CTA's interchange bytes start, per block row; the staging copy is shifted so
    // that shared and global addresses agree modulo 16
    const int shift0 = (int)((reinterpret_cast<uintptr_t>(blocks) + (size_t)((ku * TILE_KB) * N + n0) * BLOCK_BYTES) & 15);
    const int shift1 = (int)((reinterpret_cast<uintptr_t>(blocks) + (size_t)((ku * TILE_KB + 1) * N + n0) * BLOCK_BYTES) & 15);
    const int shift = kbl ? shift1 : shift0;

#pragma unroll
    for (int col = 0; col < 2; ++col) {
        int q[QK];
        uint16_t dbits;
        const bool ok = col ? ok1 : ok0;
        if (ok) {
            dbits = quantize_block<T>(v[col], q);
        } else {
            dbits = 0;                                  // padding block: d = 0, q = 8
#pragma unroll
            for (int i = 0; i < QK; ++i) q[i] = 8;
        }
        const int r = (nl + col) & 15;
        const int g = r & 7, hi8 = r >> 3;
        uint8_t *tile = s_tile[(nl + col) >> 4];
        uint16_t *sb = reinterpret_cast<uint16_t *>(&s_blk[kbl][shift + (nl + col) * BLOCK_BYTES]);
        if (blocks != nullptr) sb[0] = dbits;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            uint32_t iw = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j)
                iw |= (uint32_t)(q[8 * c + 2 * j] | (q[8 * c + 2 * j + 1] << 4)) << (8 * j);   // quantization.py:364-369
            if (blocks != nullptr) {
                sb[1 + 2 * c] = (uint16_t)(iw & 0xFFFF);
                sb[2 + 2 * c] = (uint16_t)(iw >> 16);
            }
            *reinterpret_cast<uint32_t *>(tile + slot_of(g, c) * 16 + (kbl * 2 + hi8) * 4) =
                interchange_to_prepacked_word(iw);
        }
        *reinterpret_cast<uint16_t *>(tile + TILE_QS_BYTES + g * 8 + (kbl * 2 + hi8) * 2) = dbits;
    }
    __syncthreads();

    const int64_t nt0 = n0 / TILE_N;
    if (prepacked != nullptr) {
        const int ntiles = (int)min((int64_t)(QT_N / TILE_N), NT - nt0);
        const int64_t KU = tiles_k(K);
        const uint4 *src = reinterpret_cast<const uint4 *>(&s_tile[0][0]);
        for (int i = tid; i < ntiles * (TILE_BYTES / 16); i += QT_THREADS) {
            const int t = i / (TILE_BYTES / 16), o = i % (TILE_BYTES / 16);
            reinterpret_cast<uint4 *>(prepacked + tile_offset(nt0 + t, ku, KU))[o] = src[i];
        }
    }
    if (blocks != nullptr) {
        const int ncols = (int)min((int64_t)QT_N, N - n0);
#pragma unroll
        for (int b = 0; b < TILE_KB; ++b) {
            const int64_t kbb = ku * TILE_KB + b;
            if (kbb < KB)
                copy_out_congruent(blocks + (size_t)(kbb * N + n0) * BLOCK_BYTES, &s_blk[b][b ? shift1 : shift0],
                                   ncols * BLOCK_BYTES, tid, QT_THREADS);
        }
    }
}

// Weight [N, K] (K contiguous, as torch.nn.Linear stores it).  A block is 32 contiguous values;
// four lanes share a block (8 values = one nibble word each), the block maximum is a quad
// shuffle reduction.  CTA = one prepacked tile column (16 n) x 8 blocks along k, 512 threads.
constexpr int QNK_KB = 8;
constexpr int QNK_THREADS = TILE_N * QNK_KB * 4;

constexpr int QNK_ITER = 2;            // groups of QNK_KB blocks per CTA: two loads in flight per thread at two CTAs per SM

template <typename T>
__global__ void __launch_bounds__(QNK_THREADS, 2)
quantize_nk_kernel(const T *__restrict__ w, int64_t K, int64_t N, uint8_t *__restrict__ blocks,
                   uint8_t *__restrict__ prepacked) {
    __shared__ __align__(16) uint8_t s_tile[QNK_KB / TILE_KB][TILE_BYTES];
    __shared__ __align__(16) uint8_t s_blk[QNK_KB][TILE_N * BLOCK_BYTES + 16];

    const int tid = threadIdx.x;
    const int c = tid & 3;                 // nibble word within the block
    const int kbl = (tid >> 2) & (QNK_KB - 1);
    const int r = tid >> 5;                // row within the 16-column tile (one warp per row)
    const int64_t KB = K / QK;
    const int64_t nt = blockIdx.x;
    const int64_t n = nt * TILE_N + r;
    const int64_t n0 = nt * TILE_N;
    const int g = r & 7, hi8 = r >> 3;

    // all of the CTA's loads first: a thread's QNK_ITER 16-byte (32-byte for fp32) pieces are 512
    // (1024) bytes apart in its row
    float v[QNK_ITER][8];
    bool oks[QNK_ITER];
#pragma unroll
    for (int it = 0; it < QNK_ITER; ++it) {
        const int64_t kb = ((int64_t)blockIdx.y * QNK_ITER + it) * QNK_KB + kbl;
        oks[it] = kb < KB && n < N;
        if (oks[it]) {
            const T *p = w + n * K + kb * QK + c * 8;     // 16-byte aligned when the base is (fp16/bf16), 32 for fp32
            if constexpr (sizeof(T) == 4) {
                float4 a = __ldg(reinterpret_cast<const float4 *>(p));
                float4 b = __ldg(reinterpret_cast<const float4 *>(p) + 1);
                v[it][0] = a.x; v[it][1] = a.y; v[it][2] = a.z; v[it][3] = a.w;
                v[it][4] = b.x; v[it][5] = b.y; v[it][6] = b.z; v[it][7] = b.w;
            } else {
                uint4 a = __ldg(reinterpret_cast<const uint4 *>(p));
                const T *e = reinterpret_cast<const T *>(&a);
#pragma unroll
                for (int i = 0; i < 8; ++i) v[it][i] = RoundTo<T>::ld(e + i);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[it][i] = 0.0f;
        }
    }

#pragma unroll
    for (int it = 0; it < QNK_ITER; ++it) {
        const int64_t kb0 = ((int64_t)blockIdx.y * QNK_ITER + it) * QNK_KB;
        if (kb0 >= KB) break;                              // uniform over the CTA
        const int64_t kb = kb0 + kbl;
        const bool ok = oks[it];
        float amax = 0.0f;
        bool nan = false;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float a = fabsf(v[it][i]);
            nan |= (a != a);
            amax = fmaxf(amax, a);
        }
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        int nan_i = nan ? 1 : 0;
        nan_i |= __shfl_xor_sync(0xffffffffu, nan_i, 1);
        nan_i |= __shfl_xor_sync(0xffffffffu, nan_i, 2);
        nan = nan_i != 0;
        float d = RoundTo<T>::r(__fdiv_rn(amax, 7.0f));
        if (nan || !(d > 0.0f)) d = 1.0f;
        uint32_t iw = 0x88888888u;
        uint16_t dbits = 0;
        if (ok) {
            dbits = __half_as_ushort(__float2half_rn(d));
            iw = 0;
            const BlockDivider<T> div(d);
#pragma unroll
            for (int i = 0; i < 8; i += 2) {
                float t0 = div(v[it][i]), t1 = div(v[it][i + 1]);
                round_pair<T>(t0, t1);
                t0 = __fadd_rn(t0, 8.0f);
                t1 = __fadd_rn(t1, 8.0f);
                round_pair<T>(t0, t1);
                iw |= (uint32_t)round_clamp_q(t0) << (4 * i);          // byte j = q[2j] | q[2j+1] << 4
                iw |= (uint32_t)round_clamp_q(t1) << (4 * i + 4);
            }
        }
        uint8_t *tile = s_tile[kbl >> 1];
        *reinterpret_cast<uint32_t *>(tile + slot_of(g, c) * 16 + ((kbl & 1) * 2 + hi8) * 4) =
            interchange_to_prepacked_word(iw);
        if (c == 0) *reinterpret_cast<uint16_t *>(tile + TILE_QS_BYTES + g * 8 + ((kbl & 1) * 2 + hi8) * 2) = dbits;
        if (blocks != nullptr) {
            const int shift = (int)((reinterpret_cast<uintptr_t>(blocks) + (size_t)(kb * N + n0) * BLOCK_BYTES) & 15);
            uint16_t *sb = reinterpret_cast<uint16_t *>(&s_blk[kbl][shift + r * BLOCK_BYTES]);
            if (c == 0) sb[0] = dbits;
            sb[1 + 2 * c] = (uint16_t)(iw & 0xFFFF);
            sb[2 + 2 * c] = (uint16_t)(iw >> 16);
        }
        __syncthreads();
        if (prepacked != nullptr) {
            // the group's four tiles are consecutive k tiles of one column tile: contiguous in memory
            const int64_t ku0 = kb0 / TILE_KB;
            const int64_t KU = tiles_k(K);
            for (int i = tid; i < (QNK_KB / TILE_KB) * (TILE_BYTES / 16); i += QNK_THREADS) {
                const int t = i / (TILE_BYTES / 16), o = i % (TILE_BYTES / 16);
                if (ku0 + t < KU)
                    reinterpret_cast<uint4 *>(prepacked + tile_offset(nt, ku0 + t, KU))[o] =
                        reinterpret_cast<const uint4 *>(&s_tile[t][0])[o];
            }
        }
        if (blocks != nullptr) {
            const int ncols = (int)min((int64_t)TILE_N, N - n0);
            // one warp per block row copies its 16 x 18 bytes
            const int warp = tid >> 5, lane = tid & 31;
            if (warp < QNK_KB && kb0 + warp < KB) {
                uint8_t *dst = blocks + (size_t)((kb0 + warp) * N + n0) * BLOCK_BYTES;
                const int shift = (int)(reinterpret_cast<uintptr_t>(dst) & 15);
                copy_out_congruent(dst, &s_blk[warp][shift], ncols * BLOCK_BYTES, lane, 32);
            }
        }
        __syncthreads();                                    // the staging buffers are reused by the next group
    }
}

// interchange blocks -> prepacked tiles.  One warp per tile, lane = 16-byte slot.
__global__ void __launch_bounds__(128)
repack_kernel(const uint8_t *__restrict__ blocks, int64_t K, int64_t N, uint8_t *__restrict__ prepacked) {
    const int64_t KB = K / QK, NT = tiles_n(N), KU = tiles_k(K);
    const int64_t tile_id = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (tile_id >= NT * KU) return;
    const int64_t nt = tile_id / KU, ku = tile_id % KU;
    const int p = threadIdx.x & 31;
    int g, c;
    slot_inverse(p, g, c);
    uint32_t wds[4];
    uint16_t ds[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int64_t kb = ku * TILE_KB + (j >> 1);
        const int64_t n = nt * TILE_N + g + 8 * (j & 1);
        wds[j] = 0x88888888u;
        ds[j] = 0;
        if (kb < KB && n < N) {
            const uint16_t *b = reinterpret_cast<const uint16_t *>(blocks + (size_t)(kb * N + n) * BLOCK_BYTES);
            ds[j] = __ldg(b);
            const uint32_t iw = (uint32_t)__ldg(b + 1 + 2 * c) | ((uint32_t)__ldg(b + 2 + 2 * c) << 16);
            wds[j] = interchange_to_prepacked_word(iw);
        }
    }
    uint8_t *tile = prepacked + (size_t)tile_id * TILE_BYTES;
    *reinterpret_cast<uint4 *>(tile + p * 16) = make_uint4(wds[0], wds[1], wds[2], wds[3]);
    if (c == 0)      // the scales of row g are the same for every k-octet; one lane writes them
        *reinterpret_cast<uint2 *>(tile + TILE_QS_BYTES + g * 8) =
            make_uint2((uint32_t)ds[0] | ((uint32_t)ds[1] << 16), (uint32_t)ds[2] | ((uint32_t)ds[3] << 16));
}

// prepacked tiles -> interchange blocks (the inverse permutation).
__global__ void __launch_bounds__(128)
unpack_kernel(const uint8_t *__restrict__ prepacked, int64_t K, int64_t N, uint8_t *__restrict__ blocks) {
    const int64_t KB = K / QK, NT = tiles_n(N), KU = tiles_k(K);
    const int64_t tile_id = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (tile_id >= NT * KU) return;
    const int64_t nt = tile_id / KU, ku = tile_id % KU;
    const int p = threadIdx.x & 31;
    int g, c;
    slot_inverse(p, g, c);
    const uint8_t *tile = prepacked + (size_t)tile_id * TILE_BYTES;
    const uint4 qw = __ldg(reinterpret_cast<const uint4 *>(tile + p * 16));
    const uint2 dw = __ldg(reinterpret_cast<const uint2 *>(tile + TILE_QS_BYTES + g * 8));
    const uint32_t wds[4] = {qw.x, qw.y, qw.z, qw.w};
    const uint16_t ds[4] = {(uint16_t)(dw.x & 0xFFFF), (uint16_t)(dw.x >> 16), (uint16_t)(dw.y & 0xFFFF),
                            (uint16_t)(dw.y >> 16)};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int64_t kb = ku * TILE_KB + (j >> 1);
        const int64_t n = nt * TILE_N + g + 8 * (j & 1);
        if (kb < KB && n < N) {
            uint16_t *b = reinterpret_cast<uint16_t *>(blocks + (size_t)(kb * N + n) * BLOCK_BYTES);
            const uint32_t iw = prepacked_to_interchange_word(wds[j]);
            if (c == 0) b[0] = ds[j];
            b[1 + 2 * c] = (uint16_t)(iw & 0xFFFF);
            b[2 + 2 * c] = (uint16_t)(iw >> 16);
        }
    }
}

// interchange blocks -> dense W [K, N]: (q - 8) * float(d) in fp32, then cast
// (quantization.py:391-419).  One thread per block, column-contiguous stores.
template <typename T> __device__ __forceinline__ T cast_out(float v);
template <> __device__ __forceinline__ float cast_out<float>(float v) { return v; }
template <> __device__ __forceinline__ __half cast_out<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 cast_out<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <typename T>
__global__ void __launch_bounds__(128)
dequantize_kernel(const uint8_t *__restrict__ blocks, int64_t K, int64_t N, T *__restrict__ w) {
    const int64_t n = (int64_t)blockIdx.x * 128 + threadIdx.x;
    const int64_t kb = blockIdx.y;
    if (n >= N) return;
    const uint16_t *b = reinterpret_cast<const uint16_t *>(blocks + (size_t)(kb * N + n) * BLOCK_BYTES);
    const float d = __half2float(__ushort_as_half(__ldg(b)));
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const uint32_t two = __ldg(b + 1 + j);           // bytes 2j, 2j+1 -> q[4j .. 4j+3]
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int q = (two >> (4 * i)) & 0xF;
            w[(kb * QK + 4 * j + i) * N + n] = cast_out<T>(__fmul_rn((float)(q - 8), d));
        }
    }
}

}  // namespace q4b

using namespace q4b;

static int check_kn(int64_t K, int64_t N) {
    if (K <= 0 || N <= 0) return Q4B_ERR_ARG;
    if (K % QK) return Q4B_ERR_SHAPE;
    if (tiles_k(K) > 65535 || K / QK > 65535 || N > (int64_t)1 << 31) return Q4B_ERR_SHAPE;
    return Q4B_OK;
}

extern "C" size_t q4b_prepacked_bytes(int64_t K, int64_t N) {
    if (K <= 0 || N <= 0 || K % QK) return 0;
    return (size_t)tiles_k(K) * (size_t)tiles_n(N) * TILE_BYTES;
}

template <typename T>
static int launch_quantize(const void *w, int64_t K, int64_t N, int layout, uint8_t *blocks, uint8_t *prepacked,
                           cudaStream_t st) {
    if (layout == Q4B_LAYOUT_KN) {
        dim3 grid((unsigned)ceil_div(N, QT_N), (unsigned)tiles_k(K));
        const bool vec2 = (N % 2 == 0) && aligned(w, 2 * sizeof(T));
        if (vec2)
            quantize_kn_kernel<T, true><<<grid, QT_THREADS, 0, st>>>((const T *)w, K, N, blocks, prepacked);
        else
            quantize_kn_kernel<T, false><<<grid, QT_THREADS, 0, st>>>((const T *)w, K, N, blocks, prepacked);
    } else {
        if (!aligned(w, 16)) return Q4B_ERR_ALIGN;
        dim3 grid((unsigned)tiles_n(N), (unsigned)ceil_div(K / QK, QNK_KB * QNK_ITER));
        quantize_nk_kernel<T><<<grid, QNK_THREADS, 0, st>>>((const T *)w, K, N, blocks, prepacked);
    }
    Q4B_LAUNCH_CHECK();
    return Q4B_OK;
}

extern "C" int q4b_quantize(const void *w, int w_dtype, int64_t K, int64_t N, int layout, void *blocks_out,
                            void *prepacked_out, void *stream) {
    if (w == nullptr || (blocks_out == nullptr && prepacked_out == nullptr)) return Q4B_ERR_ARG;
    if (layout != Q4B_LAYOUT_KN && layout != Q4B_LAYOUT_NK) return Q4B_ERR_ARG;
    if (int rc = check_kn(K, N)) return rc;
    if (prepacked_out != nullptr && !aligned(prepacked_out, 16)) return Q4B_ERR_ALIGN;
    if (blocks_out != nullptr && !aligned(blocks_out, 2)) return Q4B_ERR_ALIGN;
    if (layout == Q4B_LAYOUT_KN && ceil_div(N, QT_N) > 2147483647LL) return Q4B_ERR_SHAPE;
    cudaStream_t st = (cudaStream_t)stream;
    uint8_t *b = (uint8_t *)blocks_out, *p = (uint8_t *)prepacked_out;
    switch (w_dtype) {
        case Q4B_F32: return launch_quantize<float>(w, K, N, layout, b, p, st);
        case Q4B_F16: return launch_quantize<__half>(w, K, N, layout, b, p, st);
        case Q4B_BF16: return launch_quantize<__nv_bfloat16>(w, K, N, layout, b, p, st);
        default: return Q4B_ERR_DTYPE;
    }
}

extern "C" int q4b_repack(const void *blocks, int64_t K, int64_t N, void *prepacked_out, void *stream) {
    if (blocks == nullptr || prepacked_out == nullptr) return Q4B_ERR_ARG;
    if (int rc = check_kn(K, N)) return rc;
    if (!aligned(prepacked_out, 16) || !aligned(blocks, 2)) return Q4B_ERR_ALIGN;
    const int64_t tiles = tiles_k(K) * tiles_n(N);
    repack_kernel<<<(unsigned)ceil_div(tiles, 4), 128, 0, (cudaStream_t)stream>>>((const uint8_t *)blocks, K, N,
                                                                                 (uint8_t *)prepacked_out);
    Q4B_LAUNCH_CHECK();
    return Q4B_OK;
}

extern "C" int q4b_unpack(const void *prepacked, int64_t K, int64_t N, void *blocks_out, void *stream) {
    if (prepacked == nullptr || blocks_out == nullptr) return Q4B_ERR_ARG;
    if (int rc = check_kn(K, N)) return rc;
    if (!aligned(prepacked, 16) || !aligned(blocks_out, 2)) return Q4B_ERR_ALIGN;
    const int64_t tiles = tiles_k(K) * tiles_n(N);
    unpack_kernel<<<(unsigned)ceil_div(tiles, 4), 128, 0, (cudaStream_t)stream>>>((const uint8_t *)prepacked, K, N,
                                                                                 (uint8_t *)blocks_out);
    Q4B_LAUNCH_CHECK();
    return Q4B_OK;
}

extern "C" int q4b_dequantize(const void *blocks, int64_t K, int64_t N, void *w_out, int out_dtype, void *stream) {
    if (blocks == nullptr || w_out == nullptr) return Q4B_ERR_ARG;
    if (int rc = check_kn(K, N)) return rc;
    if (!aligned(blocks, 2)) return Q4B_ERR_ALIGN;
    dim3 grid((unsigned)ceil_div(N, 128), (unsigned)(K / QK));
    cudaStream_t st = (cudaStream_t)stream;
    switch (out_dtype) {
        case Q4B_F32: dequantize_kernel<float><<<grid, 128, 0, st>>>((const uint8_t *)blocks, K, N, (float *)w_out); break;
        case Q4B_F16: dequantize_kernel<__half><<<grid, 128, 0, st>>>((const uint8_t *)blocks, K, N, (__half *)w_out); break;
        case Q4B_BF16:
            dequantize_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>((const uint8_t *)blocks, K, N, (__nv_bfloat16 *)w_out);
            break;
        default: return Q4B_ERR_DTYPE;
    }
    Q4B_LAUNCH_CHECK();
    return Q4B_OK;
}
