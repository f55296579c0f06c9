// Group-wise asymmetric INT4 format of the reference: quantize, dequantize, and the conversion
// that lets the q4_0 matmul kernels serve it.
//
// Reference: quantize_int4 / dequantize_int4 / matmul_int4 in
// packages/metalcore/src/metalcore/quantization.py:26-239, the Metal quantizer quantize_to_int4
// (quant_kernels.metal:634-690, core_mps.mm:4655-4705) and dispatcher matmul_int4_metal
// (core_mps.mm:5612-5776).  W = (q - zero) * scale with one (scale, zero) per `group` rows of k
// and column; weight_packed [K/2, N] holds k = 2r in the low and 2r+1 in the high nibble.
//
// How the matmul is served: (q - zero) * scale = (q - 8) * d + [q * (scale - d) + 8 * d - zero * scale]
// with d = fp16(scale).  The first term is exactly what the q4_0 tiles compute; the bracket is
// replaced by its q-independent part corr = 8 * d - zero * scale (dropping q * (scale - d), a
// relative weight error of at most 2^-12), which contributes corr[g, n] * sum_{k in g} x[m, k]:
// a small fp32 [M, N] addend that the matmul kernels add before their single rounding.
#include "q4b_common.cuh"

namespace q4b {

template <typename T> struct Num;
template <> struct Num<float> {
    static __device__ __forceinline__ float r(float v) { return v; }
    static __device__ __forceinline__ float ld(const float *p) { return __ldg(p); }
    static __device__ __forceinline__ void st(float *p, float v) { *p = v; }
};
template <> struct Num<__half> {
    static __device__ __forceinline__ float r(float v) { return __half2float(__float2half_rn(v)); }
    static __device__ __forceinline__ float ld(const __half *p) { return __half2float(__ldg(p)); }
    static __device__ __forceinline__ void st(__half *p, float v) { *p = __float2half_rn(v); }
};
template <> struct Num<__nv_bfloat16> {
    static __device__ __forceinline__ float r(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
    static __device__ __forceinline__ float ld(const __nv_bfloat16 *p) { return __bfloat162float(__ldg(p)); }
    static __device__ __forceinline__ void st(__nv_bfloat16 *p, float v) { *p = __float2bfloat16_rn(v); }
};

// One thread per (group, column).  Every arithmetic step is rounded to the weight's dtype, as
// the reference's separate torch ops do (quantization.py:69-83).
template <typename T>
__global__ void __launch_bounds__(128)
int4g_quantize_kernel(const T *__restrict__ w, int64_t K, int64_t N, int64_t group, uint8_t *__restrict__ packed,
                      T *__restrict__ scales, T *__restrict__ zeros) {
    const int64_t n = (int64_t)blockIdx.x * 128 + threadIdx.x;
    const int64_t g = blockIdx.y;
    if (n >= N) return;
    const int64_t k0 = g * group, k1 = min(k0 + group, K);
    float lo = INFINITY, hi = -INFINITY;
    bool nan = false;
    for (int64_t k = k0; k < k1; ++k) {
        const float v = Num<T>::ld(w + k * N + n);
        nan |= (v != v);
        lo = fminf(lo, v);
        hi = fmaxf(hi, v);
    }
    if (nan) { lo = NAN; hi = NAN; }                                        // torch min/max propagate NaN
    float scale = Num<T>::r(__fdiv_rn(Num<T>::r(__fsub_rn(hi, lo)), 15.0f));   // quantization.py:74
    const float tiny = Num<T>::r(1e-8f);                                     // clamp(min=1e-8) in T: 0 for fp16
    if (scale < tiny) scale = tiny;                                          // quantization.py:75 (NaN stays NaN)
    const float zero = Num<T>::r(__fdiv_rn(-lo, scale));                     // quantization.py:76
    Num<T>::st(scales + g * N + n, scale);
    Num<T>::st(zeros + g * N + n, zero);
    auto quant = [&](int64_t k) -> uint32_t {
        float t = Num<T>::r(__fdiv_rn(Num<T>::ld(w + k * N + n), scale));    // quantization.py:83, op by op
        t = Num<T>::r(__fadd_rn(t, zero));
        t = fminf(fmaxf(rintf(t), 0.0f), 15.0f);                             // NaN -> 0
        return (uint32_t)t;
    };
    for (int64_t k = k0; k + 1 < k1; k += 2)                                // group and K are even
        packed[(k >> 1) * N + n] = (uint8_t)(quant(k) | (quant(k + 1) << 4));
}

// ((q - zero) * scale) in fp32, then cast (quantization.py:131-153).  One thread per packed byte.
template <typename TS, typename TO>
__global__ void __launch_bounds__(128)
int4g_dequantize_kernel(const uint8_t *__restrict__ packed, const TS *__restrict__ scales, const TS *__restrict__ zeros,
                        int64_t K, int64_t N, int64_t group, TO *__restrict__ w) {
    const int64_t n = (int64_t)blockIdx.x * 128 + threadIdx.x;
    const int64_t r = blockIdx.y;
    if (n >= N) return;
    const uint32_t b = packed[r * N + n];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int64_t k = 2 * r + i;
        const int64_t g = k / group;
        const float q = (float)((b >> (4 * i)) & 0xF);
        const float v = __fmul_rn(__fsub_rn(q, Num<TS>::ld(zeros + g * N + n)), Num<TS>::ld(scales + g * N + n));
        Num<TO>::st(w + k * N + n, v);
    }
}

// packed [K/2, N] + scales -> streaming tiles with block scale d = fp16(scale).  One warp per tile.
template <typename TS>
__global__ void __launch_bounds__(128)
int4g_prepack_kernel(const uint8_t *__restrict__ packed, const TS *__restrict__ scales, int64_t K, int64_t N,
                     int64_t group, uint8_t *__restrict__ prepacked) {
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
            const int64_t r0 = kb * (QK / 2) + 4 * c;          // packed rows of k = kb*32 + 8c .. +7
            uint32_t iw = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) iw |= (uint32_t)packed[(r0 + i) * N + n] << (8 * i);
            wds[j] = interchange_to_prepacked_word(iw);
            ds[j] = __half_as_ushort(__float2half_rn(Num<TS>::ld(scales + ((kb * QK) / group) * N + n)));
        }
    }
    uint8_t *tile = prepacked + (size_t)tile_id * TILE_BYTES;
    *reinterpret_cast<uint4 *>(tile + p * 16) = make_uint4(wds[0], wds[1], wds[2], wds[3]);
    if (c == 0)
        *reinterpret_cast<uint2 *>(tile + TILE_QS_BYTES + g * 8) =
            make_uint2((uint32_t)ds[0] | ((uint32_t)ds[1] << 16), (uint32_t)ds[2] | ((uint32_t)ds[3] << 16));
}

// set when a group scale does not fit the fp16 block scale of the streaming tiles (read and cleared by
// q4b_int4g_prepack_status)
__device__ int g_int4g_range = 0;

// corr[g, n] = 8 * fp16(scale) - zero * scale
template <typename TS>
__global__ void __launch_bounds__(128)
int4g_corr_kernel(const TS *__restrict__ scales, const TS *__restrict__ zeros, int64_t count, float *__restrict__ corr) {
    const int64_t i = (int64_t)blockIdx.x * 128 + threadIdx.x;
    if (i >= count) return;
    const float s = Num<TS>::ld(scales + i), z = Num<TS>::ld(zeros + i);
    if (!(fabsf(s) <= 65504.0f)) g_int4g_range = 1;            // also catches NaN
    const float d = __half2float(__float2half_rn(s));
    corr[i] = __fsub_rn(__fmul_rn(8.0f, d), __fmul_rn(z, s));
}

// The group-wise format's zero-point term, addend[m, n] = sum_g corr[g, n] * (sum of x[m, k] over group g)
// (+ bias[n]), is a product of rank G = K / group.  Two kernels:
//   int4g_rowsum_kernel  R[m, g]: a warp per (row, group), coalesced loads, fixed-order shuffle reduction;
//                        X is read once.
//   int4g_addend_kernel  a CTA takes 512 columns x 32 rows: a thread owns two columns, their corr[g, n]
//                        values arrive 16 groups at a time (coalesced over the CTA), the rows' group sums
//                        are broadcast from shared memory (one 16-byte read of four rows feeds four
//                        two-wide FMAs, fma.rn.f32x2), 2 x 32 accumulators per thread, coalesced fp32 stores.  corr is re-read once per row
//                        tile, from L2.
// Sum of x[k0 .. k1) over the warp, the same value on every lane, in a fixed order.  When the group is
// 128 sixteen-bit values and 16-byte aligned, sixteen lanes read it with one 16-byte load each (lanes 16-31
// repeat the loads of lanes 0-15 and take no part in the sum).
template <typename TX>
__device__ __forceinline__ float warp_group_sum(const TX *xr, int64_t k0, int64_t k1, int lane) {
    float s = 0.0f;
    if (sizeof(TX) == 2 && k1 - k0 == 128 && (reinterpret_cast<uintptr_t>(xr + k0) & 15) == 0) {
        const uint4 v = __ldg(reinterpret_cast<const uint4 *>(xr + k0) + (lane & 15));
        const TX *e = reinterpret_cast<const TX *>(&v);
#pragma unroll
        for (int i = 0; i < 8; ++i) s += Num<TX>::r((float)e[i]);
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        return s;
    }
    for (int64_t k = k0 + lane; k < k1; k += 32) s += Num<TX>::ld(xr + k);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    return s;
}

template <typename TX>
__global__ void __launch_bounds__(256)
int4g_rowsum_kernel(const TX *__restrict__ x, int64_t M, int64_t ldx, int64_t K, int64_t group, int G, float *__restrict__ rowsums) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t pairs = M * G;
    for (int64_t p = (int64_t)blockIdx.x * 8 + warp; p < pairs; p += (int64_t)gridDim.x * 8) {
        int64_t m;
        int g;
        if (pairs < (1LL << 31)) {                       // the usual case: 32-bit division
            m = (int)((unsigned)p / (unsigned)G);
            g = (int)((unsigned)p % (unsigned)G);
        } else {
            m = p / G;
            g = (int)(p % G);
        }
        const TX *xr = x + m * ldx;
        const int64_t k0 = (int64_t)g * group, k1 = min(k0 + group, K);
        const float s = warp_group_sum<TX>(xr, k0, k1, lane);
        if (lane == 0) rowsums[p] = s;
    }
}

constexpr int ADD_ROWS = 32;       // rows per CTA of the addend kernel: corr is re-read from L2 once per this many rows
constexpr int ADD_COLS = 512;      // columns per CTA: two per thread, so a broadcast read of four group sums feeds eight FMAs
constexpr int ADD_GCHUNK = 16;     // groups per pass

// two independent fp32 FMAs in one instruction: d = a * b + c on both halves of the pairs
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
    float2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;"
        : "=l"(reinterpret_cast<unsigned long long &>(d))
        : "l"(reinterpret_cast<const unsigned long long &>(a)), "l"(reinterpret_cast<const unsigned long long &>(b)),
          "l"(reinterpret_cast<const unsigned long long &>(c)));
    return d;
}

__global__ void __launch_bounds__(256, 2)
int4g_addend_kernel(const float *__restrict__ rowsums, int64_t M, const float *__restrict__ corr,
                    const float *__restrict__ bias, int64_t N, int G, float *__restrict__ addend) {
    __shared__ __align__(16) float rs[ADD_GCHUNK][ADD_ROWS];                    // [group][row]: four rows per 16-byte read
    const int64_t n = (int64_t)blockIdx.x * ADD_COLS + 2 * threadIdx.x;          // this thread's columns: n, n + 1
    const int64_t m0 = (int64_t)blockIdx.y * ADD_ROWS;
    const int nrows = (int)min((int64_t)ADD_ROWS, M - m0);
    const bool ok0 = n < N, ok1 = n + 1 < N;
    const bool pair = ok1 && (N % 2 == 0);                                        // both columns, 8-byte aligned
    float2 acc0[ADD_ROWS / 2], acc1[ADD_ROWS / 2];                                // (row 2i, row 2i + 1) of column n / n + 1
    const float b0 = (bias != nullptr && ok0) ? bias[n] : 0.0f, b1 = (bias != nullptr && ok1) ? bias[n + 1] : 0.0f;
#pragma unroll
    for (int r = 0; r < ADD_ROWS / 2; ++r) { acc0[r] = make_float2(b0, b0); acc1[r] = make_float2(b1, b1); }
    for (int g0 = 0; g0 < G; g0 += ADD_GCHUNK) {
        __syncthreads();
        for (int i = threadIdx.x; i < ADD_ROWS * ADD_GCHUNK; i += 256) {
            const int r = i / ADD_GCHUNK, j = i % ADD_GCHUNK;                    // consecutive threads: consecutive groups of a row
            rs[j][r] = (r < nrows && g0 + j < G) ? rowsums[(m0 + r) * G + g0 + j] : 0.0f;
        }
        float2 c0[ADD_GCHUNK], c1[ADD_GCHUNK];                                    // corr[g, n] and corr[g, n + 1], each twice
#pragma unroll
        for (int j = 0; j < ADD_GCHUNK; ++j) {
            const float *cp = corr + (int64_t)(g0 + j) * N + n;
            float v0, v1;
            if (g0 + j < G && pair) {
                const float2 v = *reinterpret_cast<const float2 *>(cp);
                v0 = v.x;
                v1 = v.y;
            } else {
                v0 = (g0 + j < G && ok0) ? cp[0] : 0.0f;
                v1 = (g0 + j < G && ok1) ? cp[1] : 0.0f;
            }
            c0[j] = make_float2(v0, v0);
            c1[j] = make_float2(v1, v1);
        }
        __syncthreads();
#pragma unroll
        for (int j = 0; j < ADD_GCHUNK; ++j) {
#pragma unroll
            for (int r = 0; r < ADD_ROWS; r += 4) {
                const float4 v = *reinterpret_cast<const float4 *>(&rs[j][r]);    // the same address in every lane: a broadcast
                const float2 lo = make_float2(v.x, v.y), hi = make_float2(v.z, v.w);
                acc0[r / 2] = fma2(c0[j], lo, acc0[r / 2]);
                acc0[r / 2 + 1] = fma2(c0[j], hi, acc0[r / 2 + 1]);
                acc1[r / 2] = fma2(c1[j], lo, acc1[r / 2]);
                acc1[r / 2 + 1] = fma2(c1[j], hi, acc1[r / 2 + 1]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < ADD_ROWS; ++r) {
        if (r < nrows) {
            const float a0 = (r & 1) ? acc0[r / 2].y : acc0[r / 2].x, a1 = (r & 1) ? acc1[r / 2].y : acc1[r / 2].x;
            float *op = addend + (m0 + r) * N + n;
            if (pair) *reinterpret_cast<float2 *>(op) = make_float2(a0, a1);
            else {
                if (ok0) op[0] = a0;
                if (ok1) op[1] = a1;
            }
        }
    }
}

// ---- the zero-point term folded into the tensor-core contraction --------------------------------------
// sum_g R[m, g] * C[g, n] needs fp32-like accuracy from bf16 operands: each factor is split into three bf16
// terms (hi + mid + lo = 24 bits) and the six largest products are kept (hi.hi, mid.hi, hi.mid, lo.hi,
// hi.lo, mid.mid; what is dropped is below 2^-24 of |R C|).  That makes 6 G extra k, padded with zeros to
// whole 64-k tiles.  Segment s of the extra k range holds, for g = 0..G-1:
//      rows  (X side):    R_hi, R_mid, R_hi,  R_lo, R_hi, R_mid
//      operand (W side):  C_hi, C_hi,  C_mid, C_hi, C_lo, C_mid
__device__ __forceinline__ void split3_bf16(float v, uint16_t &hi, uint16_t &mid, uint16_t &lo) {
    const __nv_bfloat16 h = __float2bfloat16_rn(v);
    const float r1 = v - __bfloat162float(h);                   // exact
    const __nv_bfloat16 m = __float2bfloat16_rn(r1);
    const float r2 = r1 - __bfloat162float(m);                  // exact
    hi = __bfloat16_as_ushort(h);
    mid = __bfloat16_as_ushort(m);
    lo = __bfloat16_as_ushort(__float2bfloat16_rn(r2));
}

// out [N, E] bf16 from corr [G, N] fp32; E = 64 * ceil(6 G / 64).  A thread per (n, g).
__global__ void __launch_bounds__(256)
int4g_fold_operand_kernel(const float *__restrict__ corr, int G, int64_t N, int E, uint16_t *__restrict__ out) {
    const int64_t idx = (int64_t)blockIdx.x * 256 + threadIdx.x;
    const int64_t n = idx % N;                                   // consecutive threads: consecutive columns of corr
    const int64_t g = idx / N;
    if (g >= G) {
        // the threads past the last group clear the padding of their column
        const int64_t pad = g - G;
        if (pad == 0)
            for (int e = 6 * G; e < E; ++e) out[n * E + e] = 0;
        return;
    }
    uint16_t hi, mid, lo;
    split3_bf16(corr[g * N + n], hi, mid, lo);
    uint16_t *o = out + n * E + g;
    o[0] = hi; o[G] = hi; o[2 * G] = mid; o[3 * G] = hi; o[4 * G] = lo; o[5 * G] = mid;
}

// rows [M, E] bf16 from X.  Generic form: a warp per (row, group) as in int4g_rowsum_kernel.
__device__ __forceinline__ void store_fold_row_terms(uint16_t *o, int G, int g, float s) {
    uint16_t hi, mid, lo;
    split3_bf16(s, hi, mid, lo);
    o[g] = hi; o[G + g] = mid; o[2 * G + g] = hi; o[3 * G + g] = lo; o[4 * G + g] = hi; o[5 * G + g] = mid;
}

template <typename TX>
__global__ void __launch_bounds__(256)
int4g_fold_rows_kernel(const TX *__restrict__ x, int64_t M, int64_t ldx, int64_t K, int64_t group, int G, int E,
                       uint16_t *__restrict__ rows_out) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t pairs = M * G;
    for (int64_t p = (int64_t)blockIdx.x * 8 + warp; p < pairs; p += (int64_t)gridDim.x * 8) {
        int64_t m;
        int g;
        if (pairs < (1LL << 31)) {
            m = (int)((unsigned)p / (unsigned)G);
            g = (int)((unsigned)p % (unsigned)G);
        } else {
            m = p / G;
            g = (int)(p % G);
        }
        const int64_t k0 = (int64_t)g * group, k1 = min(k0 + group, K);
        const float s = warp_group_sum<TX>(x + m * ldx, k0, k1, lane);
        uint16_t *o = rows_out + m * E;
        if (lane == 0) store_fold_row_terms(o, G, g, s);
        if (g == 0)
            for (int e = 6 * G + lane; e < E; e += 32) o[e] = 0;
    }
}

// Groups of 128 sixteen-bit values, rows 16-byte aligned, K a multiple of 128: a warp takes sixteen
// consecutive groups of a row (4 KB): eight 16-byte loads per lane in flight, half-warp reductions, then
// lanes 0..15 each split one group sum and store its six terms (consecutive lanes, consecutive addresses).
template <typename TX>
__global__ void __launch_bounds__(256)
int4g_fold_rows128_kernel(const TX *__restrict__ x, int64_t M, int64_t ldx, int G, int E, uint16_t *__restrict__ rows_out) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int chunks = (G + 15) / 16;                            // warps per row
    const int64_t units = M * chunks;
    for (int64_t u = (int64_t)blockIdx.x * 8 + warp; u < units; u += (int64_t)gridDim.x * 8) {
        const int64_t m = u / chunks;
        const int g0 = (int)(u % chunks) * 16;
        const uint4 *src = reinterpret_cast<const uint4 *>(x + m * ldx + (int64_t)g0 * 128);
        uint4 v[8];
#pragma unroll
        for (int t = 0; t < 8; ++t)
            v[t] = g0 + 2 * t + (lane >> 4) < G ? __ldg(src + t * 32 + lane) : make_uint4(0u, 0u, 0u, 0u);
        float mine = 0.0f;                                       // lane l < 16 ends up with the sum of group g0 + l
#pragma unroll
        for (int t = 0; t < 8; ++t) {
            const TX *e = reinterpret_cast<const TX *>(&v[t]);
            float s = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) s += Num<TX>::r((float)e[i]);
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            const float lo_half = __shfl_sync(0xffffffffu, s, 0), hi_half = __shfl_sync(0xffffffffu, s, 16);
            if (lane == 2 * t) mine = lo_half;
            if (lane == 2 * t + 1) mine = hi_half;
        }
        uint16_t *o = rows_out + m * E;
        if (lane < 16 && g0 + lane < G) store_fold_row_terms(o, G, g0 + lane, mine);
        if (g0 == 0)
            for (int e = 6 * G + lane; e < E; e += 32) o[e] = 0;
    }
}

}  // namespace q4b

using namespace q4b;

static int check_g(int64_t K, int64_t N, int64_t group) {
    if (K <= 0 || N <= 0 || group <= 0) return Q4B_ERR_ARG;
    if ((K % 2) || (group % 2)) return Q4B_ERR_SHAPE;
    if (ceil_div(K, group) > 65535 || K / 2 > 2147483647LL) return Q4B_ERR_SHAPE;
    return Q4B_OK;
}

extern "C" int q4b_int4g_quantize(const void *w, int w_dtype, int64_t K, int64_t N, int64_t group, void *packed_out,
                                  void *scales_out, void *zeros_out, void *stream) {
    if (w == nullptr || packed_out == nullptr || scales_out == nullptr || zeros_out == nullptr) return Q4B_ERR_ARG;
    if (int rc = check_g(K, N, group)) return rc;
    dim3 grid((unsigned)ceil_div(N, 128), (unsigned)ceil_div(K, group));
    cudaStream_t st = (cudaStream_t)stream;
    uint8_t *p = (uint8_t *)packed_out;
    switch (w_dtype) {
        case Q4B_F32: int4g_quantize_kernel<float><<<grid, 128, 0, st>>>((const float *)w, K, N, group, p, (float *)scales_out, (float *)zeros_out); break;
        case Q4B_F16: int4g_quantize_kernel<__half><<<grid, 128, 0, st>>>((const __half *)w, K, N, group, p, (__half *)scales_out, (__half *)zeros_out); break;
        case Q4B_BF16: int4g_quantize_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>((const __nv_bfloat16 *)w, K, N, group, p, (__nv_bfloat16 *)scales_out, (__nv_bfloat16 *)zeros_out); break;
        default: return Q4B_ERR_DTYPE;
    }
    Q4B_LAUNCH_CHECK();
    return Q4B_OK;
}

template <typename TS>
static int launch_deq(const void *packed, const void *scales, const void *zeros, int64_t K, int64_t N, int64_t group,
                      void *w_out, int out_dtype, cudaStream_t st) {
    dim3 grid((unsigned)ceil_div(N, 128), (unsigned)(K / 2));
    const uint8_t *p = (const uint8_t *)packed;
    const TS *s = (const TS *)scales, *z = (const TS *)zeros;
    switch (out_dtype) {
        case Q4B_F32: int4g_dequantize_kernel<TS, float><<<grid, 128, 0, st>>>(p, s, z, K, N, group, (float *)w_out); break;
        case Q4B_F16: int4g_dequantize_kernel<TS, __half><<<grid, 128, 0, st>>>(p, s, z, K, N, group, (__half *)w_out); break;
        case Q4B_BF16: int4g_dequantize_kernel<TS, __nv_bfloat16><<<grid, 128, 0, st>>>(p, s, z, K, N, group, (__nv_bfloat16 *)w_out); break;
        default: return Q4B_ERR_DTYPE;
    }
    Q4B_LAUNCH_CHECK();
    return Q4B_OK;
}

extern "C" int q4b_int4g_dequantize(const void *packed, const void *scales, const void *zeros, int sz_dtype, int64_t K,
                                    int64_t N, int64_t group, void *w_out, int out_dtype, void *stream) {
    if (packed == nullptr || scales == nullptr || zeros == nullptr || w_out == nullptr) return Q4B_ERR_ARG;
    if (int rc = check_g(K, N, group)) return rc;
    if (K / 2 > 65535) return Q4B_ERR_SHAPE;                 // grid.y
    cudaStream_t st = (cudaStream_t)stream;
    switch (sz_dtype) {
        case Q4B_F32: return launch_deq<float>(packed, scales, zeros, K, N, group, w_out, out_dtype, st);
        case Q4B_F16: return launch_deq<__half>(packed, scales, zeros, K, N, group, w_out, out_dtype, st);
        case Q4B_BF16: return launch_deq<__nv_bfloat16>(packed, scales, zeros, K, N, group, w_out, out_dtype, st);
        default: return Q4B_ERR_DTYPE;
    }
}

template <typename TS>
static int launch_prepack(const void *packed, const void *scales, const void *zeros, int64_t K, int64_t N, int64_t group,
                          void *prepacked_out, float *corr_out, cudaStream_t st) {
    const int64_t tiles = tiles_k(K) * tiles_n(N);
    int4g_prepack_kernel<TS><<<(unsigned)ceil_div(tiles, 4), 128, 0, st>>>((const uint8_t *)packed, (const TS *)scales, K, N,
                                                                           group, (uint8_t *)prepacked_out);
    Q4B_LAUNCH_CHECK();
    const int64_t count = ceil_div(K, group) * N;
    int4g_corr_kernel<TS><<<(unsigned)ceil_div(count, 128), 128, 0, st>>>((const TS *)scales, (const TS *)zeros, count, corr_out);
    Q4B_LAUNCH_CHECK();
    return Q4B_OK;
}

extern "C" int q4b_int4g_prepack(const void *packed, const void *scales, const void *zeros, int sz_dtype, int64_t K,
                                 int64_t N, int64_t group, void *prepacked_out, float *corr_out, void *stream) {
    if (packed == nullptr || scales == nullptr || zeros == nullptr || prepacked_out == nullptr || corr_out == nullptr)
        return Q4B_ERR_ARG;
    if (int rc = check_g(K, N, group)) return rc;
    if ((K % QK) || (group % QK)) return Q4B_ERR_SHAPE;       // a 32-k block must lie inside one group
    if (!aligned(prepacked_out, 16)) return Q4B_ERR_ALIGN;
    cudaStream_t st = (cudaStream_t)stream;
    switch (sz_dtype) {
        case Q4B_F32: return launch_prepack<float>(packed, scales, zeros, K, N, group, prepacked_out, corr_out, st);
        case Q4B_F16: return launch_prepack<__half>(packed, scales, zeros, K, N, group, prepacked_out, corr_out, st);
        case Q4B_BF16: return launch_prepack<__nv_bfloat16>(packed, scales, zeros, K, N, group, prepacked_out, corr_out, st);
        default: return Q4B_ERR_DTYPE;
    }
}

extern "C" size_t q4b_int4g_rowsums_bytes(int64_t M, int64_t K, int64_t group) {
    if (M < 1 || K < 1 || group < 1) return 0;
    return (size_t)M * (size_t)ceil_div(K, group) * sizeof(float);
}

extern "C" int q4b_int4g_rowsums(const void *x, int x_dtype, int64_t M, int64_t ldx, int64_t K, int64_t group, float *rowsums_out,
                                 void *stream) {
    if (x == nullptr || rowsums_out == nullptr) return Q4B_ERR_ARG;
    if (M < 1 || ldx < K || K < 1 || group < 1) return Q4B_ERR_ARG;
    const int64_t G = ceil_div(K, group);
    const int64_t pairs = M * G;
    const unsigned grid1 = (unsigned)(ceil_div(pairs, 8) < 16384 ? ceil_div(pairs, 8) : 16384);
    cudaStream_t st = (cudaStream_t)stream;
    switch (x_dtype) {
        case Q4B_F16: int4g_rowsum_kernel<__half><<<grid1, 256, 0, st>>>((const __half *)x, M, ldx, K, group, (int)G, rowsums_out); break;
        case Q4B_BF16: int4g_rowsum_kernel<__nv_bfloat16><<<grid1, 256, 0, st>>>((const __nv_bfloat16 *)x, M, ldx, K, group, (int)G, rowsums_out); break;
        default: return Q4B_ERR_DTYPE;
    }
    Q4B_LAUNCH_CHECK();
    return Q4B_OK;
}

extern "C" int q4b_int4g_addend(const void *x, int x_dtype, int64_t M, int64_t ldx, const float *corr, const float *bias,
                                int64_t K, int64_t N, int64_t group, float *rowsums_ws, float *addend_out, void *stream) {
    if (x == nullptr || corr == nullptr || addend_out == nullptr || rowsums_ws == nullptr) return Q4B_ERR_ARG;
    if (M < 1 || ldx < K) return Q4B_ERR_ARG;
    if (int rc = check_g(K, N, group)) return rc;
    const int64_t G = ceil_div(K, group);
    if (ceil_div(M, ADD_ROWS) > 65535) {
        // more row tiles than grid.y holds: in slices of 65535 tiles
        const int64_t step = (int64_t)65535 * ADD_ROWS;
        for (int64_t m0 = 0; m0 < M; m0 += step) {
            const int64_t rows = M - m0 < step ? M - m0 : step;
            if (int rc = q4b_int4g_addend((const uint8_t *)x + (size_t)m0 * ldx * 2, x_dtype, rows, ldx, corr, bias, K, N, group,
                                          rowsums_ws + m0 * G, addend_out + m0 * N, stream))
                return rc;
        }
        return Q4B_OK;
    }
    const int64_t pairs = M * G;
    const unsigned grid1 = (unsigned)(ceil_div(pairs, 8) < 16384 ? ceil_div(pairs, 8) : 16384);
    cudaStream_t st = (cudaStream_t)stream;
    switch (x_dtype) {
        case Q4B_F16: int4g_rowsum_kernel<__half><<<grid1, 256, 0, st>>>((const __half *)x, M, ldx, K, group, (int)G, rowsums_ws); break;
        case Q4B_BF16: int4g_rowsum_kernel<__nv_bfloat16><<<grid1, 256, 0, st>>>((const __nv_bfloat16 *)x, M, ldx, K, group, (int)G, rowsums_ws); break;
        default: return Q4B_ERR_DTYPE;
    }
    Q4B_LAUNCH_CHECK();
    dim3 grid2((unsigned)ceil_div(N, ADD_COLS), (unsigned)ceil_div(M, ADD_ROWS));
    int4g_addend_kernel<<<grid2, 256, 0, st>>>(rowsums_ws, M, corr, bias, N, (int)G, addend_out);
    Q4B_LAUNCH_CHECK();
    return Q4B_OK;
}

extern "C" int q4b_int4g_fold_ktiles(int64_t K, int64_t group) {
    if (K < 1 || group < 1) return 0;
    return (int)ceil_div(6 * ceil_div(K, group), TILE_K);
}

extern "C" int q4b_int4g_fold_operand(const float *corr, int64_t K, int64_t N, int64_t group, void *operand_out, void *stream) {
    if (corr == nullptr || operand_out == nullptr) return Q4B_ERR_ARG;
    if (int rc = check_g(K, N, group)) return rc;
    if (!aligned(operand_out, 16)) return Q4B_ERR_ALIGN;
    const int64_t G = ceil_div(K, group);
    const int E = q4b_int4g_fold_ktiles(K, group) * TILE_K;
    const int64_t threads = (G + 1) * N;                          // one more "group" of threads clears the padding
    int4g_fold_operand_kernel<<<(unsigned)ceil_div(threads, 256), 256, 0, (cudaStream_t)stream>>>(corr, (int)G, N, E, (uint16_t *)operand_out);
    Q4B_LAUNCH_CHECK();
    return Q4B_OK;
}

extern "C" int q4b_int4g_fold_rows(const void *x, int x_dtype, int64_t M, int64_t ldx, int64_t K, int64_t group, void *rows_out,
                                   void *stream) {
    if (x == nullptr || rows_out == nullptr) return Q4B_ERR_ARG;
    if (M < 1 || ldx < K || K < 1 || group < 1) return Q4B_ERR_ARG;
    if (!aligned(rows_out, 16)) return Q4B_ERR_ALIGN;
    const int64_t G = ceil_div(K, group);
    if (G > 65535) return Q4B_ERR_SHAPE;
    const int E = q4b_int4g_fold_ktiles(K, group) * TILE_K;
    const int64_t pairs = M * G;
    const unsigned grid = (unsigned)(ceil_div(pairs, 8) < 16384 ? ceil_div(pairs, 8) : 16384);
    cudaStream_t st = (cudaStream_t)stream;
    if (group == 128 && K % 128 == 0 && ldx % 8 == 0 && aligned(x, 16)) {
        const int64_t units = M * ceil_div(G, 16);
        const unsigned grid128 = (unsigned)(ceil_div(units, 8) < 16384 ? ceil_div(units, 8) : 16384);
        switch (x_dtype) {
            case Q4B_F16: int4g_fold_rows128_kernel<__half><<<grid128, 256, 0, st>>>((const __half *)x, M, ldx, (int)G, E, (uint16_t *)rows_out); break;
            case Q4B_BF16: int4g_fold_rows128_kernel<__nv_bfloat16><<<grid128, 256, 0, st>>>((const __nv_bfloat16 *)x, M, ldx, (int)G, E, (uint16_t *)rows_out); break;
            default: return Q4B_ERR_DTYPE;
        }
        Q4B_LAUNCH_CHECK();
        return Q4B_OK;
    }
    switch (x_dtype) {
        case Q4B_F16: int4g_fold_rows_kernel<__half><<<grid, 256, 0, st>>>((const __half *)x, M, ldx, K, group, (int)G, E, (uint16_t *)rows_out); break;
        case Q4B_BF16: int4g_fold_rows_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16 *)x, M, ldx, K, group, (int)G, E, (uint16_t *)rows_out); break;
        default: return Q4B_ERR_DTYPE;
    }
    Q4B_LAUNCH_CHECK();
    return Q4B_OK;
}

extern "C" int q4b_int4g_prepack_status(void *stream, int *out_of_range) {
    Q4B_CUDA_TRY(cudaStreamSynchronize((cudaStream_t)stream));
    int h = 0;
    Q4B_CUDA_TRY(cudaMemcpyFromSymbol(&h, g_int4g_range, sizeof(int)));
    if (h != 0) {
        const int zero = 0;
        Q4B_CUDA_TRY(cudaMemcpyToSymbol(g_int4g_range, &zero, sizeof(int)));
    }
    if (out_of_range != nullptr) *out_of_range = h;
    return Q4B_OK;
}
