// Two side entrances of the INT4 path.
//
// 1. Weights quantised by other GGML tools.  The reference states where its block format comes
//    from (packages/metalcore/src/metalcore/quantization.py:292-304) and carries a helper that reads
//    the original nibble order (quant_kernels.metal:1714-1731: byte j of a block holds value j in
//    its low and value j + 16 in its high nibble, rows of K/32 blocks per output feature).
//      q4b_import_ggml    [N, K/32, 18] in that order  ->  this library's [K/32, N, 18]
//      q4b_quantize_ggml  the scale rule of those tools: d = (the value of largest magnitude) / -8,
//                         q = clamp(round(w / d) + 8, 0, 15), an all-zero block has d = 0, q = 8
//                         (arithmetic in fp32, ties to even), written in this library's layout.
// 2. The reference's group-wise INT8 weights (quantization.py:242-286; kernels
//    quant_kernels.metal:40-109, host core_mps.mm:4516-4574): W = (w_q - zero) * scale with int8
//    w_q [K, N] and scales / zeros [ceil(K / group), N].  q4b_int8g_matmul streams the weights once
//    with 128-byte row reads and accumulates in fp32 on the CUDA cores: HBM-bound for the few rows
//    of a decode step; larger M is tiled eight rows at a time (re-reading the weights per row tile).
#include "q4b_common.cuh"

namespace q4b {

// ---- GGML import ------------------------------------------------------------------------------
__global__ void __launch_bounds__(128)
import_ggml_kernel(const uint8_t *__restrict__ raw, int64_t KB, int64_t N, uint8_t *__restrict__ blocks) {
    const int64_t n = (int64_t)blockIdx.x * 128 + threadIdx.x;
    const int64_t kb = blockIdx.y;
    if (n >= N) return;
    const uint16_t *src = reinterpret_cast<const uint16_t *>(raw + (size_t)(n * KB + kb) * BLOCK_BYTES);
    uint16_t *dst = reinterpret_cast<uint16_t *>(blocks + (size_t)(kb * N + n) * BLOCK_BYTES);
    uint8_t qs[16];
    dst[0] = __ldg(src);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const uint16_t two = __ldg(src + 1 + j);
        qs[2 * j] = (uint8_t)(two & 0xFF);
        qs[2 * j + 1] = (uint8_t)(two >> 8);
    }
    // value i of the block: i < 16 ? low nibble of byte i : high nibble of byte i - 16
#pragma unroll
    for (int j = 0; j < 8; ++j) {                       // output bytes 2j, 2j+1 hold values 4j .. 4j+3
        uint32_t v[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = 4 * j + i;
            v[i] = idx < 16 ? (qs[idx] & 0xF) : (qs[idx - 16] >> 4);
        }
        dst[1 + j] = (uint16_t)(v[0] | (v[1] << 4) | (v[2] << 8) | (v[3] << 12));
    }
}

template <typename T> __device__ __forceinline__ float ld_as_float(const T *p);
template <> __device__ __forceinline__ float ld_as_float<float>(const float *p) { return __ldg(p); }
template <> __device__ __forceinline__ float ld_as_float<__half>(const __half *p) { return __half2float(__ldg(p)); }
template <> __device__ __forceinline__ float ld_as_float<__nv_bfloat16>(const __nv_bfloat16 *p) { return __bfloat162float(__ldg(p)); }

// one thread per block; adjacent threads take adjacent columns
template <typename T>
__global__ void __launch_bounds__(128)
quantize_ggml_kernel(const T *__restrict__ w, int64_t K, int64_t N, int nk_layout, uint8_t *__restrict__ blocks) {
    const int64_t n = (int64_t)blockIdx.x * 128 + threadIdx.x;
    const int64_t kb = blockIdx.y;
    if (n >= N) return;
    float v[QK];
#pragma unroll
    for (int i = 0; i < QK; ++i) {
        const int64_t k = kb * QK + i;
        v[i] = ld_as_float<T>(nk_layout ? w + n * K + k : w + k * N + n);
    }
    float amax = 0.0f, vmax = 0.0f;                     // the first value of the largest magnitude
#pragma unroll
    for (int i = 0; i < QK; ++i) {
        const float a = fabsf(v[i]);
        if (a > amax) { amax = a; vmax = v[i]; }
    }
    const float d = vmax == 0.0f ? 0.0f : __fdiv_rn(vmax, -8.0f);       // +0 for an all-zero block
    uint16_t *dst = reinterpret_cast<uint16_t *>(blocks + (size_t)(kb * N + n) * BLOCK_BYTES);
    dst[0] = __half_as_ushort(__float2half_rn(d));
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        uint32_t word = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float t = 8.0f;
            if (d != 0.0f) t = fminf(fmaxf(__fadd_rn(rintf(__fdiv_rn(v[4 * j + i], d)), 8.0f), 0.0f), 15.0f);
            word |= (uint32_t)(int)t << (4 * i);
        }
        dst[1 + j] = (uint16_t)word;
    }
}

// ---- group-wise INT8 matmul ---------------------------------------------------------------------
constexpr int I8_THREADS = 256;                  // 8 warps split k
constexpr int I8_COLS = 32;                      // columns per CTA: 4 per lane, 8 lanes across
constexpr int I8_ROWS = 8;                       // rows of X per CTA
constexpr int I8_KC = 512;                       // k per shared-memory slice of X
constexpr int I8_UNROLL = 8;                     // weight loads in flight per lane

template <typename T> __device__ __forceinline__ T out_cast(float v);
template <> __device__ __forceinline__ __half out_cast<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 out_cast<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// int8 byte `sel` of word w as a float, exactly: the byte (offset by 128) is planted in the mantissa
// of 2^23 and the bias taken off again
__device__ __forceinline__ float byte_to_float(uint32_t w_xor80, int sel) {
    return __uint_as_float(__byte_perm(w_xor80, 0x4B000000u, 0x7650 | sel) & 0xFFFF00FFu | 0x4B000000u) - 8388736.0f;
}

// NIBBLES: wq is the group-wise INT4 format instead, uint8 [K/2, N], byte r of a column = value 2r in
// its low and value 2r + 1 in its high nibble (values 0..15).
//
// A CTA takes 32 columns and up to 8 rows of X.  A warp load covers four consecutive k rows of the
// weight, 32 bytes (one sector) of each: lane = (k row of the four, column quad).  The eight warps take
// the k rows 4w..4w+3, + 32, + 64, ...; eight loads per lane are issued before their values are used.
// (scale, zero) of the lane's columns are reloaded only when its k crosses into another group.  At the
// end the four k rows of a warp are summed by shuffles and the eight warps through shared memory, both
// in a fixed order.
template <typename TX, typename TS, bool NIBBLES>
__global__ void __launch_bounds__(I8_THREADS, 3)
int8g_matmul_kernel(const TX *__restrict__ x, int M, int64_t ldx, const int8_t *__restrict__ wq, const TS *__restrict__ scales,
                    const TS *__restrict__ zeros, int64_t K, int64_t N, int group, TX *__restrict__ y, int64_t ldy) {
    __shared__ __align__(16) float xs[I8_KC][I8_ROWS];       // [k][row]: a k's eight rows are two 16-byte reads
    __shared__ float red[I8_THREADS / 32][I8_ROWS][I8_COLS];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int cq = lane & 7, ks = lane >> 3;
    const int64_t n0 = (int64_t)blockIdx.x * I8_COLS + cq * 4;
    const int m0 = (int)blockIdx.y * I8_ROWS;
    const int rows = min(I8_ROWS, M - m0);
    const bool vec = (N % 4 == 0) && n0 + 3 < N;
    float acc[I8_ROWS][4];
#pragma unroll
    for (int r = 0; r < I8_ROWS; ++r)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[r][j] = 0.0f;
    float sc[4] = {0.0f, 0.0f, 0.0f, 0.0f}, zr[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    int64_t g_end = 0;                                  // the cached (scale, zero) hold for k < g_end

    for (int64_t kc = 0; kc < K; kc += I8_KC) {
        const int klen = (int)min((int64_t)I8_KC, K - kc);
        __syncthreads();
        for (int i = threadIdx.x; i < I8_ROWS * I8_KC; i += I8_THREADS) {
            const int r = i / I8_KC, k = i % I8_KC;                    // consecutive threads read consecutive k of a row
            xs[k][r] = (r < rows && k < klen) ? (float)x[(size_t)(m0 + r) * ldx + kc + k] : 0.0f;
        }
        __syncthreads();
        for (int t0 = 0; t0 < I8_KC / 32; t0 += I8_UNROLL) {
            if (t0 * 32 >= klen) break;                 // uniform over the CTA
            uint32_t word[I8_UNROLL];
#pragma unroll
            for (int u = 0; u < I8_UNROLL; ++u) {
                const int k = warp * 4 + ks + 32 * (t0 + u);
                const int64_t kk = kc + k;
                word[u] = 0;
                if (k < klen) {
                    const uint8_t *row = NIBBLES ? reinterpret_cast<const uint8_t *>(wq) + (kk >> 1) * N
                                                 : reinterpret_cast<const uint8_t *>(wq) + kk * N;
                    if (vec) {
                        word[u] = __ldg(reinterpret_cast<const uint32_t *>(row + n0));
                    } else {
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            if (n0 + j < N) word[u] |= (uint32_t)row[n0 + j] << (8 * j);
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < I8_UNROLL; ++u) {
                const int k = warp * 4 + ks + 32 * (t0 + u);
                if (k < klen) {
                    const int64_t kk = kc + k;
                    if (kk >= g_end) {                  // another group: its scale and zero point
                        const int64_t gi = kk / group;
                        g_end = (gi + 1) * (int64_t)group;
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const bool ok = n0 + j < N;
                            sc[j] = ok ? (float)scales[gi * N + n0 + j] : 0.0f;
                            zr[j] = ok ? (float)zeros[gi * N + n0 + j] : 0.0f;
                        }
                    }
                    float wv[4];
                    if constexpr (NIBBLES) {
                        const int sh = (int)(kk & 1) * 4;
#pragma unroll
                        for (int j = 0; j < 4; ++j) wv[j] = (float)((word[u] >> (8 * j + sh)) & 0xFu);
                    } else {
                        const uint32_t wx = word[u] ^ 0x80808080u;
#pragma unroll
                        for (int j = 0; j < 4; ++j) wv[j] = byte_to_float(wx, j);
                    }
#pragma unroll
                    for (int j = 0; j < 4; ++j) wv[j] = (wv[j] - zr[j]) * sc[j];      // (w_q - zero) * scale, as the reference
                    const float4 xa = *reinterpret_cast<const float4 *>(&xs[k][0]);
                    const float xr[4] = {xa.x, xa.y, xa.z, xa.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[0][j] = fmaf(xr[0], wv[j], acc[0][j]);
                    if (rows > 1) {                                 // uniform over the CTA: a single row is the common case
#pragma unroll
                        for (int r = 1; r < 4; ++r)
#pragma unroll
                            for (int j = 0; j < 4; ++j) acc[r][j] = fmaf(xr[r], wv[j], acc[r][j]);
                    }
                    if (rows > 4) {
                        const float4 xb = *reinterpret_cast<const float4 *>(&xs[k][4]);
                        const float xq[4] = {xb.x, xb.y, xb.z, xb.w};
#pragma unroll
                        for (int r = 0; r < 4; ++r)
#pragma unroll
                            for (int j = 0; j < 4; ++j) acc[4 + r][j] = fmaf(xq[r], wv[j], acc[4 + r][j]);
                    }
                }
            }
        }
    }
    // the warp's four k rows: lanes l, l + 8, l + 16, l + 24 hold the same columns
#pragma unroll
    for (int r = 0; r < I8_ROWS; ++r)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            acc[r][j] += __shfl_xor_sync(0xffffffffu, acc[r][j], 8);
            acc[r][j] += __shfl_xor_sync(0xffffffffu, acc[r][j], 16);
        }
    if (ks == 0) {
#pragma unroll
        for (int r = 0; r < I8_ROWS; ++r)
#pragma unroll
            for (int j = 0; j < 4; ++j) red[warp][r][cq * 4 + j] = acc[r][j];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < I8_ROWS * I8_COLS; i += I8_THREADS) {
        const int r = i / I8_COLS, cidx = i % I8_COLS;
        const int64_t n = (int64_t)blockIdx.x * I8_COLS + cidx;
        if (r < rows && n < N) {
            float s = 0.0f;
#pragma unroll
            for (int w = 0; w < I8_THREADS / 32; ++w) s += red[w][r][cidx];
            y[(size_t)(m0 + r) * ldy + n] = out_cast<TX>(s);
        }
    }
}

}  // namespace q4b

using namespace q4b;

extern "C" int q4b_import_ggml(const void *raw, int64_t K, int64_t N, void *blocks_out, void *stream) {
    if (raw == nullptr || blocks_out == nullptr || K <= 0 || N <= 0) return Q4B_ERR_ARG;
    if (K % QK || K / QK > 65535) return Q4B_ERR_SHAPE;
    if (!aligned(raw, 2) || !aligned(blocks_out, 2)) return Q4B_ERR_ALIGN;
    dim3 grid((unsigned)ceil_div(N, 128), (unsigned)(K / QK));
    import_ggml_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>((const uint8_t *)raw, K / QK, N, (uint8_t *)blocks_out);
    Q4B_LAUNCH_CHECK();
    return Q4B_OK;
}

extern "C" int q4b_quantize_ggml(const void *w, int w_dtype, int64_t K, int64_t N, int layout, void *blocks_out,
                                 void *prepacked_out, void *stream) {
    if (w == nullptr || blocks_out == nullptr || K <= 0 || N <= 0) return Q4B_ERR_ARG;
    if (layout != Q4B_LAYOUT_KN && layout != Q4B_LAYOUT_NK) return Q4B_ERR_ARG;
    if (K % QK || K / QK > 65535) return Q4B_ERR_SHAPE;
    if (!aligned(blocks_out, 2)) return Q4B_ERR_ALIGN;
    dim3 grid((unsigned)ceil_div(N, 128), (unsigned)(K / QK));
    cudaStream_t st = (cudaStream_t)stream;
    const int nk = layout == Q4B_LAYOUT_NK ? 1 : 0;
    switch (w_dtype) {
        case Q4B_F32: quantize_ggml_kernel<float><<<grid, 128, 0, st>>>((const float *)w, K, N, nk, (uint8_t *)blocks_out); break;
        case Q4B_F16: quantize_ggml_kernel<__half><<<grid, 128, 0, st>>>((const __half *)w, K, N, nk, (uint8_t *)blocks_out); break;
        case Q4B_BF16:
            quantize_ggml_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>((const __nv_bfloat16 *)w, K, N, nk, (uint8_t *)blocks_out);
            break;
        default: return Q4B_ERR_DTYPE;
    }
    Q4B_LAUNCH_CHECK();
    if (prepacked_out != nullptr) return q4b_repack(blocks_out, K, N, prepacked_out, stream);
    return Q4B_OK;
}

template <typename TX, typename TS, bool NIBBLES>
static int launch_int8g(const void *x, int64_t M, int64_t ldx, const void *wq, const void *scales, const void *zeros, int64_t K,
                        int64_t N, int64_t group, void *y, int64_t ldy, cudaStream_t st) {
    dim3 grid((unsigned)ceil_div(N, I8_COLS), (unsigned)ceil_div(M, I8_ROWS));
    int8g_matmul_kernel<TX, TS, NIBBLES><<<grid, I8_THREADS, 0, st>>>((const TX *)x, (int)M, ldx, (const int8_t *)wq,
                                                                     (const TS *)scales, (const TS *)zeros, K, N, (int)group,
                                                                     (TX *)y, ldy);
    Q4B_LAUNCH_CHECK();
    return Q4B_OK;
}

template <bool NIBBLES>
static int groupwise_matmul(const void *x, int x_dtype, int64_t M, int64_t ldx, const void *wq, const void *scales,
                            const void *zeros, int sz_dtype, int64_t K, int64_t N, int64_t group, void *y, int64_t ldy,
                            void *stream) {
    if (x == nullptr || wq == nullptr || scales == nullptr || zeros == nullptr || y == nullptr) return Q4B_ERR_ARG;
    if (M < 1 || K <= 0 || N <= 0 || group <= 0 || ldx < K || ldy < N) return Q4B_ERR_ARG;
    if (NIBBLES && (K % 2)) return Q4B_ERR_SHAPE;
    if (M > 65535LL * I8_ROWS || group > (1LL << 30)) return Q4B_ERR_TOO_LARGE;
    if (x_dtype != Q4B_F16 && x_dtype != Q4B_BF16) return Q4B_ERR_DTYPE;
    if (!aligned(wq, 4) || !aligned(x, 2) || !aligned(y, 2)) return Q4B_ERR_ALIGN;
    cudaStream_t st = (cudaStream_t)stream;
    const bool xb = x_dtype == Q4B_BF16;
    switch (sz_dtype) {
        case Q4B_F32:
            return xb ? launch_int8g<__nv_bfloat16, float, NIBBLES>(x, M, ldx, wq, scales, zeros, K, N, group, y, ldy, st)
                      : launch_int8g<__half, float, NIBBLES>(x, M, ldx, wq, scales, zeros, K, N, group, y, ldy, st);
        case Q4B_F16:
            return xb ? launch_int8g<__nv_bfloat16, __half, NIBBLES>(x, M, ldx, wq, scales, zeros, K, N, group, y, ldy, st)
                      : launch_int8g<__half, __half, NIBBLES>(x, M, ldx, wq, scales, zeros, K, N, group, y, ldy, st);
        case Q4B_BF16:
            return xb ? launch_int8g<__nv_bfloat16, __nv_bfloat16, NIBBLES>(x, M, ldx, wq, scales, zeros, K, N, group, y, ldy, st)
                      : launch_int8g<__half, __nv_bfloat16, NIBBLES>(x, M, ldx, wq, scales, zeros, K, N, group, y, ldy, st);
        default: return Q4B_ERR_DTYPE;
    }
}

extern "C" int q4b_int8g_matmul(const void *x, int x_dtype, int64_t M, int64_t ldx, const void *w_int8, const void *scales,
                                const void *zeros, int sz_dtype, int64_t K, int64_t N, int64_t group, void *y, int64_t ldy,
                                void *stream) {
    return groupwise_matmul<false>(x, x_dtype, M, ldx, w_int8, scales, zeros, sz_dtype, K, N, group, y, ldy, stream);
}

extern "C" int q4b_int4g_matmul_generic(const void *x, int x_dtype, int64_t M, int64_t ldx, const void *packed,
                                        const void *scales, const void *zeros, int sz_dtype, int64_t K, int64_t N, int64_t group,
                                        void *y, int64_t ldy, void *stream) {
    return groupwise_matmul<true>(x, x_dtype, M, ldx, packed, scales, zeros, sz_dtype, K, N, group, y, ldy, stream);
}
