// Decode path: Y[M, N] = X[M, K] . dequant(W) for 1 <= M <= 16, HBM-bound.
//
// Takes the role the reference gives to its 64x32-tile Metal kernel at small M
// (packages/metalcore/src/metalcore/native/quant_kernels.metal:1738-1886, launched by
// core_mps.mm:5917-5975), which has no GEMV specialisation.
//
// Each warp owns one 16-column tile and streams its share of the k range: per 64-k tile one
// 128-bit load of nibbles and one 64-bit load of scales per lane (the prepacked layout makes
// a lane's 16 bytes exactly its mma fragment), kept D tiles ahead in registers.  Nibbles are
// turned into (q-8) fp16/bf16 pairs in registers; the 16 columns form the 16-row A operand of
// mma.sync.m16n8k16 and up to 8 activation rows the B operand, so M = 1..8 costs the same and
// M = 9..16 one more fragment.  The per-block scale multiplies the fp32 partial product of
// each 32-k block, accumulation is fp32 throughout.  Warps of a CTA that share a column tile
// split k and are reduced through shared memory.
#include "q4b_common.cuh"

namespace q4b {

constexpr int GEMV_WARPS = 8;
constexpr int GEMV_THREADS = GEMV_WARPS * 32;
constexpr int GEMV_DEPTH = 4;      // tiles in flight per warp (register ring)

__device__ __forceinline__ uint4 ldg_stream_v4(const void *p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}
__device__ __forceinline__ uint2 ldg_stream_v2(const void *p) {
    uint2 r;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(r.x), "=r"(r.y) : "l"(p));
    return r;
}
__device__ __forceinline__ uint4 ld_x_v4(const void *p) {
    uint4 r;
    asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p) : "memory");
    return r;
}

template <bool BF16>
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1, const float (&z)[4]) {
    if constexpr (BF16) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
                     : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(z[0]), "f"(z[1]), "f"(z[2]), "f"(z[3]));
    } else {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
                     : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(z[0]), "f"(z[1]), "f"(z[2]), "f"(z[3]));
    }
}

template <bool BF16> __device__ __forceinline__ uint16_t out_bits(float v) {
    if constexpr (BF16) return __bfloat16_as_ushort(__float2bfloat16_rn(v));
    else return __half_as_ushort(__float2half_rn(v));
}

// KS = warps of a CTA that split k for the same column tile; the CTA covers 8/KS column tiles.
template <bool BF16, int MF, int KS>
__global__ void __launch_bounds__(GEMV_THREADS)
gemv_kernel(const uint16_t *__restrict__ x, int M, int64_t ldx, const uint8_t *__restrict__ prepacked, int64_t K,
            int64_t N, uint16_t *__restrict__ y, int64_t ldy) {
    constexpr int NTC = GEMV_WARPS / KS;
    __shared__ float red[GEMV_WARPS][MF][TILE_N * 8];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, c = lane & 3;
    const int ks = warp % KS, ntl = warp / KS;
    const int64_t NT = tiles_n(N);
    const int KU = (int)tiles_k(K);
    const int64_t nt = (int64_t)blockIdx.x * NTC + ntl;
    const bool active = nt < NT;
    const int ku0 = (int)((int64_t)KU * ks / KS), ku1 = (int)((int64_t)KU * (ks + 1) / KS);

    const uint8_t *wbase = prepacked + (size_t)(active ? nt : 0) * TILE_BYTES;
    const size_t wstride = (size_t)NT * TILE_BYTES;
    const int qoff = (c * 8 + g) * 16, doff = TILE_QS_BYTES + g * 8;

    uint4 qbuf[GEMV_DEPTH];
    uint2 dbuf[GEMV_DEPTH];
#pragma unroll
    for (int i = 0; i < GEMV_DEPTH; ++i) {
        if (active && ku0 + i < ku1) {
            const uint8_t *t = wbase + (size_t)(ku0 + i) * wstride;
            qbuf[i] = ldg_stream_v4(t + qoff);
            dbuf[i] = ldg_stream_v2(t + doff);
        }
    }
    // Weights never depend on earlier kernels of the stream; x and y do.  Under programmatic
    // dependent launch the loads above overlap the previous kernel's tail.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    float acc[MF][4];
#pragma unroll
    for (int f = 0; f < MF; ++f)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[f][i] = 0.0f;
    const float zero4[4] = {0.0f, 0.0f, 0.0f, 0.0f};

    const uint16_t *xrow[MF];
#pragma unroll
    for (int f = 0; f < MF; ++f) xrow[f] = x + (size_t)min(f * 8 + g, M - 1) * ldx + c * 8;

    if (active) {
        for (int kub = ku0; kub < ku1; kub += GEMV_DEPTH) {
#pragma unroll
            for (int i = 0; i < GEMV_DEPTH; ++i) {
                const int ku = kub + i;
                if (ku < ku1) {
                    const uint4 qw = qbuf[i];
                    const uint2 dw = dbuf[i];
                    if (ku + GEMV_DEPTH < ku1) {
                        const uint8_t *t = wbase + (size_t)(ku + GEMV_DEPTH) * wstride;
                        qbuf[i] = ldg_stream_v4(t + qoff);
                        dbuf[i] = ldg_stream_v2(t + doff);
                    }
#pragma unroll
                    for (int kbl = 0; kbl < TILE_KB; ++kbl) {
                        const int64_t k = (int64_t)ku * TILE_K + kbl * QK;
                        uint32_t hlo[4], hhi[4];
                        dequant_word<BF16>(kbl ? qw.z : qw.x, hlo);     // column g
                        dequant_word<BF16>(kbl ? qw.w : qw.y, hhi);     // column g + 8
                        const uint32_t dpair = kbl ? dw.y : dw.x;
                        const float dlo = __half2float(__ushort_as_half((uint16_t)(dpair & 0xFFFF)));
                        const float dhi = __half2float(__ushort_as_half((uint16_t)(dpair >> 16)));
#pragma unroll
                        for (int f = 0; f < MF; ++f) {
                            uint4 xv = make_uint4(0u, 0u, 0u, 0u);
                            if (k < K) xv = ld_x_v4(xrow[f] + k);       // the pad block of an odd K/32 has d = 0
                            float part[4];
                            mma16816<BF16>(part, hlo[0], hhi[0], hlo[1], hhi[1], xv.x, xv.y, zero4);
                            mma16816<BF16>(part, hlo[2], hhi[2], hlo[3], hhi[3], xv.z, xv.w, part);
                            acc[f][0] = fmaf(dlo, part[0], acc[f][0]);
                            acc[f][1] = fmaf(dlo, part[1], acc[f][1]);
                            acc[f][2] = fmaf(dhi, part[2], acc[f][2]);
                            acc[f][3] = fmaf(dhi, part[3], acc[f][3]);
                        }
                    }
                }
            }
        }
    }

    // acc[f][0..1] = column g, rows f*8 + 2c, 2c+1 ; acc[f][2..3] = column g+8, same rows
#pragma unroll
    for (int f = 0; f < MF; ++f) {
        red[warp][f][(2 * c) * TILE_N + g] = acc[f][0];
        red[warp][f][(2 * c + 1) * TILE_N + g] = acc[f][1];
        red[warp][f][(2 * c) * TILE_N + g + 8] = acc[f][2];
        red[warp][f][(2 * c + 1) * TILE_N + g + 8] = acc[f][3];
    }
    __syncthreads();
    for (int o = threadIdx.x; o < NTC * MF * 8 * TILE_N; o += GEMV_THREADS) {
        const int nl = o % TILE_N;
        const int m8 = (o / TILE_N) % 8;
        const int f = (o / (TILE_N * 8)) % MF;
        const int tl = o / (TILE_N * 8 * MF);
        const int m = f * 8 + m8;
        const int64_t n = ((int64_t)blockIdx.x * NTC + tl) * TILE_N + nl;
        if (m < M && n < N) {
            float s = 0.0f;
#pragma unroll
            for (int j = 0; j < KS; ++j) s += red[tl * KS + j][f][m8 * TILE_N + nl];
            y[(size_t)m * ldy + n] = out_bits<BF16>(s);
        }
    }
}

template <bool BF16, int MF, int KS>
static int launch_gemv(const void *x, int M, int64_t ldx, const void *prepacked, int64_t K, int64_t N, void *y,
                       int64_t ldy, int flags, cudaStream_t st) {
    constexpr int NTC = GEMV_WARPS / KS;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)ceil_div(tiles_n(N), NTC));
    cfg.blockDim = dim3(GEMV_THREADS);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (flags & Q4B_FLAG_PDL) ? 1 : 0;
    Q4B_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemv_kernel<BF16, MF, KS>, (const uint16_t *)x, M, ldx,
                                    (const uint8_t *)prepacked, K, N, (uint16_t *)y, ldy));
    return Q4B_OK;
}

template <bool BF16, int MF>
static int launch_gemv_ks(int ksplit, const void *x, int M, int64_t ldx, const void *prepacked, int64_t K, int64_t N,
                          void *y, int64_t ldy, int flags, cudaStream_t st) {
    switch (ksplit) {
        case 8: return launch_gemv<BF16, MF, 8>(x, M, ldx, prepacked, K, N, y, ldy, flags, st);
        case 4: return launch_gemv<BF16, MF, 4>(x, M, ldx, prepacked, K, N, y, ldy, flags, st);
        case 2: return launch_gemv<BF16, MF, 2>(x, M, ldx, prepacked, K, N, y, ldy, flags, st);
        default: return launch_gemv<BF16, MF, 1>(x, M, ldx, prepacked, K, N, y, ldy, flags, st);
    }
}

int device_sm_count();
int gemv_ksplit_override();

}  // namespace q4b

using namespace q4b;

extern "C" int q4b_gemv(const void *x, int x_dtype, int64_t M, int64_t ldx, const void *prepacked, int64_t K,
                        int64_t N, void *y, int64_t ldy, int flags, void *stream) {
    if (x == nullptr || prepacked == nullptr || y == nullptr) return Q4B_ERR_ARG;
    if (M < 1 || K <= 0 || N <= 0 || ldx < K || ldy < N) return Q4B_ERR_ARG;
    if (M > 16 || K % QK || tiles_k(K) > (1 << 24)) return Q4B_ERR_SHAPE;
    if (x_dtype != Q4B_F16 && x_dtype != Q4B_BF16) return Q4B_ERR_DTYPE;
    if (!aligned(x, 16) || (ldx % 8) || !aligned(prepacked, 16) || !aligned(y, 2)) return Q4B_ERR_ALIGN;
    // k-split: as few splits as still give every SM several CTAs, never more splits than tiles
    const int64_t NT = tiles_n(N), KU = tiles_k(K);
    int ks = gemv_ksplit_override();
    if (ks == 0) {
        const int64_t want = 4LL * device_sm_count();
        ks = 8;
        while (ks > 1 && ceil_div(NT, GEMV_WARPS / (ks / 2)) >= want) ks /= 2;
    }
    while (ks > 1 && KU < ks) ks /= 2;
    cudaStream_t st = (cudaStream_t)stream;
    const bool bf = x_dtype == Q4B_BF16;
    if (M <= 8)
        return bf ? launch_gemv_ks<true, 1>(ks, x, (int)M, ldx, prepacked, K, N, y, ldy, flags, st)
                  : launch_gemv_ks<false, 1>(ks, x, (int)M, ldx, prepacked, K, N, y, ldy, flags, st);
    return bf ? launch_gemv_ks<true, 2>(ks, x, (int)M, ldx, prepacked, K, N, y, ldy, flags, st)
              : launch_gemv_ks<false, 2>(ks, x, (int)M, ldx, prepacked, K, N, y, ldy, flags, st);
}
