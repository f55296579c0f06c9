// Decode path: Y[M, N] = X[M, K] . dequant(W) for 1 <= M <= 16, HBM-bound.
//
// Takes the role the reference gives to its 64x32-tile Metal kernel at small M
// (packages/metalcore/src/metalcore/native/quant_kernels.metal:1738-1886, launched by
// core_mps.mm:5917-5975), which has no GEMV specialisation.
//
// Each warp owns one 16-column tile and a contiguous range of its k tiles, which is one
// contiguous run of bytes in the column-tile-major prepacked layout.  Lane 0 feeds a per-warp
// ring in shared memory with bulk asynchronous copies (cp.async.bulk, completion counted on an
// mbarrier per ring slot), so the bytes in flight per SM are set by the ring size, not by
// registers.  Lanes read their 16 bytes of nibbles and 8 bytes of scales from the ring
// (conflict free), turn the nibbles into (q-8) fp16/bf16 pairs in registers, and feed them as
// the 16-row A operand of mma.sync.m16n8k16; up to 8 activation rows are the B operand, so
// M = 1..8 costs the same and M = 9..16 one more fragment.  The per-block scale multiplies the
// fp32 partial product of each 32-k block; accumulation is fp32 throughout.  Warps of a CTA
// that share a column tile split k and are reduced through shared memory.
//
// Every mbarrier wait is bounded: a wait that gives up sets g_wait_status, and the warp stops
// consuming (its outputs are then wrong, which the status reports) instead of spinning.
#include "q4b_common.cuh"

namespace q4b {

constexpr int GEMV_WARPS = 8;
constexpr int GEMV_THREADS = GEMV_WARPS * 32;
constexpr int GEMV_CHUNK = 4;                       // tiles per bulk copy (2304 bytes)
constexpr int GEMV_SLOTS = 3;                       // ring slots per warp
constexpr int GEMV_SLOT_BYTES = GEMV_CHUNK * TILE_BYTES;
constexpr int GEMV_RING_BYTES = GEMV_SLOTS * GEMV_SLOT_BYTES;          // 6912 per warp
constexpr int GEMV_SMEM_DYN = GEMV_WARPS * GEMV_RING_BYTES;            // 55296 per CTA: 3 CTAs per SM
constexpr int GEMV_SPIN_LIMIT = 1 << 22;            // try_wait polls before giving up (~0.1 s)

__device__ int g_wait_status = 0;                  // first bounded wait of this file that gave up

__device__ __forceinline__ uint32_t smem_addr_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

template <bool BF16>
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1, const float (&z)[4]) {
    if constexpr (BF16) {
        asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
            : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(z[0]), "f"(z[1]), "f"(z[2]), "f"(z[3]));
    } else {
        asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
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
    extern __shared__ __align__(128) uint8_t ring_all[];
    __shared__ __align__(8) uint64_t bars[GEMV_WARPS][GEMV_SLOTS];
    __shared__ float red[GEMV_WARPS][MF][TILE_N * 8];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, c = lane & 3;
    const int ks = warp % KS, ntl = warp / KS;
    const int64_t NT = tiles_n(N);
    const int KU = (int)tiles_k(K);
    const int64_t nt = (int64_t)blockIdx.x * NTC + ntl;
    const bool active = nt < NT;
    const int ku0 = (int)((int64_t)KU * ks / KS), ku1 = (int)((int64_t)KU * (ks + 1) / KS);
    const int ntiles = active ? ku1 - ku0 : 0;
    const int nchunks = (ntiles + GEMV_CHUNK - 1) / GEMV_CHUNK;

    const uint8_t *ring = ring_all + warp * GEMV_RING_BYTES;
    const uint32_t ring_s = smem_addr_u32(ring);
    const uint32_t bar_s = smem_addr_u32(&bars[warp][0]);
    const uint8_t *src = prepacked + tile_offset(active ? nt : 0, ku0, KU);

    auto issue = [&](int ci) {          // lane 0 only: arm the slot and start its bulk copy
        const int slot = ci % GEMV_SLOTS;
        const uint32_t bytes = (uint32_t)(min(GEMV_CHUNK, ntiles - ci * GEMV_CHUNK) * TILE_BYTES);
        const uint32_t bar = bar_s + 8u * slot;
        asm volatile("{ .reg .b64 t; mbarrier.arrive.expect_tx.shared::cta.b64 t, [%0], %1; }" ::"r"(bar), "r"(bytes) : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(ring_s + (uint32_t)(slot * GEMV_SLOT_BYTES)), "l"(src + (size_t)ci * GEMV_SLOT_BYTES), "r"(bytes), "r"(bar)
                     : "memory");
    };

    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < GEMV_SLOTS; ++s)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_s + 8u * s) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
#pragma unroll
        for (int s = 0; s < GEMV_SLOTS; ++s)
            if (s < nchunks) issue(s);
    }
    __syncwarp();
    // Weights never depend on earlier kernels of the stream; x and y do.  Under programmatic
    // dependent launch the copies above overlap the previous kernel's tail.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    float acc[MF][4];
#pragma unroll
    for (int f = 0; f < MF; ++f)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[f][i] = 0.0f;
    const float zero4[4] = {0.0f, 0.0f, 0.0f, 0.0f};

    const uint4 *xrow[MF];
#pragma unroll
    for (int f = 0; f < MF; ++f)
        xrow[f] = reinterpret_cast<const uint4 *>(x + (size_t)min(f * 8 + g, M - 1) * ldx + c * 8);

    const int qoff = slot_of(g, c) * 16, doff = TILE_QS_BYTES + g * 8;
    bool ok = true;
    for (int ci = 0; ci < nchunks && ok; ++ci) {
        const int slot = ci % GEMV_SLOTS;
        const uint32_t parity = (uint32_t)((ci / GEMV_SLOTS) & 1);
        const uint32_t bar = bar_s + 8u * slot;
        int spins = 0;
        while (true) {
            uint32_t done;
            asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                         : "=r"(done) : "r"(bar), "r"(parity) : "memory");
            if (done) break;
            if (++spins > GEMV_SPIN_LIMIT) {
                atomicCAS(&g_wait_status, 0, 100);
                ok = false;
                break;
            }
        }
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const uint8_t *sl = ring + slot * GEMV_SLOT_BYTES;
        const int tiles_here = min(GEMV_CHUNK, ntiles - ci * GEMV_CHUNK);
#pragma unroll
        for (int t = 0; t < GEMV_CHUNK; ++t) {
            if (t < tiles_here) {
                const uint4 qw = *reinterpret_cast<const uint4 *>(sl + t * TILE_BYTES + qoff);
                const uint2 dw = *reinterpret_cast<const uint2 *>(sl + t * TILE_BYTES + doff);
                const int ku = ku0 + ci * GEMV_CHUNK + t;
#pragma unroll
                for (int kbl = 0; kbl < TILE_KB; ++kbl) {
                    const int64_t k = (int64_t)ku * TILE_K + kbl * QK;
                    uint32_t hlo[4], hhi[4];
                    dequant_word<BF16>(kbl ? qw.z : qw.x, hlo);     // column g
                    dequant_word<BF16>(kbl ? qw.w : qw.y, hhi);     // column g + 8
                    const __half2 dh = *reinterpret_cast<const __half2 *>(kbl ? &dw.y : &dw.x);
                    const float2 df = __half22float2(dh);           // (d of column g, d of column g+8)
#pragma unroll
                    for (int f = 0; f < MF; ++f) {
                        uint4 xv = make_uint4(0u, 0u, 0u, 0u);
                        if (k < K) xv = xrow[f][k >> 3];            // the pad block of an odd K/32 has d = 0
                        float part[4];
                        mma16816<BF16>(part, hlo[0], hhi[0], hlo[1], hhi[1], xv.x, xv.y, zero4);
                        mma16816<BF16>(part, hlo[2], hhi[2], hlo[3], hhi[3], xv.z, xv.w, part);
                        acc[f][0] = fmaf(df.x, part[0], acc[f][0]);
                        acc[f][1] = fmaf(df.x, part[1], acc[f][1]);
                        acc[f][2] = fmaf(df.y, part[2], acc[f][2]);
                        acc[f][3] = fmaf(df.y, part[3], acc[f][3]);
                    }
                }
            }
        }
        __syncwarp();                    // every lane has consumed the slot before it is refilled
        if (lane == 0 && ci + GEMV_SLOTS < nchunks) issue(ci + GEMV_SLOTS);
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
    const int mrows = min(M - 0, MF * 8);
    for (int o = threadIdx.x; o < NTC * mrows * TILE_N; o += GEMV_THREADS) {
        const int nl = o % TILE_N;
        const int m = (o / TILE_N) % mrows;
        const int tl = o / (TILE_N * mrows);
        const int f = m >> 3, m8 = m & 7;
        const int64_t n = ((int64_t)blockIdx.x * NTC + tl) * TILE_N + nl;
        if (n < N) {
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
    // opt in to > 48 KB of dynamic shared memory once per device and instantiation
    static bool attr_done[64] = {};
    int dev = 0;
    Q4B_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
        Q4B_CUDA_TRY(cudaFuncSetAttribute(gemv_kernel<BF16, MF, KS>, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMV_SMEM_DYN));
        if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)ceil_div(tiles_n(N), NTC));
    cfg.blockDim = dim3(GEMV_THREADS);
    cfg.dynamicSmemBytes = GEMV_SMEM_DYN;
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

// read and clear this file's wait status (host side; the caller has synchronised the stream)
int gemv_wait_status(int *value) {
    int h = 0;
    Q4B_CUDA_TRY(cudaMemcpyFromSymbol(&h, g_wait_status, sizeof(int)));
    if (h != 0) {
        const int zero = 0;
        Q4B_CUDA_TRY(cudaMemcpyToSymbol(g_wait_status, &zero, sizeof(int)));
    }
    *value = h;
    return Q4B_OK;
}

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
