// Prefill path: Y[M, N] = X[M, K] . dequant(W) on the 5th-generation tensor cores.
//
// Replaces the reference's 64x32-tile simdgroup kernel matmul_ggml_q4_0
// (packages/metalcore/src/metalcore/native/quant_kernels.metal:1738-1886, launched by
// core_mps.mm:5917-5975) for M above the decode range.
//
// One persistent CTA per SM, tile 256 (M) x 256 (N), 64 k per pipeline step.  The two 128-row
// halves of the tile are two UMMA instructions that share the dequantised B operand, so every
// weight is dequantised once per 256 rows of X.  Three independent rings in shared memory:
//   A ring (3 x 32 KB)  warp 0: TMA tile loads of X (256 x 64, 128-byte swizzle)
//   W ring (4 x 9 KB)   warp 6: bulk copies of the step's packed weights (16 tiles of 576 bytes,
//                       one per lane)
//   B ring (2 x 32 KB)  warps 7-14 (two prepacked tiles each) dequantise a W stage into the K-major, 128-byte-swizzled
//                       bf16/fp16 B operand ((q-8)*d, one rounding) and fence to the async proxy
//   warp 1      one thread issues tcgen05.mma (kind::f16, M128 N256 K16), 2 halves x 4 per step,
//               accumulating in TMEM (2 x 256 columns); tcgen05.commit releases A and B stages
//   warps 2-5, 15-18  epilogue: tcgen05.ld the fp32 accumulators, convert, 16-byte stores; the
//               next tile's loads and dequantisation run underneath it
// The W ring is deep because only the dequantisers wait on it; the B ring needs two stages as
// long as dequantising a stage is faster than its 8 MMAs.
// Every mbarrier wait is bounded; a wait that gives up records a code in g_gemm_status, raises
// a CTA-wide abort flag and every role leaves through the common exit that frees TMEM.
#include <cuda.h>

#include <mutex>

#include "q4b_common.cuh"

namespace q4b {
namespace gemm {

constexpr int BM = 256, BN = 256, BK = 64, HALF_M = 128;
constexpr int SA = 3, SB = 3;                        // ring depths of the X and B operand stages
constexpr int SW_MAX = 16;                           // packed-weight ring: depth chosen per launch, see w_ring_depth
constexpr int A_BYTES = BM * BK * 2;                 // 32768
constexpr int A_HALF_BYTES = HALF_M * BK * 2;        // 16384
constexpr int B_BYTES = BN * BK * 2;                 // 32768
constexpr int W_TILES = BN / TILE_N;                 // 16 prepacked tiles per step
constexpr int NUM_DEQ_WARPS = 8;                     // prepacked tiles of a step are dealt round-robin to these warps
constexpr int WARP_A = 0, WARP_MMA = 1, WARP_W = 6, FIRST_DEQ_WARP = 7;   // warps 2..5: epilogue
constexpr int FIRST_EPI2_WARP = FIRST_DEQ_WARP + NUM_DEQ_WARPS;   // four more epilogue warps
constexpr int THREADS = (FIRST_EPI2_WARP + 4) * 32;              // 608
constexpr int TMEM_COLS = 512;                       // one 256-column fp32 accumulator per half
constexpr int SMEM_A = 0;
constexpr int SMEM_B = SMEM_A + SA * A_BYTES;
constexpr int SMEM_BAR = SMEM_B + SB * B_BYTES;
constexpr int NUM_BARS = 2 * (SA + SW_MAX + SB) + 2;
constexpr int SMEM_W = SMEM_BAR + ((NUM_BARS * 8 + 127) / 128) * 128;
constexpr int SMEM_DYN = 227 * 1024 - 256;           // all a CTA may have, less the few static words
constexpr int SMEM_W_BYTES = SMEM_DYN - 1024 - SMEM_W;   // 1024: slack to align the base
// Packed weights arrive about a microsecond after they are asked for, whatever the step length, so
// the ring holds as many steps as shared memory allows: 7 at 256 columns per tile, 14 at 128.  A
// short step (few rows of X) then still has enough bytes in flight to keep HBM busy.
__host__ __device__ inline int w_ring_depth(int bn) {
    const int d = SMEM_W_BYTES / ((bn / TILE_N) * TILE_BYTES);
    return d < SW_MAX ? d : SW_MAX;
}
constexpr long long WAIT_LIMIT_CYCLES = 1LL << 28;   // ~0.15 s; far above any legitimate wait

__device__ int g_gemm_status = 0;

// ---- thin PTX wrappers ---------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("{ .reg .b64 t; mbarrier.arrive.shared::cta.b64 t, [%0]; }" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("{ .reg .b64 t; mbarrier.arrive.expect_tx.shared::cta.b64 t, [%0], %1; }" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false when another role aborted or when this wait itself ran out, in
// which case it records `code` (first writer wins) and raises the CTA-wide abort flag.
// The abort flag and the clock are looked at every 64 polls only, and SLEEP_NS > 0 backs the
// polling off, so that a waiting thread costs few issue slots and little power.
template <int SLEEP_NS = 0>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    long long t0 = 0;
    for (int it = 1;; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if (SLEEP_NS > 0) __nanosleep(SLEEP_NS);
        if ((it & 63) == 0) {
            if (*abort_flag) return false;
            const long long now = clock64();
            if (t0 == 0) t0 = now;
            else if (now - t0 > WAIT_LIMIT_CYCLES) {
                *abort_flag = 1;
                atomicCAS(&g_gemm_status, 0, code);
                return false;
            }
        }
    }
}
// Whole-warp wait: every lane polls (one polling lane plus a warp barrier measured no faster).
template <int SLEEP_NS = 0>
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int *abort_flag, int code, int lane) {
    (void)lane;
    return __all_sync(0xffffffffu, mbar_wait<SLEEP_NS>(bar, parity, abort_flag, code));
}
// true on one lane of the (converged) warp
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{ .reg .pred p; elect.sync _|p, 0xffffffff; selp.u32 %0, 1, 0, p; }" : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p; }"
                 ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major operand tile stored as rows of 128 bytes
// (64 16-bit elements) with the 128-byte swizzle: 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t make_kmajor_sw128_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);     // start address, 16-byte units
    d |= (uint64_t)1 << 16;                          // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;                // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                          // descriptor version for sm_100
    d |= (uint64_t)2 << 61;                          // SWIZZLE_128B
    return d;
}
// Instruction descriptor: kind::f16, fp32 accumulate, A and B K-major, dense.
__host__ __device__ constexpr uint32_t make_idesc(bool bf16, int m, int n) {
    return (1u << 4)                              // D format f32
           | ((bf16 ? 1u : 0u) << 7)              // A format
           | ((bf16 ? 1u : 0u) << 10)             // B format
           | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

template <bool BF16> __device__ __forceinline__ uint32_t pack2_out(float a, float b) {
    if constexpr (BF16) {
        __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t *>(&v);
    } else {
        __half2 v = __floats2half2_rn(a, b);
        return *reinterpret_cast<uint32_t *>(&v);
    }
}
// fp16 scale bits -> packed pair (d, d) in the operand dtype
template <bool BF16> __device__ __forceinline__ uint32_t scale_pair(uint16_t dbits) {
    if constexpr (BF16) {
        __nv_bfloat16 b = __float2bfloat16_rn(__half2float(__ushort_as_half(dbits)));
        uint32_t u = __bfloat16_as_ushort(b);
        return u | (u << 16);
    } else {
        return (uint32_t)dbits | ((uint32_t)dbits << 16);
    }
}

// A ring index with its mbarrier phase
struct RingPos {
    int s = 0;
    uint32_t phase = 0;
    __device__ __forceinline__ void advance(int depth) {
        if (++s == depth) { s = 0; phase ^= 1; }
    }
};

template <bool BF16>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_x, const uint8_t *__restrict__ prepacked,
                    uint16_t *__restrict__ y, int M, int N, int K, int64_t ldy, int vec_store, int num_nt, int bn_max,
                    const float *__restrict__ addend, int64_t ld_add, int act) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;

    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    const uint32_t bar0 = base + SMEM_BAR;
    auto bar_full_a = [&](int s) { return bar0 + 8u * s; };                          // X tile landed
    auto bar_empty_a = [&](int s) { return bar0 + 8u * (SA + s); };                  // its MMAs retired
    auto bar_full_w = [&](int s) { return bar0 + 8u * (2 * SA + s); };               // packed weights landed
    auto bar_empty_w = [&](int s) { return bar0 + 8u * (2 * SA + SW_MAX + s); };         // dequantisers done reading
    auto bar_full_b = [&](int s) { return bar0 + 8u * (2 * SA + 2 * SW_MAX + s); };      // B operand written
    auto bar_empty_b = [&](int s) { return bar0 + 8u * (2 * SA + 2 * SW_MAX + SB + s); };  // its MMAs retired
    const uint32_t bar_tfull = bar0 + 8u * (2 * (SA + SW_MAX + SB));                     // accumulators complete
    const uint32_t bar_tempty = bar_tfull + 8u;                                      // accumulators drained

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int *abort_flag = &s_abort;

    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int s = 0; s < SA; ++s) { mbar_init(bar_full_a(s), 1); mbar_init(bar_empty_a(s), 1); }
        for (int s = 0; s < SW_MAX; ++s) { mbar_init(bar_full_w(s), 1); mbar_init(bar_empty_w(s), NUM_DEQ_WARPS); }
        for (int s = 0; s < SB; ++s) { mbar_init(bar_full_b(s), NUM_DEQ_WARPS); mbar_init(bar_empty_b(s), 1); }
        mbar_init(bar_tfull, 1);
        mbar_init(bar_tempty, 8);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == WARP_MMA) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = s_tmem_base;

    const int NT = (int)tiles_n(N);                    // prepacked 16-column tiles
    // The NT sixteen-column units are dealt to num_nt tiles as evenly as possible (widths differ by at
    // most one unit, none wider than bn_max): the host picks num_nt so that the tile count fills whole
    // waves of CTAs, which a single fixed width rarely does.
    auto unit0 = [&](int i) { return (int)((long long)i * NT / num_nt); };
    const int sw = w_ring_depth(bn_max);               // packed-weight ring: depth and stage size
    const int w_stage = (bn_max / TILE_N) * TILE_BYTES;
    const int num_mt = (M + BM - 1) / BM;
    const int num_tiles = num_mt * num_nt;
    const int k_steps = (K + BK - 1) / BK;

    if (warp == WARP_A) {
        // ---------------- X producer ----------------
        if (lane == 0) {
            RingPos a;
            for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
                const int mt = t % num_mt;
                for (int ks = 0; ks < k_steps; ++ks) {
                    if (!mbar_wait(bar_empty_a(a.s), a.phase ^ 1, abort_flag, 1)) goto done;
                    mbar_arrive_expect_tx(bar_full_a(a.s), (uint32_t)(M <= HALF_M ? A_HALF_BYTES : A_BYTES));
                    tma_load_2d(base + SMEM_A + a.s * A_BYTES, &tmap_x, ks * BK, mt * BM, bar_full_a(a.s));
                    a.advance(SA);
                }
            }
        }
    } else if (warp == WARP_W) {
        // ---------------- packed-weight producer ----------------
        // Lane i copies column tile i of the step: sixteen copies issued side by side instead of
        // one thread working through them (which was slower than the MMAs they feed).
        RingPos w;
        for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
            const int nt0 = unit0(t / num_mt);
            const int valid = unit0(t / num_mt + 1) - nt0;
            // the step's column tiles are k_steps tiles apart in the column-tile-major layout
            const uint8_t *src = prepacked + tile_offset(nt0 + min(lane, valid - 1), 0, k_steps);
            for (int ks = 0; ks < k_steps; ++ks) {
                if (!mbar_wait_warp(bar_empty_w(w.s), w.phase ^ 1, abort_flag, 7, lane)) goto done;
                if (lane == 0) mbar_arrive_expect_tx(bar_full_w(w.s), (uint32_t)(valid * TILE_BYTES));
                __syncwarp();
                if (lane < valid)
                    bulk_load(base + SMEM_W + w.s * w_stage + lane * TILE_BYTES, src + (size_t)ks * TILE_BYTES, TILE_BYTES,
                              bar_full_w(w.s));
                w.advance(sw);
            }
        }
    } else if (warp == WARP_MMA) {
        // ---------------- MMA issuer ----------------
        // The whole warp runs the loop, converged, and one elected lane issues: the operands of
        // tcgen05.mma then live in uniform registers instead of being moved there per instruction.
        {
            RingPos a, b;
            uint32_t tphase = 0;
            for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
                const int mt = t % num_mt;
                const uint32_t idesc = make_idesc(BF16, HALF_M, (unit0(t / num_mt + 1) - unit0(t / num_mt)) * TILE_N);
                const int halves = (M - mt * BM > HALF_M) ? 2 : 1;     // skip an all-padding lower half
                if (!mbar_wait_warp(bar_tempty, tphase ^ 1, abort_flag, 2, lane)) goto done;
                tc_fence_after();
                for (int ks = 0; ks < k_steps; ++ks) {
                    if (!mbar_wait_warp(bar_full_a(a.s), a.phase, abort_flag, 3, lane)) goto done;
                    if (!mbar_wait_warp(bar_full_b(b.s), b.phase, abort_flag, 4, lane)) goto done;
                    tc_fence_after();
                    if (elect_one()) {
                        const uint64_t bdesc = make_kmajor_sw128_desc(base + SMEM_B + b.s * B_BYTES);
                        for (int h = 0; h < halves; ++h) {
                            const uint64_t adesc = make_kmajor_sw128_desc(base + SMEM_A + a.s * A_BYTES + h * A_HALF_BYTES);
#pragma unroll
                            for (int k = 0; k < BK / 16; ++k)             // +32 bytes per k16 inside the swizzle atom
                                tc_mma_f16(tmem_base + (uint32_t)(h * BN), adesc + 2 * k, bdesc + 2 * k, idesc, (ks | k) != 0);
                        }
                        tc_commit(bar_empty_a(a.s));
                        tc_commit(bar_empty_b(b.s));
                        if (ks == k_steps - 1) tc_commit(bar_tfull);
                    }
                    __syncwarp();
                    a.advance(SA);
                    b.advance(SB);
                }
                tphase ^= 1;
            }
        }
    } else if (warp < WARP_W || warp >= FIRST_EPI2_WARP) {
        // ---------------- epilogue: two warps per TMEM lane quadrant, alternate 32-column chunks ----
        const int quad = warp & 3;                      // TMEM lane quadrant this warp may read
        const int grp = warp >= FIRST_EPI2_WARP ? 1 : 0;
        uint32_t tphase = 0;
        for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
            const int mt = t % num_mt, nt = t / num_mt;
            const int halves = (M - mt * BM > HALF_M) ? 2 : 1;
            if (!mbar_wait_warp<256>(bar_tfull, tphase, abort_flag, 5, lane)) goto done;
            tc_fence_after();
            const int n_base = unit0(nt) * TILE_N;
            const int n_end = min(N, unit0(nt + 1) * TILE_N);          // this tile's columns end here
            const int bn = unit0(nt + 1) * TILE_N - n_base;
            for (int h = 0; h < halves; ++h) {
                const int m = mt * BM + h * HALF_M + quad * 32 + lane;
                uint16_t *yrow = y + (size_t)m * ldy;
#pragma unroll 1
                for (int ch = grp; ch < (bn + 31) / 32; ch += 2) {
                    uint32_t r[32];
                    tc_ld_32x32b_x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(h * BN + ch * 32), r);
                    tc_wait_ld();
                    const int n0 = n_base + ch * 32;
                    if (addend != nullptr && m < M) {            // fp32 term added before the one rounding
                        const float *arow = addend + (size_t)m * ld_add + n0;
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (n0 + j < n_end) r[j] = __float_as_uint(__uint_as_float(r[j]) + arow[j]);
                    }
                    if (act != 0) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(apply_act(__uint_as_float(r[j]), act));
                    }
                    if (m < M && n0 < n_end) {
                        const int cols = min(32, n_end - n0);              // a tile's last chunk may be half full
                        if (vec_store && cols % 8 == 0) {
#pragma unroll
                            for (int v = 0; v < 4; ++v) {
                                if (8 * v < cols) {
                                    uint4 o;
                                    o.x = pack2_out<BF16>(__uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1]));
                                    o.y = pack2_out<BF16>(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3]));
                                    o.z = pack2_out<BF16>(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5]));
                                    o.w = pack2_out<BF16>(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7]));
                                    *reinterpret_cast<uint4 *>(yrow + n0 + 8 * v) = o;
                                }
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (j < cols) yrow[n0 + j] = (uint16_t)(pack2_out<BF16>(__uint_as_float(r[j]), 0.0f) & 0xFFFF);
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_tempty);
            tphase ^= 1;
        }
    } else {
        // ---------------- dequantise: W stage -> swizzled K-major B stage ----------------
        const int dw = warp - FIRST_DEQ_WARP;            // this warp's prepacked tile within the step
        const int g = lane & 7, c = lane >> 3;           // a quarter-warp covers 8 rows of one k-octet
        // Byte offsets, inside a B stage, of the four 16-byte chunks this lane writes.  Word j of
        // its slot is block kb = j/2 of row g + 8*(j%2): row (dw*16 + g + 8*(j%2)) of the operand,
        // chunk (j/2)*4 + c of that row's 128 bytes, XOR-swizzled with the row index modulo 8 (= g).
        uint32_t boff[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
            boff[j] = (uint32_t)((dw * 2 + (j & 1)) * 1024 + g * 128 + ((((j >> 1) * 4 + c) ^ g) << 4));
        const uint32_t qoff = (uint32_t)(dw * TILE_BYTES + slot_of(g, c) * 16);
        const uint32_t doff = (uint32_t)(dw * TILE_BYTES + TILE_QS_BYTES + g * 8);
        constexpr int TILES_PER_WARP = W_TILES / NUM_DEQ_WARPS;      // tile dw + i*NUM_DEQ_WARPS, i < TILES_PER_WARP
        RingPos w, b;
        for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
            const int valid = unit0(t / num_mt + 1) - unit0(t / num_mt);
            for (int ks = 0; ks < k_steps; ++ks) {
                if (!mbar_wait_warp(bar_full_w(w.s), w.phase, abort_flag, 6, lane)) goto done;
                if (!mbar_wait_warp(bar_empty_b(b.s), b.phase ^ 1, abort_flag, 8, lane)) goto done;
#pragma unroll
                for (int i = 0; i < TILES_PER_WARP; ++i) {
                    if (dw + i * NUM_DEQ_WARPS >= valid) break;
                    const uint32_t wst = base + SMEM_W + w.s * w_stage + i * NUM_DEQ_WARPS * TILE_BYTES;
                    const uint32_t bst = base + SMEM_B + b.s * B_BYTES + i * NUM_DEQ_WARPS * 2048;
                    uint4 qw;
                    uint2 dq;
                    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(qw.x), "=r"(qw.y), "=r"(qw.z), "=r"(qw.w) : "r"(wst + qoff));
                    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(dq.x), "=r"(dq.y) : "r"(wst + doff));
                    const uint32_t words[4] = {qw.x, qw.y, qw.z, qw.w};
                    const uint16_t dbits[4] = {(uint16_t)(dq.x & 0xFFFF), (uint16_t)(dq.x >> 16),
                                               (uint16_t)(dq.y & 0xFFFF), (uint16_t)(dq.y >> 16)};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        uint32_t h[4];
                        dequant_word<BF16>(words[j], h);
                        const uint32_t d2 = scale_pair<BF16>(dbits[j]);
                        uint4 o;
                        if constexpr (BF16) {
                            o.x = bmul2_bits(h[0], d2); o.y = bmul2_bits(h[1], d2);
                            o.z = bmul2_bits(h[2], d2); o.w = bmul2_bits(h[3], d2);
                        } else {
                            o.x = hmul2_bits(h[0], d2); o.y = hmul2_bits(h[1], d2);
                            o.z = hmul2_bits(h[2], d2); o.w = hmul2_bits(h[3], d2);
                        }
                        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(bst + boff[j]), "r"(o.x), "r"(o.y), "r"(o.z), "r"(o.w) : "memory");
                    }
                }
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(bar_full_b(b.s));
                    mbar_arrive(bar_empty_w(w.s));
                }
                w.advance(sw);
                b.advance(SB);
            }
        }
    }

done:
    tc_fence_before();
    __syncthreads();
    if (s_abort) {
        // give copies and MMAs still in flight time to land before shared memory and TMEM go away
        for (int i = 0; i < 64; ++i) __nanosleep(20000);
        __syncthreads();
    }
    if (warp == WARP_MMA) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// cuTensorMapEncodeTiled through the runtime, so the library has no link dependency on libcuda
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
        else
            (void)cudaGetLastError();
    });
    return fn;
}

template <bool BF16>
static int launch(const CUtensorMap &tmap, const void *prepacked, void *y, int M, int N, int K, int64_t ldy,
                  int vec_store, int sms, const float *addend, int64_t ld_add, int act, cudaStream_t st) {
    // Tiles per row block: the count that needs the least (waves x (widest tile + fixed cost)).  A 64-k
    // step costs its MMAs, proportional to the tile's width, plus about what 160 columns of MMAs cost
    // (measured: operand traffic from L2 and the hand-overs between the roles do not shrink with the
    // tile), so wide tiles win unless a narrower width fills the last wave.
    const int mt = (M + BM - 1) / BM;
    const int units = (int)tiles_n(N);
    int num_nt = (units + BN / TILE_N - 1) / (BN / TILE_N), bn_max = BN;
    long best = -1;
    for (int cand = num_nt; cand <= units; ++cand) {
        const int widest = ((units + cand - 1) / cand) * TILE_N;
        const long waves = ((long)mt * cand + sms - 1) / sms;
        const long cost = waves * (widest + 160);
        if (best < 0 || cost < best) { best = cost; num_nt = cand; bn_max = widest; }
        if (widest <= 2 * TILE_N) break;
    }
    {   // opt in to the large dynamic shared memory once per device and instantiation
        static bool attr_done[64] = {};
        static std::mutex attr_mu;
        int dev = 0;
        Q4B_CUDA_TRY(cudaGetDevice(&dev));
        std::lock_guard<std::mutex> attr_lock(attr_mu);
        if (dev < 0 || dev >= 64 || !attr_done[dev]) {
            Q4B_CUDA_TRY(cudaFuncSetAttribute(gemm_tcgen05_kernel<BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_DYN));
            if (dev >= 0 && dev < 64) attr_done[dev] = true;
        }
    }
    const int tiles = mt * num_nt;
    const int grid = tiles < sms ? tiles : sms;
    gemm_tcgen05_kernel<BF16><<<grid, THREADS, SMEM_DYN, st>>>(tmap, (const uint8_t *)prepacked, (uint16_t *)y, M, N, K,
                                                             ldy, vec_store, num_nt, bn_max, addend, ld_add, act);
    Q4B_LAUNCH_CHECK();
    return Q4B_OK;
}

}  // namespace gemm

int device_sm_count();
int gemv_wait_status(int *value);
int gemm_tmem_wait_status(int *value);
namespace chain { int wait_status(int *value); }
int selftest_wait_status(int *value);
int gemm_tmem_launch(const void *x, int bf16, int M, int64_t ldx, const void *prepacked, int64_t K, int64_t N,
                     const float *addend, int64_t ld_add, void *y, int64_t ldy, int flags, cudaStream_t st);
}  // namespace q4b

using namespace q4b;

extern "C" int q4b_gemm(const void *x, int x_dtype, int64_t M, int64_t ldx, const void *prepacked, int64_t K,
                        int64_t N, void *y, int64_t ldy, int flags, void *stream) {
    return q4b_gemm_addend(x, x_dtype, M, ldx, prepacked, K, N, nullptr, 0, y, ldy, flags, stream);
}

extern "C" int q4b_gemm_addend(const void *x, int x_dtype, int64_t M, int64_t ldx, const void *prepacked, int64_t K,
                               int64_t N, const float *addend, int64_t ld_add, void *y, int64_t ldy, int flags,
                               void *stream) {
    // ld_add == 0: the addend is one row of N values added to every row of the result (a bias)
    if (addend != nullptr && ld_add != 0 && ld_add < N) return Q4B_ERR_ARG;
    if (x == nullptr || prepacked == nullptr || y == nullptr) return Q4B_ERR_ARG;
    if (M < 1 || K <= 0 || N <= 0 || ldx < K || ldy < N) return Q4B_ERR_ARG;
    if (act_of_flags(flags) == 3) return Q4B_ERR_ARG;
    if (K % QK || M > (1 << 30) || N > (1 << 30) || K > (1 << 30)) return Q4B_ERR_SHAPE;
    if (x_dtype != Q4B_F16 && x_dtype != Q4B_BF16) return Q4B_ERR_DTYPE;
    if (!aligned(x, 16) || (ldx % 8) || !aligned(prepacked, 16) || !aligned(y, 2)) return Q4B_ERR_ALIGN;
    if (q4b_device_ok() != Q4B_OK) return Q4B_ERR_ARCH;
    // Up to 128 rows: the tensor-memory kernel (weights as the A operand), whose step cost does not
    // depend on M, unless the weight has more 128-column panels than two per SM (it is not
    // persistent: several waves of CTAs each pay its prologue and reduction).
    if (M <= 128 && ceil_div(tiles_n(N), 8) <= 2 * device_sm_count())
        return gemm_tmem_launch(x, x_dtype == Q4B_BF16, (int)M, ldx, prepacked, K, N, addend, ld_add, y, ldy, flags,
                                (cudaStream_t)stream);
    gemm::EncodeTiledFn enc = gemm::get_encode_fn();
    if (enc == nullptr) return Q4B_ERR_CUDA;

    CUtensorMap tmap;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
    const cuuint64_t strides[1] = {(cuuint64_t)ldx * 2};
    // 64 k x 256 rows per copy; a single half tile (M <= 128) is copied as 128 rows
    const cuuint32_t box[2] = {(cuuint32_t)gemm::BK, (cuuint32_t)(M <= gemm::HALF_M ? gemm::HALF_M : gemm::BM)};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(&tmap, x_dtype == Q4B_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                     const_cast<void *>(x), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return Q4B_ERR_ARG;
    const int vec_store = (aligned(y, 16) && ldy % 8 == 0) ? 1 : 0;
    const int sms = device_sm_count();
    cudaStream_t st = (cudaStream_t)stream;
    return x_dtype == Q4B_BF16
               ? gemm::launch<true>(tmap, prepacked, y, (int)M, (int)N, (int)K, ldy, vec_store, sms, addend, ld_add,
                                    act_of_flags(flags), st)
               : gemm::launch<false>(tmap, prepacked, y, (int)M, (int)N, (int)K, ldy, vec_store, sms, addend, ld_add,
                                     act_of_flags(flags), st);
}


extern "C" int q4b_wait_status(void *stream, int *detail) {
    Q4B_CUDA_TRY(cudaStreamSynchronize((cudaStream_t)stream));
    int h = 0, hv = 0;
    Q4B_CUDA_TRY(cudaMemcpyFromSymbol(&h, gemm::g_gemm_status, sizeof(int)));
    if (h != 0) {
        const int zero = 0;
        Q4B_CUDA_TRY(cudaMemcpyToSymbol(gemm::g_gemm_status, &zero, sizeof(int)));
    }
    if (int rc = gemv_wait_status(&hv)) return rc;
    if (h == 0) h = hv;
    if (int rc = gemm_tmem_wait_status(&hv)) return rc;
    if (h == 0) h = hv;
    if (int rc = chain::wait_status(&hv)) return rc;
    if (h == 0) h = hv;
    if (int rc = selftest_wait_status(&hv)) return rc;
    if (h == 0) h = hv;
    if (detail) *detail = h;
    return h != 0 ? Q4B_ERR_TIMEOUT : Q4B_OK;
}
