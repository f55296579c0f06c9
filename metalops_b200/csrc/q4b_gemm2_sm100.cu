// Prefill path for many rows: Y[M, N] = X[M, K] . dequant(W) with CTA-pair tensor-core instructions.
//
// Same contraction as q4b_gemm_sm100.cu (the reference's kernel is
// packages/metalcore/src/metalcore/native/quant_kernels.metal:1738-1886), for M above 256.
//
// Two CTAs on neighbouring SMs form a cluster and work on one 256 (M) x bn (N) tile per step of
// 64 k with tcgen05.mma.cta_group::2: each CTA loads its own 128 rows of X and dequantises its own
// HALF of the tile's columns, and the instruction, issued by the pair's first CTA, reads both
// halves.  Per SM that halves the B-operand bytes dequantised, written and read per flop compared
// with the one-CTA kernel, which is what bounds that kernel.  Accumulators (128 lanes x bn columns
// per CTA) are double-buffered in tensor memory, so a tile's epilogue runs under the next tile's
// main loop.
//
// Roles in each CTA (19 warps):
//   warp 0      TMA loads of this CTA's 128 x 64 X tile (128-byte swizzle), completion counted on
//               the FIRST CTA's barrier (cp.async.bulk.tensor with cta_group::2, no multicast)
//   warp 6      bulk copies of this CTA's packed weight tiles of the step, one per lane
//   warps 7-14  dequantise a W stage into the K-major swizzled B half; arrive on the first CTA's
//               "B full" barrier (remotely from the second CTA)
//   warp 1      first CTA only: one elected lane issues the MMAs; tcgen05.commit with cluster
//               multicast releases the A and B stages of both CTAs and hands over accumulators
//   warps 2-5, 15-18  epilogue of this CTA's 128 rows
// Every mbarrier wait is bounded; a wait that gives up records a code, raises the CTA's abort flag
// and every role leaves through the common exit, which both CTAs pass before either frees TMEM.
#include <cuda.h>

#include <cstdlib>
#include <mutex>

#include "q4b_common.cuh"

namespace q4b {
namespace gemm2 {

constexpr int PAIR_M = 256, CTA_M = 128, BN = 256, BK = 64;
constexpr int SA = 4, SB = 6;                         // ring depths of the X and B operand stages
constexpr int SW_MAX = 8;                             // packed-weight ring: depth chosen per launch
constexpr int A_BYTES = CTA_M * BK * 2;               // 16384: this CTA's rows of the X tile
constexpr int B_BYTES = (BN / 2) * BK * 2;            // 16384: this CTA's half of the B operand
constexpr int NUM_DEQ_WARPS = 8;                      // warps that share one step: a prepacked tile each
constexpr int DEQ_GROUPS = 2;                         // groups of them; group i takes steps i, i + 2, ...
constexpr int WARP_A = 0, WARP_MMA = 1, WARP_W = 6, FIRST_DEQ_WARP = 7;   // warps 2..5: epilogue
constexpr int FIRST_EPI2_WARP = FIRST_DEQ_WARP + DEQ_GROUPS * NUM_DEQ_WARPS;
constexpr int NUM_EPI_WARPS = 8;
constexpr int THREADS = (FIRST_EPI2_WARP + 4) * 32;   // 864
constexpr int SMEM_A = 0;
constexpr int SMEM_B = SMEM_A + SA * A_BYTES;
constexpr int SMEM_BAR = SMEM_B + SB * B_BYTES;
constexpr int NUM_BARS = 2 * (SA + SW_MAX + SB) + 4;
constexpr int SMEM_W = SMEM_BAR + ((NUM_BARS * 8 + 127) / 128) * 128;
constexpr int SMEM_DYN = 227 * 1024 - 256;
constexpr int SMEM_W_BYTES = SMEM_DYN - 1024 - SMEM_W;
constexpr long long WAIT_LIMIT_CYCLES = 1LL << 28;    // ~0.15 s; far above any legitimate wait

__host__ __device__ inline int w_ring_depth(int half_tiles) {
    const int d = SMEM_W_BYTES / (half_tiles * TILE_BYTES);
    return d < SW_MAX ? d : SW_MAX;
}

__device__ int g_gemm2_status = 0;

// ---- thin PTX wrappers ---------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("{ .reg .b64 t; mbarrier.arrive.shared::cta.b64 t, [%0]; }" ::"r"(bar) : "memory");
}
// arrive on a barrier anywhere in the cluster (address from map_to_rank)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
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
                atomicCAS(&g_gemm2_status, 0, code);
                return false;
            }
        }
    }
}
template <int SLEEP_NS = 0>
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int *abort_flag, int code) {
    return __all_sync(0xffffffffu, mbar_wait<SLEEP_NS>(bar, parity, abort_flag, code));
}
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{ .reg .pred p; elect.sync _|p, 0xffffffff; selp.u32 %0, 1, 0, p; }" : "=r"(pred));
    return pred != 0;
}
// tile load into this CTA's shared memory; the byte count completes on `cluster_bar`, which may
// belong to the other CTA of the pair
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t cluster_bar) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(cluster_bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// arrives on the barrier at this offset in BOTH CTAs once all MMAs issued so far have retired
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void tc_mma_pair_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p; }"
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

// K-major operand tile stored as rows of 128 bytes with the 128-byte swizzle: 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t make_kmajor_sw128_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);     // start address, 16-byte units
    d |= (uint64_t)1 << 16;                          // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;                // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                          // descriptor version for sm_100
    d |= (uint64_t)2 << 61;                          // SWIZZLE_128B
    return d;
}
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
template <bool BF16> __device__ __forceinline__ uint32_t scale_pair(uint16_t dbits) {
    if constexpr (BF16) {
        __nv_bfloat16 b = __float2bfloat16_rn(__half2float(__ushort_as_half(dbits)));
        uint32_t u = __bfloat16_as_ushort(b);
        return u | (u << 16);
    } else {
        return (uint32_t)dbits | ((uint32_t)dbits << 16);
    }
}
struct RingPos {
    int s = 0;
    uint32_t phase = 0;
    __device__ __forceinline__ void advance(int depth) {
        if (++s == depth) { s = 0; phase ^= 1; }
    }
};

constexpr int NACC = 2;                              // accumulator buffers in tensor memory

template <bool BF16>
__global__ void __launch_bounds__(THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_x, const uint8_t *__restrict__ prepacked,
                 uint16_t *__restrict__ y, int M, int N, int K, int64_t ldy, int vec_store, int bn,
                 const float *__restrict__ addend, int64_t ld_add, int act) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;

    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;      // the same offset in both CTAs of the pair
    const uint32_t bar0 = base + SMEM_BAR;
    auto bar_full_a = [&](int s) { return bar0 + 8u * s; };                                  // first CTA: both X tiles landed
    auto bar_empty_a = [&](int s) { return bar0 + 8u * (SA + s); };                          // their MMAs retired
    auto bar_full_w = [&](int s) { return bar0 + 8u * (2 * SA + s); };                       // packed weights landed
    auto bar_empty_w = [&](int s) { return bar0 + 8u * (2 * SA + SW_MAX + s); };             // dequantisers done reading
    auto bar_full_b = [&](int s) { return bar0 + 8u * (2 * SA + 2 * SW_MAX + s); };          // first CTA: both B halves written
    auto bar_empty_b = [&](int s) { return bar0 + 8u * (2 * SA + 2 * SW_MAX + SB + s); };    // their MMAs retired
    auto bar_tfull = [&](int i) { return bar0 + 8u * (2 * (SA + SW_MAX + SB) + i); };        // accumulators complete
    auto bar_tempty = [&](int i) { return bar0 + 8u * (2 * (SA + SW_MAX + SB) + 2 + i); };   // first CTA: both drained

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();              // 0: issues the MMAs
    volatile int *abort_flag = &s_abort;

    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int s = 0; s < SA; ++s) { mbar_init(bar_full_a(s), 1); mbar_init(bar_empty_a(s), 1); }
        for (int s = 0; s < SW_MAX; ++s) { mbar_init(bar_full_w(s), 1); mbar_init(bar_empty_w(s), NUM_DEQ_WARPS); }
        // "B full": this CTA's eight dequantising warps, plus, in the first CTA, one arrival relayed from the second
        for (int s = 0; s < SB; ++s) { mbar_init(bar_full_b(s), NUM_DEQ_WARPS + (rank == 0 ? 1 : 0)); mbar_init(bar_empty_b(s), 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(bar_tfull(i), 1); mbar_init(bar_tempty(i), 2 * NUM_EPI_WARPS); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == WARP_MMA) {
        // one warp of each CTA of the pair takes part in the allocation
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)), "r"(NACC * BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    cluster_sync_all();                                // both CTAs' barriers exist before anything signals them
    tc_fence_after();
    const uint32_t tmem_base = s_tmem_base;

    const int NT = (int)tiles_n(N);
    const int w_tiles = bn / TILE_N, half_tiles = w_tiles / 2;     // column tiles of the pair / of this CTA
    const int sw = w_ring_depth(half_tiles);
    const int w_stage = half_tiles * TILE_BYTES;
    const int num_mt = (M + PAIR_M - 1) / PAIR_M, num_nt = (N + bn - 1) / bn;
    const int num_tiles = num_mt * num_nt;
    const int k_steps = (K + BK - 1) / BK;
    const int pair = (int)blockIdx.x >> 1, num_pairs = (int)gridDim.x >> 1;

    if (warp == WARP_A) {
        // ---------------- X producer ----------------
        if (lane == 0) {
            RingPos a;
            for (int t = pair; t < num_tiles; t += num_pairs) {
                const int mt = t % num_mt;
                for (int ks = 0; ks < k_steps; ++ks) {
                    if (!mbar_wait(bar_empty_a(a.s), a.phase ^ 1, abort_flag, 301)) goto done;
                    if (rank == 0) mbar_arrive_expect_tx(bar_full_a(a.s), 2u * A_BYTES);     // both CTAs' bytes
                    tma_load_2d_pair(base + SMEM_A + a.s * A_BYTES, &tmap_x, ks * BK, mt * PAIR_M + (int)rank * CTA_M,
                                     map_to_rank(bar_full_a(a.s), 0));
                    a.advance(SA);
                }
            }
        }
    } else if (warp == WARP_W) {
        // ---------------- packed-weight producer: lane i copies this CTA's column tile i of the step ----------------
        RingPos w;
        for (int t = pair; t < num_tiles; t += num_pairs) {
            const int nt0 = (t / num_mt) * w_tiles + (int)rank * half_tiles;
            const int valid = max(0, min(half_tiles, NT - nt0));
            const uint8_t *src = prepacked + tile_offset(min(nt0 + min(lane, max(valid - 1, 0)), NT - 1), 0, k_steps);
            for (int ks = 0; ks < k_steps; ++ks) {
                if (!mbar_wait_warp(bar_empty_w(w.s), w.phase ^ 1, abort_flag, 307)) goto done;
                if (lane == 0) {
                    if (valid > 0) mbar_arrive_expect_tx(bar_full_w(w.s), (uint32_t)(valid * TILE_BYTES));
                    else mbar_arrive(bar_full_w(w.s));
                }
                __syncwarp();
                if (lane < valid)
                    bulk_load(base + SMEM_W + w.s * w_stage + lane * TILE_BYTES, src + (size_t)ks * TILE_BYTES, TILE_BYTES,
                              bar_full_w(w.s));
                w.advance(sw);
            }
        }
    } else if (warp == WARP_MMA) {
        // ---------------- MMA issuer (first CTA of the pair) ----------------
        if (rank == 0) {
            const uint32_t idesc = make_idesc(BF16, PAIR_M, bn);
            RingPos a, b;
            int it = 0;
            for (int t = pair; t < num_tiles; t += num_pairs, ++it) {
                const int ab = it % NACC;
                if (!mbar_wait_warp(bar_tempty(ab), (((uint32_t)(it / NACC)) & 1u) ^ 1u, abort_flag, 302)) goto done;
                tc_fence_after();
                for (int ks = 0; ks < k_steps; ++ks) {
                    if (!mbar_wait_warp(bar_full_a(a.s), a.phase, abort_flag, 303)) goto done;
                    if (!mbar_wait_warp(bar_full_b(b.s), b.phase, abort_flag, 304)) goto done;
                    tc_fence_after();
                    if (elect_one()) {
                        const uint64_t adesc = make_kmajor_sw128_desc(base + SMEM_A + a.s * A_BYTES);
                        const uint64_t bdesc = make_kmajor_sw128_desc(base + SMEM_B + b.s * B_BYTES);
#pragma unroll
                        for (int k = 0; k < BK / 16; ++k)                 // +32 bytes per k16 inside the swizzle atom
                            tc_mma_pair_f16(tmem_base + (uint32_t)(ab * BN), adesc + 2 * k, bdesc + 2 * k, idesc, (ks | k) != 0);
                        tc_commit_pair(bar_empty_a(a.s));
                        tc_commit_pair(bar_empty_b(b.s));
                        if (ks == k_steps - 1) tc_commit_pair(bar_tfull(ab));
                    }
                    __syncwarp();
                    a.advance(SA);
                    b.advance(SB);
                }
            }
        } else if (lane == 0) {
            // Second CTA: relay.  Its dequantising warps arrive on their own CTA's "B full" barrier, which
            // is cheap; this otherwise idle thread passes each completed phase on to the first CTA, so the
            // latency of the remote arrival is off their path.
            RingPos b;
            for (int t = pair; t < num_tiles; t += num_pairs) {
                for (int ks = 0; ks < k_steps; ++ks) {
                    if (!mbar_wait(bar_full_b(b.s), b.phase, abort_flag, 309)) goto done;
                    mbar_arrive_cluster(map_to_rank(bar_full_b(b.s), 0));
                    b.advance(SB);
                }
            }
        }
    } else if (warp < WARP_W || warp >= FIRST_EPI2_WARP) {
        // ---------------- epilogue: two warps per TMEM lane quadrant, alternate 32-column chunks ----
        const int quad = warp & 3;                      // TMEM lane quadrant this warp may read
        const int grp = warp >= FIRST_EPI2_WARP ? 1 : 0;
        int it = 0;
        for (int t = pair; t < num_tiles; t += num_pairs, ++it) {
            const int mt = t % num_mt, nt = t / num_mt;
            const int ab = it % NACC;
            if (!mbar_wait_warp<256>(bar_tfull(ab), ((uint32_t)(it / NACC)) & 1u, abort_flag, 305)) goto done;
            tc_fence_after();
            const int n_base = nt * bn;
            const int m = mt * PAIR_M + (int)rank * CTA_M + quad * 32 + lane;
            uint16_t *yrow = y + (size_t)m * ldy;
#pragma unroll 1
            for (int ch = grp; ch < bn / 32; ch += 2) {
                uint32_t r[32];
                tc_ld_32x32b_x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(ab * BN + ch * 32), r);
                tc_wait_ld();
                const int n0 = n_base + ch * 32;
                if (addend != nullptr && m < M) {            // fp32 term added before the one rounding
                    const float *arow = addend + (size_t)m * ld_add + n0;
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (n0 + j < N) r[j] = __float_as_uint(__uint_as_float(r[j]) + arow[j]);
                }
                if (act != 0) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(apply_act(__uint_as_float(r[j]), act));
                }
                if (m < M && n0 < N) {
                    if (vec_store && n0 + 32 <= N) {
#pragma unroll
                        for (int v = 0; v < 4; ++v) {
                            uint4 o;
                            o.x = pack2_out<BF16>(__uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1]));
                            o.y = pack2_out<BF16>(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3]));
                            o.z = pack2_out<BF16>(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5]));
                            o.w = pack2_out<BF16>(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7]));
                            *reinterpret_cast<uint4 *>(yrow + n0 + 8 * v) = o;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (n0 + j < N) yrow[n0 + j] = (uint16_t)(pack2_out<BF16>(__uint_as_float(r[j]), 0.0f) & 0xFFFF);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_rank(bar_tempty(ab), 0));
        }
    } else {
        // ---------------- dequantise: W stage -> this CTA's half of the swizzled K-major B stage ----------------
        const int dgrp = (warp - FIRST_DEQ_WARP) / NUM_DEQ_WARPS;    // which steps this warp works on
        const int dw = (warp - FIRST_DEQ_WARP) % NUM_DEQ_WARPS;      // its prepacked tile within a step
        const int g = lane & 7, c = lane >> 3;           // a quarter-warp covers 8 rows of one k-octet
        uint32_t boff[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
            boff[j] = (uint32_t)((dw * 2 + (j & 1)) * 1024 + g * 128 + ((((j >> 1) * 4 + c) ^ g) << 4));
        const uint32_t qoff = (uint32_t)(dw * TILE_BYTES + slot_of(g, c) * 16);
        const uint32_t doff = (uint32_t)(dw * TILE_BYTES + TILE_QS_BYTES + g * 8);
        uint32_t step = 0;                               // running index over all (tile, k step) pairs of this CTA
        for (int t = pair; t < num_tiles; t += num_pairs) {
            const int nt0 = (t / num_mt) * w_tiles + (int)rank * half_tiles;
            const int valid = max(0, min(half_tiles, NT - nt0));
            for (int ks = 0; ks < k_steps; ++ks, ++step) {
                if ((int)(step % DEQ_GROUPS) != dgrp) continue;
                const int ws = (int)(step % (uint32_t)sw), bs = (int)(step % SB);
                const uint32_t wphase = (step / (uint32_t)sw) & 1u, bphase = (step / SB) & 1u;
                if (!mbar_wait_warp(bar_full_w(ws), wphase, abort_flag, 306)) goto done;
                if (!mbar_wait_warp(bar_empty_b(bs), bphase ^ 1, abort_flag, 308)) goto done;
                if (dw < valid) {
                    const uint32_t wst = base + SMEM_W + ws * w_stage;
                    const uint32_t bst = base + SMEM_B + bs * B_BYTES;
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
                    mbar_arrive(bar_full_b(bs));         // own CTA's barrier; the second CTA's is relayed by its warp 1
                    mbar_arrive(bar_empty_w(ws));
                }
            }
        }
    }

done:
    tc_fence_before();
    __syncthreads();
    if (s_abort) {
        // give copies and MMAs still in flight time to land before shared memory and TMEM go away
        for (int i = 0; i < 64; ++i) __nanosleep(20000);
    }
    cluster_sync_all();                                // neither CTA frees anything the other may still signal or read
    if (warp == WARP_MMA) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(NACC * BN) : "memory");
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
    // Columns per pair tile: least (waves of CTA pairs x tile width), slightly biased to wide tiles
    const int mt = (M + PAIR_M - 1) / PAIR_M;
    const int pairs_max = sms / 2;
    int bn = BN;
    long best = -1;
    for (int cand = BN; cand >= 64; cand -= 32) {
        const long t = (long)mt * ((N + cand - 1) / cand);
        const long cost = ((t + pairs_max - 1) / pairs_max) * (cand + 24);
        if (best < 0 || cost < best) { best = cost; bn = cand; }
    }
    if (const char *e = getenv("Q4B_GEMM_BN")) { const int v = atoi(e); if (v >= 64 && v <= BN && v % 32 == 0) bn = v; }
    Q4B_CUDA_TRY(cudaFuncSetAttribute(gemm_pair_kernel<BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_DYN));
    const long tiles = (long)mt * ((N + bn - 1) / bn);
    const int pairs = (int)(tiles < pairs_max ? tiles : pairs_max);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(2 * pairs));
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = (size_t)SMEM_DYN;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    Q4B_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemm_pair_kernel<BF16>, tmap, (const uint8_t *)prepacked, (uint16_t *)y, M, N, K, ldy,
                                    vec_store, bn, addend, ld_add, act));
    return Q4B_OK;
}

}  // namespace gemm2

int device_sm_count();

// Arguments as checked by q4b_gemm_addend.
int gemm2_launch(const void *x, int bf16, int M, int64_t ldx, const void *prepacked, int K, int N, const float *addend,
                 int64_t ld_add, void *y, int64_t ldy, int act, cudaStream_t st) {
    gemm2::EncodeTiledFn enc = gemm2::get_encode_fn();
    if (enc == nullptr) return Q4B_ERR_CUDA;
    CUtensorMap tmap;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
    const cuuint64_t strides[1] = {(cuuint64_t)ldx * 2};
    const cuuint32_t box[2] = {(cuuint32_t)gemm2::BK, (cuuint32_t)gemm2::CTA_M};   // 64 k x 128 rows per copy
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(&tmap, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(x),
                     dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return Q4B_ERR_ARG;
    const int vec_store = (aligned(y, 16) && ldy % 8 == 0) ? 1 : 0;
    const int sms = device_sm_count();
    return bf16 ? gemm2::launch<true>(tmap, prepacked, y, M, N, K, ldy, vec_store, sms, addend, ld_add, act, st)
                : gemm2::launch<false>(tmap, prepacked, y, M, N, K, ldy, vec_store, sms, addend, ld_add, act, st);
}

int gemm2_wait_status(int *value) {
    int h = 0;
    Q4B_CUDA_TRY(cudaMemcpyFromSymbol(&h, gemm2::g_gemm2_status, sizeof(int)));
    if (h != 0) {
        const int zero = 0;
        Q4B_CUDA_TRY(cudaMemcpyToSymbol(gemm2::g_gemm2_status, &zero, sizeof(int)));
    }
    *value = h;
    return Q4B_OK;
}

}  // namespace q4b

