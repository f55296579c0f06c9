// Decode path for a single activation row on the 5th-generation tensor cores:
//   y[N] = x[K] . dequant(W),  tcgen05.mma with the weights as the A operand in tensor memory.
//
// Same role as q4b_gemv.cu (the reference has no GEMV specialisation at all: its one kernel,
// packages/metalcore/src/metalcore/native/quant_kernels.metal:1738-1886, runs M = 1 like M = 64).
//
// mma.sync spends a whole warp-wide instruction on 256 weights and runs on the legacy tensor path;
// at one row that path and the instruction issue slots, not HBM, set the pace.  Here a CTA owns a
// panel of 128 output columns (8 prepacked column tiles = the 128 lanes of tensor memory) and a
// range of k:
//   * one warp streams the panel's packed tiles into a shared-memory ring with bulk copies;
//   * eight warps turn nibbles into fp16/bf16 pairs and store them straight into tensor memory
//     (tcgen05.st), thread = output column, 32 consecutive k of one q4_0 block = 16 columns of
//     tensor memory; the nibbles go in biased, as (OFF + q), with no subtraction;
//   * one thread issues tcgen05.mma (M = 128, N = 16, K = 16) per half block.  The B operand is x
//     itself, read in place from shared memory: a no-swizzle K-major descriptor whose rows are
//     16 bytes apart makes accumulator column 0 the product with x[k0 .. k0+15]; the other 15
//     columns multiply later parts of x and are never read.  Each 32-k block has its own
//     accumulator, because its scale differs per output column;
//   * the warps that dequantised a block read its accumulator column back (tcgen05.ld), take off
//     sum((OFF + 8) * x) of the block (computed once per CTA), multiply by the block's scale and add
//     into one fp32 register per thread.
// CTAs that split k for the same panel form a thread-block cluster and are added up through
// distributed shared memory by the cluster's first CTA.  Every mbarrier wait is bounded; a wait
// that gives up records a code and all roles fall through to the common exit.
#include <cstdlib>

#include "q4b_sm100_ptx.cuh"

namespace q4b {
namespace gemvtc {

constexpr int PANEL_TILES = 8;                       // column tiles per CTA
constexpr int PANEL_N = PANEL_TILES * TILE_N;        // 128
constexpr int DEQ_WARPS = 8;                         // two groups of four; group i takes k-tiles i, i+2, ...
constexpr int WARP_MMA = 8, WARP_LOAD = 9;
constexpr int THREADS = 10 * 32;
constexpr int STAGE_STEPS = 2;                       // k-tiles per ring stage: one for each group
constexpr int TILE_RUN_BYTES = STAGE_STEPS * TILE_BYTES;             // 1152: one column tile's part of a stage
constexpr int STAGE_BYTES = PANEL_TILES * TILE_RUN_BYTES;            // 9216
constexpr int NSTAGE = 9;
constexpr int TM_STAGES = 4;                         // steps whose operands / accumulators tensor memory holds
constexpr int TMEM_COLS = 256;                       // D: 4 x (2 blocks x 16), A: 4 x (2 blocks x 16)
constexpr int D_COL0 = 0, A_COL0 = 128;
constexpr int X_MAX_ELEMS = 8192;                    // k range of one CTA
constexpr int X_PAD_BYTES = 512;                     // what the unused accumulator columns read past the end
constexpr int SMEM_RING = 0;
constexpr int SMEM_X = SMEM_RING + NSTAGE * STAGE_BYTES;
constexpr int SMEM_S = SMEM_X + X_MAX_ELEMS * 2 + X_PAD_BYTES;       // per-block sums, fp32
constexpr int SMEM_PART = SMEM_S + (X_MAX_ELEMS / QK) * 4;           // 2 x 128 partial outputs
constexpr int SMEM_BAR = SMEM_PART + 2 * PANEL_N * 4;
constexpr int NUM_BARS = 2 * NSTAGE + 2 * TM_STAGES + 1;
constexpr int SMEM_DYN = SMEM_BAR + NUM_BARS * 8 + 128;

__device__ int g_tc_status = 0;
#ifdef Q4B_TC_PROFILE
// development aid: cycle counters summed over CTAs (see the PROF_ADD sites)
__device__ unsigned long long g_tc_prof[16];
#define PROF_T0() const long long _pt = clock64()
#define PROF_ADD(slot) prof[slot] += clock64() - _pt
#else
#define PROF_T0()
#define PROF_ADD(slot)
#endif

using namespace ptx;

// bounded waits of this file record their code in g_tc_status
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int code) {
    return ptx::mbar_wait(bar, parity, abort_flag, &g_tc_status, code);
}
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int *abort_flag, int code) {
    return ptx::mbar_wait_warp(bar, parity, abort_flag, &g_tc_status, code);
}
__device__ __forceinline__ uint32_t tc_ld_32x32b_x1(uint32_t taddr) {
    uint32_t r;
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(r) : "r"(taddr) : "memory");
    return r;
}
__device__ __forceinline__ void deq_group_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

// K-major operand without swizzle: core matrices of 8 rows x 16 bytes.  Rows are 16 bytes apart
// and the next core matrix along k starts 16 bytes on, so row 0 is 32 contiguous bytes of x and
// row r the 32 bytes that start 16 r further on; the second group of 8 rows starts 128 bytes on.
__device__ __forceinline__ uint64_t make_x_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);     // start address, 16-byte units
    d |= (uint64_t)(16 >> 4) << 16;                  // leading byte offset: next core matrix along k
    d |= (uint64_t)(128 >> 4) << 32;                 // stride byte offset: next 8 rows
    d |= (uint64_t)1 << 46;                          // descriptor version for sm_100
    return d;                                        // layout type 0: no swizzle
}

template <bool BF16>
__global__ void __launch_bounds__(THREADS, 2)
gemv_tc_kernel(const uint16_t *__restrict__ x, const uint8_t *__restrict__ prepacked, int64_t K, int64_t N,
               uint16_t *__restrict__ y, const float *__restrict__ addend, int KS, int act) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;

    const uint32_t base = smem_u32(smem);
    const uint32_t bar0 = base + SMEM_BAR;
    auto bar_full_w = [&](int s) { return bar0 + 8u * s; };                           // packed tiles landed
    auto bar_empty_w = [&](int s) { return bar0 + 8u * (NSTAGE + s); };               // both groups have read them
    auto bar_a_full = [&](int s) { return bar0 + 8u * (2 * NSTAGE + s); };            // A operand in tensor memory
    auto bar_d_full = [&](int s) { return bar0 + 8u * (2 * NSTAGE + TM_STAGES + s); };  // its MMAs retired
    const uint32_t bar_x_full = bar0 + 8u * (2 * NSTAGE + 2 * TM_STAGES);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int *abort_flag = &s_abort;

    const int NT = (int)tiles_n(N);
    const int KU = (int)tiles_k(K);
    const int panel = (int)blockIdx.x / KS, ks = (int)blockIdx.x % KS;    // ks = rank in the cluster
    const int nt0 = panel * PANEL_TILES;
    const int valid = min(PANEL_TILES, NT - nt0);                          // column tiles that exist
    const int ku0 = (int)((int64_t)KU * ks / KS), ku1 = (int)((int64_t)KU * (ks + 1) / KS);
    const int nsteps = ku1 - ku0;                                          // k-tiles of this CTA
    const int nstages = (nsteps + STAGE_STEPS - 1) / STAGE_STEPS;
    const int xelems = (int)(min((int64_t)ku1 * TILE_K, K) - (int64_t)ku0 * TILE_K);

    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int s = 0; s < NSTAGE; ++s) { mbar_init(bar_full_w(s), 1); mbar_init(bar_empty_w(s), DEQ_WARPS); }
        for (int s = 0; s < TM_STAGES; ++s) { mbar_init(bar_a_full(s), DEQ_WARPS / 2); mbar_init(bar_d_full(s), 1); }
        mbar_init(bar_x_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == WARP_MMA) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // x slice and what lies past it start out as zeros (pad blocks and unused columns read them)
    for (int i = threadIdx.x * 16; i < X_MAX_ELEMS * 2 + X_PAD_BYTES; i += THREADS * 16)
        *reinterpret_cast<uint4 *>(smem + SMEM_X + i) = make_uint4(0u, 0u, 0u, 0u);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = s_tmem_base;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    float acc = 0.0f;                                  // dequantising threads: output column 32 (warp % 4) + lane

    if (warp == WARP_LOAD) {
        // ---------------- packed-weight and x producer ----------------
        // lane t copies column tile t's run of the stage (STAGE_STEPS consecutive k-tiles)
        const uint8_t *src = prepacked + tile_offset(nt0 + min(lane, valid - 1), ku0, KU);
        auto issue_stage = [&](int q) {
            const int slot = q % NSTAGE;
            const uint32_t bytes = (uint32_t)(min(STAGE_STEPS, nsteps - q * STAGE_STEPS) * TILE_BYTES);
            if (lane == 0) mbar_arrive_expect_tx(bar_full_w(slot), (uint32_t)valid * bytes);
            __syncwarp();
            if (lane < valid)
                bulk_load(base + SMEM_RING + slot * STAGE_BYTES + lane * TILE_RUN_BYTES, src + (size_t)q * TILE_RUN_BYTES, bytes,
                          bar_full_w(slot));
        };
        const int first = min(nstages, NSTAGE);
        for (int q = 0; q < first; ++q) issue_stage(q);
        // weights never depend on earlier kernels of the stream; x does
        asm volatile("griddepcontrol.wait;" ::: "memory");
        if (lane == 0) {
            mbar_arrive_expect_tx(bar_x_full, (uint32_t)xelems * 2);
            bulk_load(base + SMEM_X, x + (int64_t)ku0 * TILE_K, (uint32_t)xelems * 2, bar_x_full);
        }
        for (int q = first; q < nstages; ++q) {
            if (!mbar_wait_warp(bar_empty_w(q % NSTAGE), ((q / NSTAGE) & 1) ^ 1, abort_flag, 201)) goto done;
            issue_stage(q);
        }
    } else if (warp == WARP_MMA) {
        // ---------------- MMA issuer ----------------
        // The whole warp runs the loop, converged, and one elected lane issues: operands of
        // tcgen05.mma then sit in uniform registers instead of being moved there per instruction.
        asm volatile("griddepcontrol.wait;" ::: "memory");
        {
            const uint32_t idesc = make_idesc(BF16, PANEL_N, 16);
#ifdef Q4B_TC_PROFILE
            long long prof[4] = {0, 0, 0, 0};
            const long long prof_start = clock64();
#endif
            if (!mbar_wait_warp(bar_x_full, 0, abort_flag, 202)) goto done;
            for (int i = 0; i < nsteps; ++i) {
                const int st = i % TM_STAGES;
                { PROF_T0(); if (!mbar_wait_warp(bar_a_full(st), (i / TM_STAGES) & 1, abort_flag, 203)) goto done; PROF_ADD(0); }
                tc_fence_after();
                PROF_T0();
                if (elect_one()) {
#pragma unroll
                    for (int h = 0; h < 2; ++h) {           // the two blocks' accumulation chains side by side
#pragma unroll
                        for (int b = 0; b < TILE_KB; ++b) {
                            const uint64_t bdesc = make_x_desc(base + SMEM_X + (uint32_t)((i * TILE_K + b * QK + h * 16) * 2));
                            tc_mma_ts_f16(tmem_base + (uint32_t)(D_COL0 + st * 32 + b * 16),
                                          tmem_base + (uint32_t)(A_COL0 + st * 32 + b * 16 + h * 8), bdesc, idesc, (uint32_t)h);
                        }
                    }
                    tc_commit(bar_d_full(st));
                }
                __syncwarp();
                PROF_ADD(1);
            }
#ifdef Q4B_TC_PROFILE
            if (lane == 0) {
                atomicAdd(&g_tc_prof[0], (unsigned long long)prof[0]);
                atomicAdd(&g_tc_prof[1], (unsigned long long)(clock64() - prof_start));
                atomicAdd(&g_tc_prof[3], (unsigned long long)prof[1]);
                atomicAdd(&g_tc_prof[2], (unsigned long long)nsteps);
            }
#endif
        }
    } else {
        // ---------------- dequantise into tensor memory, then scale what comes back ----------------
        const int grp = warp >> 2, wq = warp & 3;                 // wq = tensor-memory lane quadrant
        const int tile = 2 * wq + (lane >> 4);                    // column tile of the panel
        const int r = lane & 15, g = r & 7, hi = r >> 3;          // row of the tile: g + 8 hi
        const uint32_t lane_taddr = tmem_base + ((uint32_t)(wq * 32) << 16);
        // word (kb, octet c) of this row: slot_of(g, c) * 16 + (kb * 2 + hi) * 4 inside the tile
        uint32_t woff[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) woff[c] = (uint32_t)(tile * TILE_RUN_BYTES + slot_of(g, c) * 16 + hi * 4);
        const uint32_t doff = (uint32_t)(tile * TILE_RUN_BYTES + TILE_QS_BYTES + g * 8 + hi * 2);

        asm volatile("griddepcontrol.wait;" ::: "memory");
        // sum((OFF + 8) * x) of every block of this CTA's k range, once
        if (!mbar_wait_warp(bar_x_full, 0, abort_flag, 204)) goto done;
        {
            constexpr float CL = BF16 ? 136.0f : 1032.0f;      // k offsets 0,1,4,5 of an octet
            constexpr float CH = BF16 ? 136.0f : 72.0f;        // k offsets 2,3,6,7
            float *S = reinterpret_cast<float *>(smem + SMEM_S);
            for (int b = threadIdx.x; b < nsteps * TILE_KB; b += DEQ_WARPS * 32) {
                float s = 0.0f;
#pragma unroll
                for (int o = 0; o < 4; ++o) {
                    const uint4 xo = *reinterpret_cast<const uint4 *>(smem + SMEM_X + b * QK * 2 + o * 16);
                    float2 p0, p1, p2, p3;
                    if constexpr (BF16) {
                        p0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&xo.x));
                        p1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&xo.y));
                        p2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&xo.z));
                        p3 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&xo.w));
                    } else {
                        p0 = __half22float2(*reinterpret_cast<const __half2 *>(&xo.x));
                        p1 = __half22float2(*reinterpret_cast<const __half2 *>(&xo.y));
                        p2 = __half22float2(*reinterpret_cast<const __half2 *>(&xo.z));
                        p3 = __half22float2(*reinterpret_cast<const __half2 *>(&xo.w));
                    }
                    s += CL * ((p0.x + p0.y) + (p2.x + p2.y)) + CH * ((p1.x + p1.y) + (p3.x + p3.y));
                }
                S[b] = s;
            }
        }
        deq_group_sync();

        const float *S = reinterpret_cast<const float *>(smem + SMEM_S);
        float dprev0 = 0.0f, dprev1 = 0.0f;
        int iprev = -1;
#ifdef Q4B_TC_PROFILE
        long long prof[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        const long long prof_start = clock64();
#endif
        // scale and add the accumulator columns of step i (this thread's own row)
        auto epilogue = [&](int i, float d0, float d1) -> bool {
            const int st = i % TM_STAGES;
            { PROF_T0(); if (!mbar_wait_warp(bar_d_full(st), (i / TM_STAGES) & 1, abort_flag, 205)) return false; PROF_ADD(3); }
            tc_fence_after();
            PROF_T0();
            const uint32_t v0 = tc_ld_32x32b_x1(lane_taddr + (uint32_t)(D_COL0 + st * 32));
            const uint32_t v1 = tc_ld_32x32b_x1(lane_taddr + (uint32_t)(D_COL0 + st * 32 + 16));
            tc_wait_ld();
            PROF_ADD(4);
            const float2 s2 = *reinterpret_cast<const float2 *>(&S[i * TILE_KB]);
            acc = fmaf(d0, __uint_as_float(v0) - s2.x, acc);
            acc = fmaf(d1, __uint_as_float(v1) - s2.y, acc);
            return true;
        };
        for (int i = grp; i < nsteps; i += 2) {
            const int q = i / STAGE_STEPS, slot = q % NSTAGE;
            { PROF_T0(); if (!mbar_wait_warp(bar_full_w(slot), (q / NSTAGE) & 1, abort_flag, 206)) goto done; PROF_ADD(0); }
#ifdef Q4B_TC_PROFILE
            const long long _deq0 = clock64();
#endif
            const uint32_t wst = base + SMEM_RING + slot * STAGE_BYTES + (i % STAGE_STEPS) * TILE_BYTES;
            uint32_t w[2][4];
#pragma unroll
            for (int kb = 0; kb < 2; ++kb)
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w[kb][c]) : "r"(wst + woff[c] + kb * 8));
            uint32_t dbits0, dbits1;
            asm volatile("ld.shared.u16 %0, [%1];" : "=r"(dbits0) : "r"(wst + doff));
            asm volatile("ld.shared.u16 %0, [%1];" : "=r"(dbits1) : "r"(wst + doff + 4));
            const int st = i % TM_STAGES;
#pragma unroll
            for (int kb = 0; kb < 2; ++kb) {
                uint32_t regs[16];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t h[4];
                    dequant_word_biased<BF16>(w[kb][c], h);
                    regs[4 * c + 0] = h[0]; regs[4 * c + 1] = h[1]; regs[4 * c + 2] = h[2]; regs[4 * c + 3] = h[3];
                }
                tc_st_32x32b_x16(lane_taddr + (uint32_t)(A_COL0 + st * 32 + kb * 16), regs);
            }
#ifdef Q4B_TC_PROFILE
            prof[1] += clock64() - _deq0;
#endif
            { PROF_T0(); tc_wait_st(); PROF_ADD(2); }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(bar_a_full(st));
                mbar_arrive(bar_empty_w(slot));
            }
            // the step this group dequantised before: its MMAs have had a whole step to finish
            if (iprev >= 0 && !epilogue(iprev, dprev0, dprev1)) goto done;
            iprev = i;
            dprev0 = __half2float(__ushort_as_half((uint16_t)dbits0));
            dprev1 = __half2float(__ushort_as_half((uint16_t)dbits1));
        }
        if (iprev >= 0 && !epilogue(iprev, dprev0, dprev1)) goto done;
        reinterpret_cast<float *>(smem + SMEM_PART)[grp * PANEL_N + wq * 32 + lane] = acc;
#ifdef Q4B_TC_PROFILE
        if (warp == 0 && lane == 0) {
            for (int j = 0; j < 5; ++j) atomicAdd(&g_tc_prof[4 + j], (unsigned long long)prof[j]);
            atomicAdd(&g_tc_prof[9], (unsigned long long)(clock64() - prof_start));
            atomicAdd(&g_tc_prof[10], 1ull);
        }
#endif
    }

done:
    tc_fence_before();
    __syncthreads();
    if (KS > 1) cluster_sync_all();                    // every CTA's partial sums are in its shared memory
    if (threadIdx.x < PANEL_N && ks == 0) {
        const uint32_t p0 = base + SMEM_PART + threadIdx.x * 4, p1 = p0 + PANEL_N * 4;
        const float *part = reinterpret_cast<const float *>(smem + SMEM_PART);
        float sum = part[threadIdx.x] + part[PANEL_N + threadIdx.x];
        for (int rk = 1; rk < KS; ++rk) sum += ld_cluster_f32(p0, (uint32_t)rk) + ld_cluster_f32(p1, (uint32_t)rk);
        const int n = nt0 * TILE_N + (int)threadIdx.x;
        if (n < N && !s_abort) {
            if (addend != nullptr) sum += addend[n];           // fp32 term added before the one rounding
            sum = apply_act(sum, act);
            if constexpr (BF16) y[n] = __bfloat16_as_ushort(__float2bfloat16_rn(sum));
            else y[n] = __half_as_ushort(__float2half_rn(sum));
        }
    }
    if (KS > 1) cluster_sync_all();                    // nobody leaves while its sums may still be read
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

template <bool BF16>
static int launch(const void *x, const void *prepacked, int64_t K, int64_t N, void *y, const float *addend, int ks,
                  int flags, cudaStream_t st) {
    Q4B_CUDA_TRY(cudaFuncSetAttribute(gemv_tc_kernel<BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_DYN));
    const int64_t panels = ceil_div(tiles_n(N), PANEL_TILES);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(panels * ks));
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = (size_t)SMEM_DYN;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (flags & Q4B_FLAG_PDL) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    if (ks > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = (unsigned)ks;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = (unsigned)na;
    Q4B_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemv_tc_kernel<BF16>, (const uint16_t *)x, (const uint8_t *)prepacked, K, N,
                                    (uint16_t *)y, addend, ks, act_of_flags(flags)));
    return Q4B_OK;
}

}  // namespace gemvtc

// k-split of the tensor-core decode kernel for this shape: as many CTAs as two per SM allow, each
// with at most X_MAX_ELEMS of k.  0 when the shape does not fit the kernel.
int gemv_tc_ksplit(int64_t K, int64_t N, int sms) {
    const int64_t panels = ceil_div(tiles_n(N), gemvtc::PANEL_TILES), KU = tiles_k(K);
    int64_t ks = (2LL * sms) / panels;
    if (ks > 8) ks = 8;
    if (ks < 1) ks = 1;
    if (ks > KU) ks = KU;
    while (ks < 8 && ceil_div(KU, ks) * TILE_K > gemvtc::X_MAX_ELEMS) ++ks;
    if (ceil_div(KU, ks) * TILE_K > gemvtc::X_MAX_ELEMS) return 0;
    return (int)ks;
}

int gemv_tc_launch(const void *x, int bf16, const void *prepacked, int64_t K, int64_t N, void *y, const float *addend, int ks,
                   int flags, cudaStream_t st) {
    return bf16 ? gemvtc::launch<true>(x, prepacked, K, N, y, addend, ks, flags, st)
                : gemvtc::launch<false>(x, prepacked, K, N, y, addend, ks, flags, st);
}

#ifdef Q4B_TC_PROFILE
extern "C" __attribute__((visibility("default"))) int q4b_debug_tc_profile(unsigned long long *out, int reset) {
    if (cudaMemcpyFromSymbol(out, gemvtc::g_tc_prof, sizeof(unsigned long long) * 16) != cudaSuccess) return 6;
    if (reset) {
        unsigned long long z[16] = {};
        cudaMemcpyToSymbol(gemvtc::g_tc_prof, z, sizeof(z));
    }
    return 0;
}
#endif

// read and clear this file's wait status (host side; the caller has synchronised the stream)
int gemv_tc_wait_status(int *value) {
    int h = 0;
    Q4B_CUDA_TRY(cudaMemcpyFromSymbol(&h, gemvtc::g_tc_status, sizeof(int)));
    if (h != 0) {
        const int zero = 0;
        Q4B_CUDA_TRY(cudaMemcpyToSymbol(gemvtc::g_tc_status, &zero, sizeof(int)));
    }
    *value = h;
    return Q4B_OK;
}

}  // namespace q4b
