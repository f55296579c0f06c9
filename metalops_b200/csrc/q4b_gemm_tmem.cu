// Small-batch path: Y[M, N] = X[M, K] . dequant(W) for M <= 128 with the WEIGHTS as the tensor
// cores' A operand in tensor memory ("swap A and B").
//
// Same contraction as q4b_gemm_wt.cu (reference kernel:
// packages/metalcore/src/metalcore/native/quant_kernels.metal:1738-1886).  With few rows the
// prefill kernel's 128-row X tile is mostly padding and every 64-k step pays a fixed ~850 cycles;
// here the 128 lanes of tensor memory are 128 OUTPUT COLUMNS instead, so the work per step does not
// depend on M at all:
//   * a CTA owns a panel of 128 output columns (8 prepacked column tiles) and a range of k; CTAs
//     that split k for one panel form a thread-block cluster;
//   * one warp streams the panel's packed tiles into a shared-memory ring with bulk copies, another
//     loads the matching [rows x 64 k] slices of X with TMA (128-byte swizzle, rows beyond M are
//     zero fill);
//   * eight warps (two groups on alternate k-tiles) dequantise straight into tensor memory (tcgen05.st): thread = output column, one
//     q4_0 block = 16 columns of tensor memory, values (q-8)*d rounded once to fp16/bf16, as the
//     prefill kernel and the reference's Metal kernel round them;
//   * one more warp: one elected lane issues tcgen05.mma M128 x N=rows(16..128) x K16, A from tensor
//     memory, B = the X slice in shared memory, all k steps into ONE accumulator D[column][row];
//   * at the end the dequantising warps read D back (tcgen05.ld) into shared memory, the cluster's
//     first CTA adds the k-split partial sums through distributed shared memory, applies addend
//     and activation and writes Y row-major with coalesced stores.
// Every mbarrier wait is bounded; a wait that gives up records a code and all roles fall through
// to the common exit.
#include <mutex>

#include "q4b_sm100_ptx.cuh"

namespace q4b {
namespace gemmtm {

using namespace ptx;

constexpr int PANEL_TILES = 8;                       // column tiles per CTA
constexpr int PANEL_N = PANEL_TILES * TILE_N;        // 128 = lanes of tensor memory
constexpr int MAX_ROWS = 128;                        // rows of X (columns of the accumulator)
constexpr int DEQ_GROUPS = 2;                        // groups of four warps; group i takes k-tiles i, i+2, ...
constexpr int DEQ_WARPS = 4 * DEQ_GROUPS;
constexpr int WARP_MMA = DEQ_WARPS, WARP_W = DEQ_WARPS + 1, WARP_X = DEQ_WARPS + 2;
constexpr int THREADS = (DEQ_WARPS + 3) * 32;
constexpr int STAGE_STEPS = 2;                       // k-tiles per packed-weight stage: one for each group
constexpr int TILE_RUN_BYTES = STAGE_STEPS * TILE_BYTES;             // 1152
constexpr int STAGE_BYTES = PANEL_TILES * TILE_RUN_BYTES;            // 9216
constexpr int NSTAGE = 4;
constexpr int SX = 4;                                // X slices in flight
constexpr int X_STAGE_BYTES = MAX_ROWS * TILE_K * 2; // 16384
constexpr int TM_STAGES = 4;                         // k-tiles whose A operand tensor memory holds
constexpr int TMEM_COLS = 256;                       // D: up to 128 columns, A: 4 x (2 blocks x 16); two CTAs fit an SM
constexpr int D_COL0 = 0, A_COL0 = 128;
constexpr int SMEM_RING = 0;                         // ring and X slices are reused for the partial sums [rows][128] fp32 at the end
constexpr int SMEM_X = SMEM_RING + NSTAGE * STAGE_BYTES;             // 73728, a multiple of 1024
constexpr int SMEM_BAR = SMEM_X + SX * X_STAGE_BYTES;
constexpr int NUM_BARS = 2 * NSTAGE + 2 * TM_STAGES + 2 * SX + 1;
constexpr int SMEM_DYN = SMEM_BAR + NUM_BARS * 8 + 1024;             // + slack to align the base to 1024 bytes
static_assert(NSTAGE * STAGE_BYTES + SX * X_STAGE_BYTES >= MAX_ROWS * PANEL_N * 4, "the partial sums reuse the rings");
static_assert(SMEM_X % 1024 == 0, "swizzled tiles need 1024-byte alignment");

__device__ int g_status = 0;

template <bool BF16>
__global__ void __launch_bounds__(THREADS, 2)
gemm_tmem_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_r,
                 const uint8_t *__restrict__ prepacked, const uint16_t *__restrict__ corr_op, int KF, int M, int64_t K,
                 int64_t N, uint16_t *__restrict__ y, int64_t ldy, const float *__restrict__ addend, int64_t ld_add, int KS,
                 int rows, int act) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;

    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bar0 = base + SMEM_BAR;
    auto bar_full_w = [&](int s) { return bar0 + 8u * s; };                                // packed tiles landed
    auto bar_empty_w = [&](int s) { return bar0 + 8u * (NSTAGE + s); };                    // both groups have read them
    auto bar_a_full = [&](int s) { return bar0 + 8u * (2 * NSTAGE + s); };                 // A operand in tensor memory
    auto bar_a_empty = [&](int s) { return bar0 + 8u * (2 * NSTAGE + TM_STAGES + s); };    // its MMAs retired
    auto bar_x_full = [&](int s) { return bar0 + 8u * (2 * NSTAGE + 2 * TM_STAGES + s); }; // X slice landed
    auto bar_x_empty = [&](int s) { return bar0 + 8u * (2 * NSTAGE + 2 * TM_STAGES + SX + s); };
    const uint32_t bar_d_done = bar0 + 8u * (2 * NSTAGE + 2 * TM_STAGES + 2 * SX);         // every MMA retired

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int *abort_flag = &s_abort;

    const int NT = (int)tiles_n(N);
    const int KU = (int)tiles_k(K);
    const int panel = (int)blockIdx.x / KS, ks = (int)blockIdx.x % KS;    // ks = rank in the cluster
    const int nt0 = panel * PANEL_TILES;
    const int valid = min(PANEL_TILES, NT - nt0);                          // column tiles that exist
    // k-tiles of the product: first the KF tiles of the group-wise format's folded zero-point term (A operand
    // read as bf16 from corr_op [N, 64 KF], X side through tmap_r: bf16 [M, 64 KF]; KF = 0: none), then the
    // KU packed ones.  The cluster splits all of them.
    const int KT = KF + KU;
    const int ku0 = (int)((int64_t)KT * ks / KS), ku1 = (int)((int64_t)KT * (ks + 1) / KS);
    const int nsteps = ku1 - ku0;                                          // k-tiles of this CTA
    const int nstages = (nsteps + STAGE_STEPS - 1) / STAGE_STEPS;

    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int s = 0; s < NSTAGE; ++s) { mbar_init(bar_full_w(s), 1); mbar_init(bar_empty_w(s), 4 * STAGE_STEPS); }
        for (int s = 0; s < TM_STAGES; ++s) { mbar_init(bar_a_full(s), 4); mbar_init(bar_a_empty(s), 1); }
        for (int s = 0; s < SX; ++s) { mbar_init(bar_x_full(s), 1); mbar_init(bar_x_empty(s), 1); }
        mbar_init(bar_d_done, 1);
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
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == WARP_W) {
        // ---------------- packed-weight producer: lane t copies column tile t's run of the stage ----------------
        const uint8_t *src = prepacked + tile_offset(nt0 + min(lane, valid - 1), 0, KU);
        for (int q = 0; q < nstages; ++q) {
            const int slot = q % NSTAGE;
            if (!mbar_wait_warp(bar_empty_w(slot), ((q / NSTAGE) & 1) ^ 1, abort_flag, &g_status, 401)) goto done;
            const int s0 = ku0 + q * STAGE_STEPS;                          // first k-tile of the stage
            const int t0 = max(s0, KF), t1 = min(s0 + STAGE_STEPS, ku1);   // its packed k-tiles: [t0, t1)
            if (t1 <= t0) {                                                // folded-term tiles only: nothing to copy
                if (lane == 0) mbar_arrive(bar_full_w(slot));
                continue;
            }
            const uint32_t bytes = (uint32_t)((t1 - t0) * TILE_BYTES);
            if (lane == 0) mbar_arrive_expect_tx(bar_full_w(slot), (uint32_t)valid * bytes);
            __syncwarp();
            if (lane < valid)
                bulk_load(base + SMEM_RING + slot * STAGE_BYTES + lane * TILE_RUN_BYTES + (t0 - s0) * TILE_BYTES,
                          src + (size_t)(t0 - KF) * TILE_BYTES, bytes, bar_full_w(slot));
        }
    } else if (warp == WARP_X) {
        // ---------------- X producer (x depends on earlier kernels of the stream; the weights do not) ----------------
        asm volatile("griddepcontrol.wait;" ::: "memory");
        if (lane == 0) {
            for (int i = 0; i < nsteps; ++i) {
                const int s = i % SX;
                if (!mbar_wait(bar_x_empty(s), ((i / SX) & 1) ^ 1, abort_flag, &g_status, 402)) goto done;
                mbar_arrive_expect_tx(bar_x_full(s), (uint32_t)(rows * TILE_K * 2));
                const int t = ku0 + i;
                if (t >= KF) tma_load_2d(base + SMEM_X + s * X_STAGE_BYTES, &tmap_x, (t - KF) * TILE_K, 0, bar_x_full(s));
                else tma_load_2d(base + SMEM_X + s * X_STAGE_BYTES, &tmap_r, t * TILE_K, 0, bar_x_full(s));
            }
        }
    } else if (warp == WARP_MMA) {
        // ---------------- MMA issuer: converged warp, one elected lane issues ----------------
        const uint32_t idesc = make_idesc(BF16, PANEL_N, rows), idesc_fold = make_idesc(true, PANEL_N, rows);   // the folded term is bf16
        for (int i = 0; i < nsteps; ++i) {
            const int st = i % TM_STAGES, xs = i % SX;
            const uint32_t id = ku0 + i >= KF ? idesc : idesc_fold;
            if (!mbar_wait_warp(bar_a_full(st), (i / TM_STAGES) & 1, abort_flag, &g_status, 403)) goto done;
            if (!mbar_wait_warp(bar_x_full(xs), (i / SX) & 1, abort_flag, &g_status, 404)) goto done;
            tc_fence_after();
            if (elect_one()) {
                const uint64_t bdesc = make_kmajor_sw128_desc(base + SMEM_X + xs * X_STAGE_BYTES);
#pragma unroll
                for (int k = 0; k < TILE_K / 16; ++k)
                    tc_mma_ts_f16(tmem_base + D_COL0, tmem_base + (uint32_t)(A_COL0 + st * 32 + k * 8), bdesc + 2 * k, id,
                                  (uint32_t)((i | k) != 0));
                tc_commit(bar_a_empty(st));
                tc_commit(bar_x_empty(xs));
                if (i == nsteps - 1) tc_commit(bar_d_done);
            }
            __syncwarp();
        }
    } else {
        // ---------------- dequantise into tensor memory ----------------
        const int grp = warp >> 2, wq = warp & 3;                 // wq = tensor-memory lane quadrant
        const int tile = 2 * wq + (lane >> 4);                    // column tile of the panel
        const int r = lane & 15, g = r & 7, hi = r >> 3;          // row of the tile: g + 8 hi
        const uint32_t lane_taddr = tmem_base + ((uint32_t)(wq * 32) << 16);
        // word (kb, octet c) of this row: slot_of(g, c) * 16 + (kb * 2 + hi) * 4 inside the tile
        uint32_t woff[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) woff[c] = (uint32_t)(tile * TILE_RUN_BYTES + slot_of(g, c) * 16 + hi * 4);
        const uint32_t doff = (uint32_t)(tile * TILE_RUN_BYTES + TILE_QS_BYTES + g * 8 + hi * 2);

        for (int i = grp; i < nsteps; i += DEQ_GROUPS) {
            const int q = i / STAGE_STEPS, slot = q % NSTAGE, st = i % TM_STAGES;
            if (!mbar_wait_warp(bar_full_w(slot), (q / NSTAGE) & 1, abort_flag, &g_status, 405)) goto done;
            if (!mbar_wait_warp(bar_a_empty(st), ((i / TM_STAGES) & 1) ^ 1, abort_flag, &g_status, 406)) goto done;
            tc_fence_after();
            const uint32_t a_addr = lane_taddr + (uint32_t)(A_COL0 + st * 32);
            if (ku0 + i >= KF) {
                dequant_tile_to_tmem<BF16>(base + SMEM_RING + slot * STAGE_BYTES + (i % STAGE_STEPS) * TILE_BYTES, woff, doff, a_addr);
            } else {
                // a k-tile of the folded term: this thread's column of corr_op, 64 bf16 = 2 x 16 words
                const int64_t n = (int64_t)nt0 * TILE_N + wq * 32 + lane;
                const uint4 *src = reinterpret_cast<const uint4 *>(corr_op + (size_t)n * (size_t)(KF * TILE_K) + (size_t)(ku0 + i) * TILE_K);
#pragma unroll
                for (int kb = 0; kb < 2; ++kb) {
                    uint32_t regs[16];
#pragma unroll
                    for (int v4 = 0; v4 < 4; ++v4) {
                        const uint4 t = n < N ? __ldg(src + kb * 4 + v4) : make_uint4(0u, 0u, 0u, 0u);
                        regs[4 * v4] = t.x; regs[4 * v4 + 1] = t.y; regs[4 * v4 + 2] = t.z; regs[4 * v4 + 3] = t.w;
                    }
                    tc_st_32x32b_x16(a_addr + (uint32_t)(kb * 16), regs);
                }
            }
            tc_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(bar_a_full(st));
                mbar_arrive(bar_empty_w(slot));
            }
        }
        // accumulator -> shared memory, [row of X][column of the panel] fp32 (the ring is idle by now)
        if (nsteps > 0) {
            if (!mbar_wait_warp(bar_d_done, 0, abort_flag, &g_status, 407)) goto done;
            tc_fence_after();
        }
        float *part = reinterpret_cast<float *>(smem + SMEM_RING);
        for (int ch = grp; ch < rows / 16; ch += DEQ_GROUPS) {
            uint32_t v[16];
            if (nsteps > 0) {
                tc_ld_32x32b_x16(lane_taddr + (uint32_t)(D_COL0 + ch * 16), v);
                tc_wait_ld();
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] = 0u;
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) part[(ch * 16 + j) * PANEL_N + wq * 32 + lane] = __uint_as_float(v[j]);
        }
    }

done:
    tc_fence_before();
    __syncthreads();
    asm volatile("griddepcontrol.wait;" ::: "memory");   // y may still be in use by earlier work on the stream
    if (KS > 1) cluster_sync_all();                    // every CTA's partial sums are in its shared memory
    if (!s_abort) {
        // Every CTA of the cluster finishes a slice of the rows: its own partial sums plus the other
        // CTAs' (read through distributed shared memory), always added in rank order.
        const uint32_t part_s = base + SMEM_RING;
        const int m0 = rows * ks / KS, m1 = rows * (ks + 1) / KS;
        for (int idx = threadIdx.x; idx < (m1 - m0) * (PANEL_N / 4); idx += THREADS) {
            const int m = m0 + idx / (PANEL_N / 4), c4 = idx % (PANEL_N / 4);
            const uint32_t off = (uint32_t)((m * PANEL_N + c4 * 4) * 4);
            float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            for (int rk = 0; rk < KS; ++rk) {
                const float4 v = rk == ks ? *reinterpret_cast<const float4 *>(smem + SMEM_RING + off)
                                          : ld_cluster_f32x4(part_s + off, (uint32_t)rk);
                sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
            }
            const int n = nt0 * TILE_N + c4 * 4;
            if (m < M) {
                const float out[4] = {sum.x, sum.y, sum.z, sum.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (n + j < N) {
                        float v = out[j];
                        if (addend != nullptr) v += addend[(size_t)m * ld_add + n + j];     // fp32 term added before the one rounding
                        v = apply_act(v, act);
                        if constexpr (BF16) y[(size_t)m * ldy + n + j] = __bfloat16_as_ushort(__float2bfloat16_rn(v));
                        else y[(size_t)m * ldy + n + j] = __half_as_ushort(__float2half_rn(v));
                    }
                }
            }
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

// k-split: the number of CTAs per panel that needs the fewest (waves of CTAs) x (k-tiles per CTA)
static int choose_ksplit(int64_t panels, int64_t KU, int sms) {
    int best = 1;
    int64_t best_cost = -1;
    for (int ks = 1; ks <= 8 && ks <= KU; ++ks) {
        const int64_t waves = ceil_div(panels * ks, 2 * sms);            // two CTAs fit an SM
        const int64_t cost = waves * (ceil_div(KU, ks) + 6) + ks;      // + fixed cost of a wave, + the reduction
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = ks; }
    }
    return best;
}

template <bool BF16>
static int launch(const CUtensorMap &tmap, const CUtensorMap &tmap_r, const void *prepacked, const void *corr_op, int KF, int M,
                  int64_t K, int64_t N, void *y, int64_t ldy, const float *addend, int64_t ld_add, int rows, int act, int flags,
                  int sms, cudaStream_t st) {
    {   // opt in to the large dynamic shared memory once per device and instantiation
        static bool attr_done[64] = {};
        static std::mutex attr_mu;
        int dev = 0;
        Q4B_CUDA_TRY(cudaGetDevice(&dev));
        std::lock_guard<std::mutex> attr_lock(attr_mu);
        if (dev < 0 || dev >= 64 || !attr_done[dev]) {
            Q4B_CUDA_TRY(cudaFuncSetAttribute(gemm_tmem_kernel<BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_DYN));
            if (dev >= 0 && dev < 64) attr_done[dev] = true;
        }
    }
    const int64_t panels = ceil_div(tiles_n(N), PANEL_TILES);
    int ks = choose_ksplit(panels, tiles_k(K) + KF, sms);
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
    Q4B_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemm_tmem_kernel<BF16>, tmap, tmap_r, (const uint8_t *)prepacked, (const uint16_t *)corr_op, KF,
                                    M, K, N, (uint16_t *)y, ldy, addend, ld_add, ks, rows, act));
    return Q4B_OK;
}

}  // namespace gemmtm

int device_sm_count();

// Arguments as checked by the matmul entry points; 1 <= M <= 128.
int gemm_tmem_launch(const void *x, int bf16, int M, int64_t ldx, const void *prepacked, int64_t K, int64_t N,
                     const float *addend, int64_t ld_add, void *y, int64_t ldy, int flags, cudaStream_t st, const void *corr_op,
                     const void *xr, int KX) {
    if (M < 1 || M > gemmtm::MAX_ROWS) return Q4B_ERR_SHAPE;
    const int rows = (M + 15) / 16 * 16;                                   // the MMA's N: a multiple of 16
    CUtensorMap tmap, tmap_r;
    if (int rc = encode_x_tensor_map(&tmap, x, bf16, M, K, ldx, rows)) return rc;       // 64 k x `rows` rows per copy
    const bool fold = corr_op != nullptr && xr != nullptr && KX > 0;       // the group-wise format's folded term
    if (fold) {
        if (int rc = encode_x_tensor_map(&tmap_r, xr, 1, M, (int64_t)KX * TILE_K, (int64_t)KX * TILE_K, rows)) return rc;
    } else {
        tmap_r = tmap;
    }
    const int sms = device_sm_count();
    const int act = act_of_flags(flags);
    return bf16 ? gemmtm::launch<true>(tmap, tmap_r, prepacked, corr_op, fold ? KX : 0, M, K, N, y, ldy, addend, ld_add, rows, act, flags, sms, st)
                : gemmtm::launch<false>(tmap, tmap_r, prepacked, corr_op, fold ? KX : 0, M, K, N, y, ldy, addend, ld_add, rows, act, flags, sms, st);
}

// read and clear this file's wait status (host side; the caller has synchronised the stream)
int gemm_tmem_wait_status(int *value) {
    int h = 0;
    Q4B_CUDA_TRY(cudaMemcpyFromSymbol(&h, gemmtm::g_status, sizeof(int)));
    if (h != 0) {
        const int zero = 0;
        Q4B_CUDA_TRY(cudaMemcpyToSymbol(gemmtm::g_status, &zero, sizeof(int)));
    }
    *value = h;
    return Q4B_OK;
}

}  // namespace q4b
