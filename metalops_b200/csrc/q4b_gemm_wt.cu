// Prefill with the WEIGHTS as the tensor cores' A operand in tensor memory, persistent.
//
// Replaces the reference's 64x32-tile simdgroup kernel matmul_ggml_q4_0
// (packages/metalcore/src/metalcore/native/quant_kernels.metal:1738-1886, launched by
// core_mps.mm:5917-5975) for M above 128.  A kernel that dequantises into shared memory is bounded by
// what moves through shared memory per k-tile (TMA writes of X and W, the dequantised operand written
// and then read once per 128-row MMA).  Here the dequantised weights never touch shared memory:
//   * a work item is a panel of 128 output columns (the 128 lanes of tensor memory) x up to 256 rows of
//     X x all of k; one persistent CTA per SM takes items row tile by row tile, so the CTAs running at
//     any time share their X slices through L2;
//   * a pipeline stage is two k-tiles (128 k): its two [rows x 64 k] slices of X land in shared memory
//     by TMA (128-byte swizzle) and its weights are written to tensor memory by the dequantising warps,
//     all counted on ONE barrier, so the MMA warp waits once and commits once per eight MMAs (an issuing
//     thread spends about 75 cycles per tcgen05.mma and a few hundred per wait/commit pair);
//   * sixteen warps (four groups on alternate k-tiles) dequantise straight into tensor memory
//     (tcgen05.st, thread = output column, (q-8)*d rounded once to bf16/fp16 as in the other kernels);
//   * one elected lane issues tcgen05.mma M128 x N=rows x K16 with A from tensor memory and B = the X
//     slice, all k of an item into one accumulator D[column][row] (up to 256 columns of tensor memory);
//   * eight epilogue warps read D back (tcgen05.ld), add the optional fp32 addend, apply the activation
//     and store row-major, 32 consecutive columns per store instruction, while the other roles already
//     run the next item's loads and dequantisation (only its MMAs wait for the drain).
// Every mbarrier wait is bounded (codes 601-608); a wait that gives up raises the CTA's abort flag and
// all roles leave through the common exit, which frees the tensor memory.
#include <cuda.h>

#include <mutex>

#include "q4b_sm100_ptx.cuh"

namespace q4b {
namespace gemmwt {

using namespace ptx;

constexpr int PANEL_TILES = 8;                       // column tiles per item
constexpr int PANEL_N = PANEL_TILES * TILE_N;        // 128 = lanes of tensor memory
constexpr int MAX_ROWS = 256;                        // rows of X per item (columns of the accumulator)
constexpr int DEQ_GROUPS = 4;                        // groups of four warps; a group takes every fourth k-tile
constexpr int DEQ_WARPS = 4 * DEQ_GROUPS;
constexpr int EPI_WARPS = 8;                         // two per lane quadrant of tensor memory
constexpr int WARP_MMA = DEQ_WARPS, WARP_W = DEQ_WARPS + 1, WARP_X = DEQ_WARPS + 2, WARP_EPI0 = DEQ_WARPS + 3;
constexpr int THREADS = (WARP_EPI0 + EPI_WARPS) * 32;   // 864
constexpr int STAGE_STEPS = 2;                       // k-tiles per stage: one barrier wait and one commit per 8 MMAs
constexpr int TILE_RUN_BYTES = STAGE_STEPS * TILE_BYTES;
constexpr int W_STAGE_BYTES = PANEL_TILES * TILE_RUN_BYTES;          // 9216
constexpr int NSTAGE_W = 3;                          // packed-weight stages in flight
constexpr int ST = 3;                                // operand stages: X slices in shared memory, A in tensor memory
constexpr int X_TILE_BYTES = MAX_ROWS * TILE_K * 2;  // 32768: 256 rows x 64 k
constexpr int X_STAGE_BYTES = STAGE_STEPS * X_TILE_BYTES;
constexpr int TMEM_COLS = 512;                       // D: 256 columns, A: 3 stages x 2 k-tiles x (2 blocks x 16)
constexpr int D_COL0 = 0, A_COL0 = MAX_ROWS;
constexpr int SMEM_X = 0;
constexpr int SMEM_RING = SMEM_X + ST * X_STAGE_BYTES;               // 196608
constexpr int SMEM_BAR = SMEM_RING + NSTAGE_W * W_STAGE_BYTES;
constexpr int NUM_BARS = 3 * NSTAGE_W + 2 * ST + 2;
constexpr int SMEM_DYN = SMEM_BAR + NUM_BARS * 8 + 1024;             // + slack to align the base to 1024 bytes
static_assert(A_COL0 + ST * STAGE_STEPS * 32 <= TMEM_COLS, "operand stages exceed tensor memory");
static_assert(SMEM_DYN <= 227 * 1024, "shared memory");

__device__ int g_status = 0;

// GENERAL: the epilogue adds the fp32 addend and applies the activation; without it (its own instantiation,
// so that the common case keeps its registers) it only converts and stores.  FOLD: the item's first KX
// k-tiles are the group-wise format's folded zero-point term.
template <bool BF16, bool GENERAL, bool FOLD>
__global__ void __launch_bounds__(THREADS, 1)
gemm_wt_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_r,
               const uint8_t *__restrict__ prepacked, const uint16_t *__restrict__ corr_op, int KX, int M, int64_t K, int64_t N,
               uint16_t *__restrict__ y, int64_t ldy, const float *__restrict__ addend, int64_t ld_add, int rows, int act) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;

    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar0 = base + SMEM_BAR;
    // "packed tiles landed": two barriers per slot, for its even and its odd fills (see the dequantisers)
    auto bar_full_w = [&](int s, int fill) { return bar0 + 8u * (2 * s + (fill & 1)); };
    auto bar_empty_w = [&](int s) { return bar0 + 8u * (2 * NSTAGE_W + s); };        // the groups have read them
    auto bar_full = [&](int s) { return bar0 + 8u * (3 * NSTAGE_W + s); };           // stage s: X landed and A written
    auto bar_empty = [&](int s) { return bar0 + 8u * (3 * NSTAGE_W + ST + s); };     // its MMAs retired
    const uint32_t bar_d_full = bar0 + 8u * (3 * NSTAGE_W + 2 * ST);                 // an item's MMAs retired
    const uint32_t bar_d_empty = bar_d_full + 8u;                                    // the accumulator was read out

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int *abort_flag = &s_abort;

    const int NT = (int)tiles_n(N);
    const int KU = (int)tiles_k(K);
    const int panels = (NT + PANEL_TILES - 1) / PANEL_TILES;
    const int row_tiles = (M + rows - 1) / rows;               // `rows`: height of a row tile, chosen by the host
    const int items = panels * row_tiles;
    // Folded rank-G term (FOLD only): KX further k-tiles whose A operand is read as bf16 from corr_op
    // [N, 64 KX] and whose X slices come from a second tensor map (bf16 [M, 64 KX]); KT counts all k-tiles.
    // They come first in an item, so that their operand loads (global memory, not the ring) pass while the
    // previous item's accumulator is still being read out.
    const int KF = FOLD ? KX : 0;                                       // k-tiles of the folded term, first in every item
    const int KT = KU + KF;
    const int spi = (KT + STAGE_STEPS - 1) / STAGE_STEPS;                  // stages per item

    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int s = 0; s < NSTAGE_W; ++s) {
            mbar_init(bar_full_w(s, 0), 1);
            mbar_init(bar_full_w(s, 1), 1);
            mbar_init(bar_empty_w(s), 4 * STAGE_STEPS);
        }
        // a stage is full when the X producer's expect-tx arrival, its bytes and the four warps of each
        // of its two k-tiles have arrived; one tcgen05.commit empties it
        for (int s = 0; s < ST; ++s) { mbar_init(bar_full(s), 1 + 4 * STAGE_STEPS); mbar_init(bar_empty(s), 1); }
        mbar_init(bar_d_full, 1);
        mbar_init(bar_d_empty, EPI_WARPS);
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

    if (warp == WARP_W) {
        // ---------------- packed-weight producer: lane t copies column tile t's run of the stage ----------------
        int gq = 0;                                                        // stages issued so far, over all items
        for (int item = blockIdx.x; item < items; item += gridDim.x) {
            const int nt0 = (item % panels) * PANEL_TILES;
            const int valid = min(PANEL_TILES, NT - nt0);
            const uint8_t *src = prepacked + tile_offset(nt0 + min(lane, valid - 1), 0, KU);
            for (int q = 0; q < spi; ++q, ++gq) {
                const int slot = gq % NSTAGE_W, fill = gq / NSTAGE_W;
                if (!mbar_wait_warp(bar_empty_w(slot), (fill & 1) ^ 1, abort_flag, &g_status, 601)) goto done;
                // the item's k-tiles: first the KF tiles of the folded term (nothing to copy), then the packed ones
                const int t0 = max(q * STAGE_STEPS, KF), t1 = min(q * STAGE_STEPS + STAGE_STEPS, KT);   // packed tiles of the stage: [t0, t1)
                if (t1 <= t0) {
                    if (lane == 0) mbar_arrive(bar_full_w(slot, fill));
                    continue;
                }
                const uint32_t bytes = (uint32_t)((t1 - t0) * TILE_BYTES);
                if (lane == 0) mbar_arrive_expect_tx(bar_full_w(slot, fill), (uint32_t)valid * bytes);
                __syncwarp();
                if (lane < valid)
                    bulk_load(base + SMEM_RING + slot * W_STAGE_BYTES + lane * TILE_RUN_BYTES + (t0 - q * STAGE_STEPS) * TILE_BYTES,
                              src + (size_t)(t0 - KF) * TILE_BYTES, bytes, bar_full_w(slot, fill));
            }
        }
    } else if (warp == WARP_X) {
        // ---------------- X producer: the stage's one or two [rows x 64 k] slices ----------------
        if (lane == 0) {
            int gq = 0;
            for (int item = blockIdx.x; item < items; item += gridDim.x) {
                const int row0 = (item / panels) * rows;
                for (int q = 0; q < spi; ++q, ++gq) {
                    const int s = gq % ST;
                    if (!mbar_wait(bar_empty(s), ((gq / ST) & 1) ^ 1, abort_flag, &g_status, 602)) goto done;
                    const int nk = min(STAGE_STEPS, KT - q * STAGE_STEPS);
                    mbar_arrive_expect_tx(bar_full(s), (uint32_t)(nk * rows * TILE_K * 2));
                    for (int j = 0; j < nk; ++j) {
                        const int tile = q * STAGE_STEPS + j;
                        const uint32_t dst = base + SMEM_X + s * X_STAGE_BYTES + j * X_TILE_BYTES;
                        if (tile >= KF) tma_load_2d(dst, &tmap_x, (tile - KF) * TILE_K, row0, bar_full(s));
                        else tma_load_2d(dst, &tmap_r, tile * TILE_K, row0, bar_full(s));
                    }
                }
            }
        }
    } else if (warp == WARP_MMA) {
        // ---------------- MMA issuer: converged warp, one elected lane issues ----------------
        // An issuing thread spends about 75 cycles per tcgen05.mma and a few hundred per wait/commit
        // pair, and the tensor pipe queues only an instruction or two: hence one wait and one commit per
        // stage of eight MMAs.  (Splitting the rows between two issuing warps is slower: an MMA of 128
        // rows takes the pipe about 97 cycles, not half of the 128 that one of 256 rows takes.)
        const uint32_t idesc = make_idesc(BF16, PANEL_N, rows), idesc_fold = make_idesc(true, PANEL_N, rows);   // the folded term is bf16
        int gq = 0, itl = 0;
        for (int item = blockIdx.x; item < items; item += gridDim.x, ++itl) {
            if (!mbar_wait_warp(bar_d_empty, (uint32_t)(itl & 1) ^ 1u, abort_flag, &g_status, 603)) goto done;   // the previous item was read out
            tc_fence_after();
            for (int q = 0; q < spi; ++q, ++gq) {
                const int s = gq % ST;
                if (!mbar_wait_warp(bar_full(s), (gq / ST) & 1, abort_flag, &g_status, 604)) goto done;
                tc_fence_after();
                if (elect_one()) {
                    const uint64_t bdesc = make_kmajor_sw128_desc(base + SMEM_X + s * X_STAGE_BYTES);
                    const uint32_t a0 = tmem_base + (uint32_t)(A_COL0 + s * STAGE_STEPS * 32);
                    const uint32_t id0 = q * STAGE_STEPS >= KF ? idesc : idesc_fold;
                    const uint32_t id1 = q * STAGE_STEPS + 1 >= KF ? idesc : idesc_fold;
#pragma unroll
                    for (int k = 0; k < TILE_K / 16; ++k)
                        tc_mma_ts_f16(tmem_base + D_COL0, a0 + k * 8, bdesc + 2 * k, id0, (uint32_t)((q | k) != 0));
                    if (q * STAGE_STEPS + 1 < KT) {
#pragma unroll
                        for (int k = 0; k < TILE_K / 16; ++k)
                            tc_mma_ts_f16(tmem_base + D_COL0, a0 + 32 + k * 8, bdesc + (X_TILE_BYTES >> 4) + 2 * k, id1, 1u);
                    }
                    tc_commit(bar_empty(s));
                    if (q == spi - 1) tc_commit(bar_d_full);
                }
                __syncwarp();
            }
        }
    } else if (warp >= WARP_EPI0) {
        // ---------------- epilogue: two warps per lane quadrant, half of the rows each ----------------
        const int quad = warp & 3, half = (warp - WARP_EPI0) >> 2;
        const uint32_t lane_taddr = tmem_base + ((uint32_t)(quad * 32) << 16);
        const int nch = (rows + 31) / 32, ch0 = half * ((nch + 1) / 2), ch1 = half == 0 ? (nch + 1) / 2 : nch;   // chunks of 32 rows
        int itl = 0;
        for (int item = blockIdx.x; item < items; item += gridDim.x, ++itl) {
            const int row0 = (item / panels) * rows;
            const int n = (item % panels) * PANEL_N + quad * 32 + lane;
            if (GENERAL && addend != nullptr && ld_add != 0 && lane == 0) {
                // the item's main loop takes tens of microseconds: ask L2 for this warp's part of the addend
                // tile (a 128-byte line per row) now, so that the drain does not wait for DRAM
                const int nq = (item % panels) * PANEL_N + quad * 32;
                if (nq < N)
                    for (int rr = ch0 * 32; rr < min(ch1 * 32, rows) && row0 + rr < M; ++rr)
                        asm volatile("prefetch.global.L2 [%0];" ::"l"(addend + (size_t)(row0 + rr) * ld_add + nq));
            }
            if (!mbar_wait_warp(bar_d_full, (uint32_t)(itl & 1), abort_flag, &g_status, 606)) goto done;
            tc_fence_after();
#pragma unroll 1
            for (int ch = ch0; ch < ch1; ++ch) {
                uint32_t v[2][16];
                tc_ld_32x32b_x16(lane_taddr + (uint32_t)(D_COL0 + ch * 32), v[0]);
                if (ch * 32 + 16 < rows) tc_ld_32x32b_x16(lane_taddr + (uint32_t)(D_COL0 + ch * 32 + 16), v[1]);
                tc_wait_ld();
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const int m0 = row0 + ch * 32 + u * 16;
                    if (n < N && m0 < M && ch * 32 + u * 16 < rows) {
                        uint16_t *yp = y + (size_t)m0 * ldy + n;
                        if (!GENERAL && m0 + 16 <= M) {
                            // the common case costs a conversion, a store and an address step per element
#pragma unroll
                            for (int j = 0; j < 16; ++j, yp += ldy) {
                                const float f = __uint_as_float(v[u][j]);
                                if constexpr (BF16) *yp = __bfloat16_as_ushort(__float2bfloat16_rn(f));
                                else *yp = __half_as_ushort(__float2half_rn(f));
                            }
                        } else if constexpr (!GENERAL) {
                            const int jn = min(16, M - m0);
#pragma unroll
                            for (int j = 0; j < 16; ++j, yp += ldy) {
                                if (j < jn) {
                                    const float f = __uint_as_float(v[u][j]);
                                    if constexpr (BF16) *yp = __bfloat16_as_ushort(__float2bfloat16_rn(f));
                                    else *yp = __half_as_ushort(__float2half_rn(f));
                                }
                            }
                        } else {
                            // the addend's sixteen values first, all loads in flight together: interleaved
                            // with the stores they would wait for one another (the stores may alias them);
                            // a bias row (ld_add = 0) is one value for the whole column
                            const int jn = min(16, M - m0);
                            float a[16];
                            if (addend == nullptr || ld_add == 0) {
                                const float b = addend != nullptr ? __ldg(addend + n) : 0.0f;
#pragma unroll
                                for (int j = 0; j < 16; ++j) a[j] = b;
                            } else {
#pragma unroll
                                for (int j = 0; j < 16; ++j) a[j] = j < jn ? __ldg(addend + (size_t)(m0 + j) * ld_add + n) : 0.0f;
                            }
                            if (act == 0 && jn == 16) {           // uniform: a full chunk without activation
#pragma unroll
                                for (int j = 0; j < 16; ++j, yp += ldy) {
                                    const float f = __uint_as_float(v[u][j]) + a[j];              // fp32 term added before the one rounding
                                    if constexpr (BF16) *yp = __bfloat16_as_ushort(__float2bfloat16_rn(f));
                                    else *yp = __half_as_ushort(__float2half_rn(f));
                                }
                            } else {
#pragma unroll
                                for (int j = 0; j < 16; ++j, yp += ldy) {
                                    if (j < jn) {
                                        const float f = apply_act(__uint_as_float(v[u][j]) + a[j], act);
                                        if constexpr (BF16) *yp = __bfloat16_as_ushort(__float2bfloat16_rn(f));
                                        else *yp = __half_as_ushort(__float2half_rn(f));
                                    }
                                }
                            }
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_d_empty);
        }
    } else {
        // ---------------- dequantise into tensor memory ----------------
        const int grp = warp >> 2, wq = warp & 3;                 // wq = tensor-memory lane quadrant
        const int tile = 2 * wq + (lane >> 4);                    // column tile of the panel
        const int r = lane & 15, g = r & 7, hi = r >> 3;          // row of the tile: g + 8 hi
        const uint32_t lane_taddr = tmem_base + ((uint32_t)(wq * 32) << 16);
        uint32_t woff[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) woff[c] = (uint32_t)(tile * TILE_RUN_BYTES + slot_of(g, c) * 16 + hi * 4);
        const uint32_t doff = (uint32_t)(tile * TILE_RUN_BYTES + TILE_QS_BYTES + g * 8 + hi * 2);

        // A waiter on an mbarrier tells phases apart by parity only, so it must never test a barrier that
        // is still a phase behind the one before its own.  "Stage empty": a group takes every fourth
        // k-tile, so its previous wait (two stages back, hence the stage five back retired) implies that
        // the slot's use six stages back has retired, MMAs retiring in order.  "Weights landed": a slot's
        // even and odd fills complete on different barriers, so a test can only be fooled by the fill TWO
        // before its own being outstanding; that fill was consumed before the producer issued the one in
        // between, which it issued before the fill this group has already seen land (two stages back).
        int gbase = 0, itl = 0;                                   // global index of the item's first k-tile
        for (int item = blockIdx.x; item < items; item += gridDim.x, ++itl, gbase += KT) {
            // this group's k-tiles of the item: those whose global index is grp modulo the number of groups
            int i = (grp - gbase % DEQ_GROUPS + DEQ_GROUPS) % DEQ_GROUPS;
            for (; i < KT; i += DEQ_GROUPS) {
                const int gq = itl * spi + i / STAGE_STEPS, sub = i % STAGE_STEPS;
                const int wslot = gq % NSTAGE_W, fill = gq / NSTAGE_W, s = gq % ST;
                if (!mbar_wait_warp(bar_full_w(wslot, fill), (fill >> 1) & 1, abort_flag, &g_status, 607)) goto done;
                if (!mbar_wait_warp(bar_empty(s), ((gq / ST) & 1) ^ 1, abort_flag, &g_status, 608)) goto done;
                tc_fence_after();
                const uint32_t a_addr = lane_taddr + (uint32_t)(A_COL0 + (s * STAGE_STEPS + sub) * 32);
                if (!FOLD || i >= KF) {
                    dequant_tile_to_tmem<BF16>(base + SMEM_RING + wslot * W_STAGE_BYTES + sub * TILE_BYTES, woff, doff, a_addr);
                } else {
                    // a k-tile of the folded term: this thread's column of corr_op, 64 bf16 = 2 x 16 words
                    const int64_t n = (int64_t)(item % panels) * PANEL_N + wq * 32 + lane;
                    const uint4 *src = reinterpret_cast<const uint4 *>(corr_op + (size_t)n * (size_t)(KX * TILE_K) + (size_t)i * TILE_K);
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
                    mbar_arrive(bar_full(s));
                    mbar_arrive(bar_empty_w(wslot));
                    // a stage that holds a single k-tile (odd number of k-tiles, the item's last stage) still
                    // has to collect the arrivals of two
                    if ((KT & 1) && i == KT - 1) {
                        mbar_arrive(bar_full(s));
                        mbar_arrive(bar_empty_w(wslot));
                    }
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
        __syncthreads();
    }
    if (warp == WARP_MMA) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

template <bool BF16, bool GENERAL, bool FOLD>
static int launch(const CUtensorMap &tmap, const CUtensorMap &tmap_r, const void *prepacked, const void *corr_op, int KX, int M,
                  int64_t K, int64_t N, void *y, int64_t ldy, const float *addend, int64_t ld_add, int rows, int act, int sms,
                  cudaStream_t st) {
    {   // opt in to the large dynamic shared memory once per device and instantiation
        static bool attr_done[64] = {};
        static std::mutex attr_mu;
        int dev = 0;
        Q4B_CUDA_TRY(cudaGetDevice(&dev));
        std::lock_guard<std::mutex> attr_lock(attr_mu);
        if (dev < 0 || dev >= 64 || !attr_done[dev]) {
            Q4B_CUDA_TRY(cudaFuncSetAttribute(gemm_wt_kernel<BF16, GENERAL, FOLD>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_DYN));
            if (dev >= 0 && dev < 64) attr_done[dev] = true;
        }
    }
    const int64_t items = ceil_div(tiles_n(N), PANEL_TILES) * ceil_div(M, rows);
    const unsigned grid = (unsigned)(items < sms ? items : sms);
    gemm_wt_kernel<BF16, GENERAL, FOLD><<<grid, THREADS, SMEM_DYN, st>>>(tmap, tmap_r, (const uint8_t *)prepacked, (const uint16_t *)corr_op, KX,
                                                                  M, K, N, (uint16_t *)y, ldy, addend, ld_add, rows, act);
    Q4B_LAUNCH_CHECK();
    return Q4B_OK;
}

}  // namespace gemmwt

int device_sm_count();

// Arguments as checked by the matmul entry points; M >= 1.  corr_op / xr / KX: the folded rank-G term of the
// group-wise format (KX k-tiles; bf16 [N, 64 KX] and [M, 64 KX]), or null / 0.
int gemm_wt_launch(const void *x, int bf16, int M, int64_t ldx, const void *prepacked, int64_t K, int64_t N, const float *addend,
                   int64_t ld_add, void *y, int64_t ldy, int flags, cudaStream_t st, const void *corr_op, const void *xr, int KX) {
    if (M < 1) return Q4B_ERR_SHAPE;
    // Height of a row tile (the MMAs' N, a multiple of 16, at most 256): equal heights rather than full
    // tiles and a remainder (M = 300: two tiles of 160 rows, not 256 + 44).  Lower tiles than the rows
    // need never pay: an MMA of 128 rows takes the tensor pipe 97 cycles against 128 for one of 256
    // (measured), so even a tile count that fills the last wave of items better loses.
    const int sms = device_sm_count();
    const int t = (M + gemmwt::MAX_ROWS - 1) / gemmwt::MAX_ROWS;
    const int rows = ((M + t - 1) / t + 15) / 16 * 16;
    CUtensorMap tmap, tmap_r;
    if (int rc = encode_x_tensor_map(&tmap, x, bf16, M, K, ldx, rows)) return rc;       // 64 k x `rows` rows per copy
    const bool fold = corr_op != nullptr && xr != nullptr && KX > 0;
    if (fold) {
        if (int rc = encode_x_tensor_map(&tmap_r, xr, 1, M, (int64_t)KX * TILE_K, (int64_t)KX * TILE_K, rows)) return rc;
    } else {
        tmap_r = tmap;
    }
    const int act = act_of_flags(flags);
    const bool general = addend != nullptr || act != 0;
#define Q4B_WT_LAUNCH(BF, GEN, FO)                                                                                              \
    gemmwt::launch<BF, GEN, FO>(tmap, tmap_r, prepacked, FO ? corr_op : nullptr, FO ? KX : 0, M, K, N, y, ldy, GEN ? addend : nullptr, \
                                GEN ? ld_add : 0, rows, GEN ? act : 0, sms, st)
    if (bf16) {
        if (general) return fold ? Q4B_WT_LAUNCH(true, true, true) : Q4B_WT_LAUNCH(true, true, false);
        return fold ? Q4B_WT_LAUNCH(true, false, true) : Q4B_WT_LAUNCH(true, false, false);
    }
    if (general) return fold ? Q4B_WT_LAUNCH(false, true, true) : Q4B_WT_LAUNCH(false, true, false);
    return fold ? Q4B_WT_LAUNCH(false, false, true) : Q4B_WT_LAUNCH(false, false, false);
#undef Q4B_WT_LAUNCH
}

// read and clear this file's wait status (host side; the caller has synchronised the stream)
int gemm_wt_wait_status(int *value) {
    int h = 0;
    Q4B_CUDA_TRY(cudaMemcpyFromSymbol(&h, gemmwt::g_status, sizeof(int)));
    if (h != 0) {
        const int zero = 0;
        Q4B_CUDA_TRY(cudaMemcpyToSymbol(gemmwt::g_status, &zero, sizeof(int)));
    }
    *value = h;
    return Q4B_OK;
}

}  // namespace q4b
