// Single-row decode as ONE persistent kernel over a list of stages.
//
// A decode step is a chain of small dependent products (q|k|v -> o -> gate|up -> down -> ...), each
// far too short to hide the cost of a kernel boundary.  Here one CTA per SM stays resident for the
// whole list: a stage is up to four products that share their input row; a later stage may take its
// input from an earlier stage's output.  Nothing of this exists in the reference, whose Metal kernel
// (packages/metalcore/src/metalcore/native/quant_kernels.metal:1738-1886, launched per product by
// core_mps.mm:5917-5975) has no single-row specialisation at all.
//
//  * Weights never depend on activations, so every warp keeps streaming ITS share of the packed
//    tiles of this and the following stages into a private shared-memory ring (cp.async.bulk, one
//    mbarrier per slot) regardless of stage boundaries: HBM stays busy while a stage hands over.
//  * Hand-over between stages is data flow, not a grid barrier: the warp that finishes 16 output
//    columns stores them twice, plainly into y for the caller and as 8-byte (two values, epoch) words
//    into a side buffer; consumers poll those words (the flag travels with the data, so one L2 round
//    trip after the store the value is usable and no fence is needed).  The epoch lives in device
//    memory and is bumped by the last CTA to leave, so a captured launch can be replayed.
//  * Arithmetic: the input row is turned, once per stage and CTA, into 15-bit block-fixed-point
//    (per 32-k block: scale = max|x| / 16383, two signed 8-bit limbs) laid out as the B fragment of
//    mma.sync.m16n8k32.s8; nibbles become the u8 A fragment with two logic ops per register, four
//    blocks share one accumulator (B columns 2j, 2j+1 carry the limbs of block j, zero elsewhere),
//    and the exact integer dot product is scaled by (block scale of x) * (fp16 scale of the weights)
//    in fp32.  The -8 offset comes off exactly as 8 * sum(x_q) per block.  Every sum has a fixed
//    order, so results repeat bit for bit.
//  * Work split: column tiles of a stage are dealt to CTAs as contiguous runs starting at a rotating
//    CTA (so leftovers even out over the chain); inside a CTA two groups of eight warps take
//    alternate tiles and split k eight ways, reduced through shared memory.
//
// Every wait (ring mbarriers, hand-over polls) is bounded.  A wait that gives up records a code,
// raises an abort flag that all other waits observe, and the kernel runs through to its end (results
// are then garbage, which q4b_wait_status reports) after draining its own copies in flight.
#include <climits>
#include <memory>
#include <mutex>

#include "q4b_common.cuh"

namespace q4b {
namespace chain {

constexpr int WARPS = 16;                       // consumer warps: two groups of eight
constexpr int LOADER_WARPS = 4;                 // warps that prepare the next stage's input row
constexpr int THREADS = (WARPS + LOADER_WARPS) * 32;
constexpr int KSPLIT = 8;                       // warps that split k for one column tile
constexpr int PAIR_BYTES = 2 * TILE_BYTES;      // two k tiles = four q4_0 blocks of 16 columns
constexpr long long WAIT_LIMIT_CYCLES = 1LL << 28;
constexpr int MAX_PRODUCTS = Q4B_CHAIN_MAX_PRODUCTS;

__device__ int g_chain_status = 0;

struct Product {
    const uint8_t *w;
    uint16_t *y;
    unsigned long long *ll;     // hand-over words for later stages, or null
    const float *addend;
    int32_t N, nt;
    float alpha;
    int32_t act;
};
struct Stage {
    const uint16_t *x_plain;    // input row in plain memory (ready when the kernel starts), or null
    const unsigned long long *x_ll, *x_ll2;   // or hand-over words of earlier products
    int32_t K, KU, PT;          // k, k tiles, pairs of k tiles per column tile
    int32_t nprod, nt_total, cta_off, xform, pad;
    Product p[MAX_PRODUCTS];
};
struct Ctl {
    unsigned int epoch, exit_count;
    int abort, pad;
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 r;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "r"(a));
    return r;
}
__device__ __forceinline__ uint2 lds64(uint32_t a) {
    uint2 r;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(r.x), "=r"(r.y) : "r"(a));
    return r;
}
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
    uint32_t r;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(r) : "r"(a));
    return r;
}
__device__ __forceinline__ void sts64(uint32_t a, uint32_t x, uint32_t y) {
    asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(a), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// d (+)= A(16 x 32, u8) . B(32 x 8, s8), s32 accumulate
__device__ __forceinline__ void imma_first(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                           uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
__device__ __forceinline__ void imma_acc(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// What the weight producer and the work split need of a stage, copied to shared memory when the
// kernel starts (the full Stage stays in global memory: inputs, outputs, epilogue parameters).
struct alignas(16) Compact {
    int32_t nblk;               // K / 32
    int32_t base, extra, off;   // tiles per worker, workers with one more, first worker (see worker_tiles)
    const uint8_t *w[MAX_PRODUCTS];
    int32_t ntc[MAX_PRODUCTS];  // running sum of the products' column tiles (INT_MAX beyond nprod)
};
static_assert(sizeof(Compact) == 64, "compact stage record");

struct Shared {
    unsigned long long bars[WARPS][8];      // ring slots of the consumer warps
    unsigned long long x_full[2], x_empty[2];
    float red[2][2][KSPLIT][TILE_N];
    int abort;
};

// A worker is one group of eight warps; there are 2 * grid of them, numbered group-major so that a
// stage with fewer tiles than workers still reaches every SM.  Tiles are dealt out as contiguous
// runs starting at worker `off`; the first `extra` runs are one tile longer.
__device__ __forceinline__ void worker_tiles(const Compact &cs, int gi, int &t0, int &n) {
    const int W = 2 * (int)gridDim.x;
    int i = gi * (int)gridDim.x + (int)blockIdx.x - cs.off;
    if (i < 0) i += W;
    n = cs.base + (i < cs.extra ? 1 : 0);
    t0 = i * cs.base + min(i, cs.extra);
}

// four values' low bytes / second bytes gathered into one word
__device__ __forceinline__ uint32_t bytes0(uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    return __byte_perm(__byte_perm(a, b, 0x0040), __byte_perm(c, d, 0x0040), 0x5410);
}
__device__ __forceinline__ uint32_t bytes1(uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    return __byte_perm(__byte_perm(a, b, 0x0051), __byte_perm(c, d, 0x0051), 0x5410);
}

template <int CH, int SLOTS>
__global__ void __launch_bounds__(THREADS, 1)
chain_kernel(const Stage *__restrict__ stages, const Compact *__restrict__ ctab, int n_stages, Ctl *ctl, int bf16,
             int cap_blocks, int nbuf, const __grid_constant__ Stage inline_stage,
             const __grid_constant__ Compact inline_compact) {
    static_assert(SLOTS <= 8 && (SLOTS & (SLOTS - 1)) == 0, "ring slots");
    constexpr int SLOT_BYTES = CH * PAIR_BYTES;
    constexpr int RING_BYTES = WARPS * SLOTS * SLOT_BYTES;
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ Shared sh;

    const int tid = (int)threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // input-row buffers: per buffer [block][limb][k-octet][8 bytes], then [block] (scale, offset term)
    const uint32_t xbuf_bytes = (uint32_t)cap_blocks * 72u;
    const uint32_t xq_base = smem_u32(smem) + RING_BYTES;
    const Compact *tab = reinterpret_cast<const Compact *>(smem + RING_BYTES + (size_t)nbuf * xbuf_bytes);
    auto stage_at = [&](int s) -> const Stage * { return stages != nullptr ? stages + s : &inline_stage; };

    if (tid == 0) {
        sh.abort = 0;
        for (int b = 0; b < 2; ++b) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(&sh.x_full[b])), "r"(LOADER_WARPS) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(&sh.x_empty[b])), "r"(WARPS) : "memory");
        }
    }
    if (warp < WARPS && lane == 0) {
#pragma unroll
        for (int s = 0; s < SLOTS; ++s)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&sh.bars[warp][s])) : "memory");
    }
    if (lane == 0) asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    {
        const uint4 *src = reinterpret_cast<const uint4 *>(ctab != nullptr ? ctab : &inline_compact);
        uint4 *dst = reinterpret_cast<uint4 *>(smem + RING_BYTES + (size_t)nbuf * xbuf_bytes);
        for (int i = tid; i < n_stages * 4; i += THREADS) dst[i] = src[i];
    }
    __syncthreads();

    auto aborted = [&]() -> bool { return *(volatile int *)&sh.abort != 0; };
    auto give_up = [&](int code) {
        *(volatile int *)&sh.abort = 1;
        if (ctl != nullptr) *(volatile int *)&ctl->abort = 1;
        atomicCAS(&g_chain_status, 0, code);
    };
    auto other_cta_aborted = [&]() -> bool { return ctl != nullptr && *(volatile int *)&ctl->abort != 0; };
    // bounded wait on a shared-memory barrier; returns at once when the kernel is aborting
    auto wait_bar = [&](uint32_t bar, uint32_t parity, int code) {
        if (mbar_try(bar, parity) || aborted()) return;
        long long t_start = 0;
        for (int it = 1;; ++it) {
            if (mbar_try(bar, parity)) return;
            if ((it & 63) == 0) {
                if (aborted()) return;
                const long long now = clock64();
                if (t_start == 0) t_start = now;
                else if (now - t_start > WAIT_LIMIT_CYCLES) { give_up(code); return; }
            }
        }
    };
    // does this CTA have any tile in stage s (then its input row is loaded and waited for)
    auto cta_takes_part = [&](const Compact &cs) -> bool {
        int t0, n0, n1;
        worker_tiles(cs, 0, t0, n0);
        worker_tiles(cs, 1, t0, n1);
        return n0 + n1 > 0;
    };

    if (warp >= WARPS) {
        // =====================================================================================
        // loader warps: the stage's input row -> 15-bit block fixed point in shared memory, one
        // 32-element block per lane (no exchange between lanes), one buffer ahead of the consumers
        // =====================================================================================
        const int lw = warp - WARPS;
        asm volatile("griddepcontrol.wait;" ::: "memory");           // inputs may come from earlier kernels
        uint32_t epoch = 0;
        if (ctl != nullptr) asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(epoch) : "l"(&ctl->epoch) : "memory");
        int ns = 0;                                                   // stages this CTA took part in so far
#pragma unroll 1
        for (int s = 0; s < n_stages; ++s) {
            const Compact &cs = tab[s];
            if (!cta_takes_part(cs)) continue;
            const int b = ns % nbuf;
            const uint32_t ph = (uint32_t)(ns / nbuf) & 1u;
            ++ns;
            wait_bar(smem_u32(&sh.x_empty[b]), ph ^ 1u, 504);        // the consumers are done with this buffer
            const Stage *st = stage_at(s);
            const uint16_t *xp = st->x_plain;
            const unsigned long long *lla = st->x_ll, *llb = st->x_ll2;
            const int xform = st->xform;
            const int nblk = cs.nblk, nblk_pad = (((nblk + 1) >> 1) + 1) / 2 * 4;
            const uint32_t xq_s = xq_base + (uint32_t)b * xbuf_bytes, xs_s = xq_s + (uint32_t)cap_blocks * 64u;
#pragma unroll 1
            for (int base = lw * 32; base < nblk_pad; base += LOADER_WARPS * 32) {     // warp-uniform trip count
                const int blk = base + lane;
                uint32_t w[16];                                      // 32 fp16 / bf16 values, two per word
                uint32_t w2[16];
                if (xp != nullptr || blk >= nblk) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) w[i] = 0u;
                    if (blk < nblk) {
                        const uint4 *src = reinterpret_cast<const uint4 *>(xp + (size_t)blk * QK);
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const uint4 v = __ldcg(src + i);
                            w[4 * i] = v.x; w[4 * i + 1] = v.y; w[4 * i + 2] = v.z; w[4 * i + 3] = v.w;
                        }
                    }
                }
                if (xp == nullptr) {
                    // Hand-over words (two values, epoch) of an earlier stage.  A block's 32 values come
                    // from two column tiles, written by two warps.  While waiting, every lane looks only at
                    // the two words where they meet (the last of one, the first of the other): polling all
                    // sixteen from every SM saturates L2 and slows the very stores it waits for.  Once all
                    // lanes of the warp see this launch's epoch there, the sixteen words are read and every
                    // flag is checked.  The warp stays converged, so the conversion below runs once.
                    const bool mine = blk < nblk;
                    const unsigned long long *ba = lla + (size_t)blk * 16, *bb = llb + (size_t)blk * 16;
                    long long t_start = 0;
                    for (int it = 0;; ++it) {
                        uint32_t ok = 1u, f0, f1, t0, t1;
                        if (mine) {
                            asm volatile("ld.volatile.global.v2.u32 {%0,%1}, [%2];" : "=r"(t0), "=r"(f0) : "l"(ba + 7) : "memory");
                            asm volatile("ld.volatile.global.v2.u32 {%0,%1}, [%2];" : "=r"(t1), "=r"(f1) : "l"(ba + 8) : "memory");
                            ok = (f0 == epoch && f1 == epoch) ? 1u : 0u;
                            if (xform == 1) {
                                asm volatile("ld.volatile.global.v2.u32 {%0,%1}, [%2];" : "=r"(t0), "=r"(f0) : "l"(bb + 7) : "memory");
                                asm volatile("ld.volatile.global.v2.u32 {%0,%1}, [%2];" : "=r"(t1), "=r"(f1) : "l"(bb + 8) : "memory");
                                ok &= (f0 == epoch && f1 == epoch) ? 1u : 0u;
                            }
                        }
                        if (__all_sync(0xffffffffu, ok != 0u)) {
                            if (mine) {
#pragma unroll
                                for (int i = 0; i < 8; ++i) {
                                    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                                                 : "=r"(w[2 * i]), "=r"(f0), "=r"(w[2 * i + 1]), "=r"(f1) : "l"(ba + 2 * i) : "memory");
                                    ok &= (f0 == epoch && f1 == epoch) ? 1u : 0u;
                                }
                                if (xform == 1) {
#pragma unroll
                                    for (int i = 0; i < 8; ++i) {
                                        asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                                                     : "=r"(w2[2 * i]), "=r"(f0), "=r"(w2[2 * i + 1]), "=r"(f1) : "l"(bb + 2 * i) : "memory");
                                        ok &= (f0 == epoch && f1 == epoch) ? 1u : 0u;
                                    }
                                }
                            }
                            if (__all_sync(0xffffffffu, ok != 0u)) break;
                        }
                        __nanosleep(150);
                        bool stop = false;
                        if ((it & 15) == 15) {
                            if (aborted() || other_cta_aborted()) { *(volatile int *)&sh.abort = 1; stop = true; }
                            const long long now = clock64();
                            if (t_start == 0) t_start = now;
                            else if (now - t_start > WAIT_LIMIT_CYCLES) { give_up(501); stop = true; }
                        }
                        if (__any_sync(0xffffffffu, stop)) break;
                    }
                }
                float f[32];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    float2 v;
                    if (bf16) v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&w[i]));
                    else v = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
                    f[2 * i] = v.x;
                    f[2 * i + 1] = v.y;
                }
                if (xform == 1 && blk < nblk) {                       // x = silu(a) * b
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        float2 v;
                        if (bf16) v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&w2[i]));
                        else v = __half22float2(*reinterpret_cast<const __half2 *>(&w2[i]));
                        f[2 * i] = f[2 * i] / (1.0f + __expf(-f[2 * i])) * v.x;
                        f[2 * i + 1] = f[2 * i + 1] / (1.0f + __expf(-f[2 * i + 1])) * v.y;
                    }
                }
                float amax = 0.0f;
#pragma unroll
                for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(f[i]));
                // |x| * inv stays below 16381: the high limb fits a signed byte whatever the rounding of inv
                const float inv = amax > 0.0f ? __fdividef(16380.0f, amax) : 0.0f;
                const float scale = amax * (1.0f / 16380.0f);
                uint32_t v[32];                                       // 2 * x_q: byte 1 = high limb, byte 0 = 2 * low limb
                int sum = 0;
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int xi = __float2int_rn(f[i] * inv);
                    sum += xi;
                    v[i] = (uint32_t)xi << 1;
                }
                // fragment byte order per k-octet c: (k0, k4, k1, k5) then (k2, k6, k3, k7)
                uint32_t lo[8], hi[8];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const uint32_t *e = &v[8 * c];
                    lo[2 * c] = (bytes0(e[0], e[4], e[1], e[5]) >> 1) & 0x7F7F7F7Fu;
                    lo[2 * c + 1] = (bytes0(e[2], e[6], e[3], e[7]) >> 1) & 0x7F7F7F7Fu;
                    hi[2 * c] = bytes1(e[0], e[4], e[1], e[5]);
                    hi[2 * c + 1] = bytes1(e[2], e[6], e[3], e[7]);
                }
                if (blk >= nblk_pad) continue;
                const uint32_t dst = xq_s + (uint32_t)blk * 64u;
                asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst), "r"(lo[0]), "r"(lo[1]), "r"(lo[2]), "r"(lo[3]) : "memory");
                asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst + 16), "r"(lo[4]), "r"(lo[5]), "r"(lo[6]), "r"(lo[7]) : "memory");
                asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst + 32), "r"(hi[0]), "r"(hi[1]), "r"(hi[2]), "r"(hi[3]) : "memory");
                asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst + 48), "r"(hi[4]), "r"(hi[5]), "r"(hi[6]), "r"(hi[7]) : "memory");
                sts64(xs_s + (uint32_t)blk * 8u, __float_as_uint(scale), __float_as_uint(-8.0f * (float)sum * scale));
            }
            __syncwarp();
            if (lane == 0) asm volatile("{ .reg .b64 t; mbarrier.arrive.shared::cta.b64 t, [%0]; }" ::"r"(smem_u32(&sh.x_full[b])) : "memory");
        }
    } else {
        // =====================================================================================
        // consumer warps
        // =====================================================================================
        const int g = lane >> 2, c = lane & 3;
        const int gi = warp >> 3, w8 = warp & 7;
        const uint32_t ring_s = smem_u32(smem) + (uint32_t)(warp * SLOTS * SLOT_BYTES);
        const uint32_t bar_s = smem_u32(&sh.bars[warp][0]);

        // ---- producer: walks this warp's share of the weights, stage after stage.  Every lane keeps
        // the (identical) state; only lane 0's copy instructions are enabled. ----
        int ps = -1, pt = -1, prun_end = 0, pprod_end = 0, pkp = 0, pkp0 = 0, pkp1 = 0, pKU = 0;
        const uint8_t *psrc = nullptr, *ptile_src = nullptr;
        size_t ptile_stride = 0;
        uint32_t pc = 0;                     // chunks issued
        bool pdone = false;
        // moves to the next tile in which this warp has a share; false when the list is exhausted
        auto next_tile = [&]() -> bool {
            for (;;) {
                ++pt;
                if (pt < prun_end && pt < pprod_end) {
                    ptile_src += ptile_stride;           // next column tile of the same product
                } else {
                    while (pt >= prun_end) {
                        if (++ps >= n_stages) return false;
                        int t0, n;
                        worker_tiles(tab[ps], gi, t0, n);
                        pt = t0;
                        prun_end = t0 + n;
                        pKU = (tab[ps].nblk + 1) >> 1;
                        const int PT = (pKU + 1) >> 1;
                        pkp0 = w8 * PT / KSPLIT;
                        pkp1 = (w8 + 1) * PT / KSPLIT;
                        ptile_stride = (size_t)pKU * TILE_BYTES;
                    }
                    const Compact &cs = tab[ps];
                    const int p = (pt >= cs.ntc[0]) + (pt >= cs.ntc[1]) + (pt >= cs.ntc[2]);
                    pprod_end = cs.ntc[p];
                    ptile_src = cs.w[p] + tile_offset(pt - (p > 0 ? cs.ntc[p - 1] : 0), 2 * pkp0, pKU);
                }
                if (pkp0 < pkp1) break;                  // else: fewer tile pairs than warps, no share here
            }
            pkp = pkp0;
            psrc = ptile_src;
            return true;
        };
        // issues the next chunk into slot pc % SLOTS
        auto produce_one = [&]() {
            if (pdone) return;
            if (pkp >= pkp1 && !next_tile()) { pdone = true; return; }
            const int np = min(CH, pkp1 - pkp);
            const uint32_t bytes = (uint32_t)(min(2 * (pkp + np), pKU) - 2 * pkp) * TILE_BYTES;
            const uint32_t slot = pc & (SLOTS - 1);
            const uint32_t bar = bar_s + 8u * slot;
            asm volatile(
                "{\n\t.reg .pred p;\n\t.reg .b64 t;\n\t"
                "setp.eq.u32 p, %0, 0;\n\t"
                "@p mbarrier.arrive.expect_tx.shared::cta.b64 t, [%1], %2;\n\t"
                "@p cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%3], [%4], %2, [%1];\n\t"
                "}" ::"r"((uint32_t)lane), "r"(bar), "r"(bytes), "r"(ring_s + slot * SLOT_BYTES), "l"(psrc) : "memory");
            psrc += bytes;
            pkp += np;
            ++pc;
        };
        // Weights never depend on earlier kernels of the stream, so the ring fills before the wait
        // for them; outputs are written after it.
#pragma unroll 1
        for (int s = 0; s < SLOTS; ++s) produce_one();
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
        asm volatile("griddepcontrol.wait;" ::: "memory");
        uint32_t epoch = 0;
        if (ctl != nullptr) asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(epoch) : "l"(&ctl->epoch) : "memory");

        // per-lane constants
        const uint32_t qoff = (uint32_t)slot_of(g, c) * 16u;
        const uint32_t doff = (uint32_t)((c >> 1) * TILE_BYTES + TILE_QS_BYTES + g * 8 + (c & 1) * 4);
        const uint32_t xoff = (uint32_t)((g >> 1) * 64 + (g & 1) * 32 + c * 8);
        const uint32_t m0 = (g >> 1) == 0 ? 0xFFFFFFFFu : 0u, m1 = (g >> 1) == 1 ? 0xFFFFFFFFu : 0u;
        const uint32_t m2 = (g >> 1) == 2 ? 0xFFFFFFFFu : 0u, m3 = (g >> 1) == 3 ? 0xFFFFFFFFu : 0u;
        constexpr uint32_t NIB = 0x0F0F0F0Fu;

        uint32_t cc = 0;                     // chunks consumed
        int redbuf = 0, tcount = 0, ns = 0;

#pragma unroll 1
        for (int s = 0; s < n_stages; ++s) {
            const Compact &cs = tab[s];
            if (!cta_takes_part(cs)) continue;                        // the whole CTA skips (uniform)
            const int b = ns % nbuf;
            const uint32_t ph = (uint32_t)(ns / nbuf) & 1u;
            ++ns;
            const Stage *st = stage_at(s);
            const int nblk = cs.nblk, KU = (nblk + 1) >> 1, PT = (KU + 1) >> 1;
            int t0, ntile;
            worker_tiles(cs, gi, t0, ntile);
            const uint32_t xq_s = xq_base + (uint32_t)b * xbuf_bytes, xs_s = xq_s + (uint32_t)cap_blocks * 64u;
            wait_bar(smem_u32(&sh.x_full[b]), ph, 503);               // the loaders have written this stage's input row
            __syncwarp();

            const int kp0 = w8 * PT / KSPLIT, kp1 = (w8 + 1) * PT / KSPLIT;
#pragma unroll 1
            for (int t = t0; t < t0 + ntile; ++t) {
                float acc0 = 0.0f, acc1 = 0.0f;
#pragma unroll 1
                for (int kp = kp0; kp < kp1; kp += CH) {
                    const int np = min(CH, kp1 - kp);
                    const uint32_t slot = cc & (SLOTS - 1), parity = (cc / SLOTS) & 1u;
                    wait_bar(bar_s + 8u * slot, parity, 500);
                    __syncwarp();
                    const uint32_t sl = ring_s + slot * SLOT_BYTES;
                    const uint32_t xq_a = xq_s + (uint32_t)kp * 256u + xoff, xs_a = xs_s + (uint32_t)kp * 32u + (uint32_t)c * 8u;
                    const int tiles_left = KU - 2 * kp;
#pragma unroll
                    for (int i = 0; i < CH; ++i) {
                        if (i < np) {
                            const uint4 qa = lds128(sl + i * PAIR_BYTES + qoff);
                            const uint4 qb = lds128(sl + i * PAIR_BYTES + TILE_BYTES + qoff);
                            const uint2 own = lds64(xq_a + i * 256);
                            const uint2 sc = lds64(xs_a + i * 32);
                            const uint32_t dd = lds32(sl + i * PAIR_BYTES + doff);
                            int D[4];
                            imma_first(D, qa.x & NIB, qa.y & NIB, (qa.x >> 4) & NIB, (qa.y >> 4) & NIB, own.x & m0, own.y & m0);
                            imma_acc(D, qa.z & NIB, qa.w & NIB, (qa.z >> 4) & NIB, (qa.w >> 4) & NIB, own.x & m1, own.y & m1);
                            imma_acc(D, qb.x & NIB, qb.y & NIB, (qb.x >> 4) & NIB, (qb.y >> 4) & NIB, own.x & m2, own.y & m2);
                            imma_acc(D, qb.z & NIB, qb.w & NIB, (qb.z >> 4) & NIB, (qb.w >> 4) & NIB, own.x & m3, own.y & m3);
                            // D[0], D[1]: column g, low and high limb sums of block c; D[2], D[3]: column g + 8
                            const float xs = __uint_as_float(sc.x), xt = __uint_as_float(sc.y);
                            const float f0 = fmaf((float)(D[0] + (D[1] << 7)), xs, xt);
                            const float f1 = fmaf((float)(D[2] + (D[3] << 7)), xs, xt);
                            const float2 d2 = __half22float2(*reinterpret_cast<const __half2 *>(&dd));
                            const bool valid = 2 * i + (c >> 1) < tiles_left;     // the pair's second tile may not exist
                            acc0 = valid ? fmaf(d2.x, f0, acc0) : acc0;
                            acc1 = valid ? fmaf(d2.y, f1, acc1) : acc1;
                        }
                    }
                    __syncwarp();                                             // every lane has read the slot
                    ++cc;
                    if (!aborted()) produce_one();
                }
                // lanes of a quad hold different blocks of columns g and g + 8
                acc0 += __shfl_xor_sync(0xffffffffu, acc0, 1);
                acc1 += __shfl_xor_sync(0xffffffffu, acc1, 1);
                acc0 += __shfl_xor_sync(0xffffffffu, acc0, 2);
                acc1 += __shfl_xor_sync(0xffffffffu, acc1, 2);
                if (c == 0) {
                    sh.red[gi][redbuf][w8][g] = acc0;
                    sh.red[gi][redbuf][w8][g + 8] = acc1;
                }
                asm volatile("bar.sync %0, %1;" ::"r"(1 + gi), "r"(KSPLIT * 32) : "memory");
                if (w8 == (tcount & 7)) {                                      // the tiles' epilogues rotate over the warps
                    const int p = (t >= cs.ntc[0]) + (t >= cs.ntc[1]) + (t >= cs.ntc[2]);
                    const int nt = t - (p > 0 ? cs.ntc[p - 1] : 0);
                    const Product *pr = &st->p[p];
                    const int col = lane & 15, n = nt * TILE_N + col, N = pr->N;
                    float v = 0.0f;
#pragma unroll
                    for (int j = 0; j < KSPLIT; ++j) v += sh.red[gi][redbuf][j][col];
                    v *= pr->alpha;
                    if (pr->addend != nullptr && n < N) v += __ldg(pr->addend + n);
                    v = apply_act(v, pr->act);
                    const uint32_t bits = bf16 ? (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(v))
                                               : (uint32_t)__half_as_ushort(__float2half_rn(v));
                    const uint32_t nb = __shfl_down_sync(0xffffffffu, bits, 1);
                    if (lane < 16 && n < N) {
                        pr->y[n] = (uint16_t)bits;
                        if (pr->ll != nullptr && (col & 1) == 0) {
                            const uint32_t word = bits | ((n + 1 < N ? nb : 0u) << 16);
                            asm volatile("st.volatile.global.v2.u32 [%0], {%1,%2};" ::"l"(pr->ll + (n >> 1)), "r"(word), "r"(epoch) : "memory");
                        }
                    }
                }
                redbuf ^= 1;
                ++tcount;
            }
            __syncwarp();
            if (lane == 0) asm volatile("{ .reg .b64 t; mbarrier.arrive.shared::cta.b64 t, [%0]; }" ::"r"(smem_u32(&sh.x_empty[b])) : "memory");
        }

        // Copies still in flight must land before the CTA's shared memory goes away: wait for the last
        // chunk issued into every slot (a phase that was already consumed answers at once).
        if (lane == 0) {
            for (uint32_t back = 1; back <= (uint32_t)SLOTS && back <= pc; ++back) {
                const uint32_t j = pc - back, slot = j & (SLOTS - 1), parity = (j / SLOTS) & 1u;
                const long long t_start = clock64();
                while (!mbar_try(bar_s + 8u * slot, parity))
                    if (clock64() - t_start > WAIT_LIMIT_CYCLES) { atomicCAS(&g_chain_status, 0, 502); break; }
            }
        }
    }
    __syncthreads();
    if (ctl != nullptr && tid == 0) {
        __threadfence();
        const unsigned int old = atomicAdd(&ctl->exit_count, 1u);
        if (old == gridDim.x - 1) {                                            // last CTA out: next launch, next epoch
            ctl->exit_count = 0;
            ctl->abort = 0;
            __threadfence();
            atomicAdd(&ctl->epoch, 1u);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
constexpr int CH = 4, SLOTS = 2;
constexpr int RING_BYTES = WARPS * SLOTS * CH * PAIR_BYTES;
constexpr int MAX_DYN_SMEM = 227 * 1024 - 4096;           // what is left beside the static part
constexpr size_t ALIGN = 256;
inline size_t round_up(size_t v) { return (v + ALIGN - 1) & ~(ALIGN - 1); }

static int prepare_device(int *sms_out) {
    static std::mutex mu;
    static bool done[64] = {};
    static int sms[64] = {};
    int dev = 0;
    Q4B_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return Q4B_ERR_ARG;
    std::lock_guard<std::mutex> lk(mu);
    if (!done[dev]) {
        Q4B_CUDA_TRY(cudaFuncSetAttribute(chain_kernel<CH, SLOTS>, cudaFuncAttributeMaxDynamicSharedMemorySize, MAX_DYN_SMEM));
        Q4B_CUDA_TRY(cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev));
        done[dev] = true;
    }
    *sms_out = sms[dev];
    return Q4B_OK;
}

// blocks of the fixed-point input row a stage needs room for (padded to whole tile pairs)
static int64_t stage_blocks(int64_t K) { return ceil_div(tiles_k(K), 2) * 4; }
// dynamic shared memory of a launch: rings, nbuf input-row buffers (72 bytes per block), the stage table
static int64_t smem_bytes(int64_t max_k, int n_stages, int nbuf) {
    return RING_BYTES + nbuf * stage_blocks(max_k) * 72 + (int64_t)n_stages * (int64_t)sizeof(Compact);
}
// two input-row buffers (the loaders work one stage ahead) when they fit, else one; 0: too large
static int input_buffers(int64_t max_k, int n_stages) {
    if (n_stages > 1 && smem_bytes(max_k, n_stages, 2) <= MAX_DYN_SMEM) return 2;
    return smem_bytes(max_k, n_stages, 1) <= MAX_DYN_SMEM ? 1 : 0;
}

static int check_stage(const q4b_chain_stage &s, int index) {
    if (s.K <= 0 || s.n_products < 1 || s.n_products > MAX_PRODUCTS) return Q4B_ERR_ARG;
    if (s.K % QK || tiles_k(s.K) > (1 << 20)) return Q4B_ERR_SHAPE;
    if (s.xform != Q4B_CHAIN_X_PLAIN && s.xform != Q4B_CHAIN_X_SILU_MUL) return Q4B_ERR_ARG;
    if (s.x != nullptr) {
        if (s.xform != Q4B_CHAIN_X_PLAIN) return Q4B_ERR_ARG;
        if (!aligned(s.x, 16)) return Q4B_ERR_ALIGN;
    } else {
        if (s.x_stage < 0 || s.x_stage >= index || s.x_product < 0) return Q4B_ERR_ARG;
        if (s.xform == Q4B_CHAIN_X_SILU_MUL && (s.x_stage2 < 0 || s.x_stage2 >= index || s.x_product2 < 0)) return Q4B_ERR_ARG;
    }
    int64_t nt = 0;
    for (int p = 0; p < s.n_products; ++p) {
        const q4b_chain_product &pr = s.products[p];
        if (pr.prepacked == nullptr || pr.y == nullptr || pr.N <= 0) return Q4B_ERR_ARG;
        if (!aligned(pr.prepacked, 16) || !aligned(pr.y, 2)) return Q4B_ERR_ALIGN;
        if (act_of_flags(pr.flags) == 3) return Q4B_ERR_ARG;
        nt += tiles_n(pr.N);
    }
    if (nt > (1 << 24)) return Q4B_ERR_SHAPE;
    return Q4B_OK;
}

// fills the device-side records of one stage; `off` is the worker the stage's first run goes to
static void fill_stage(const q4b_chain_stage &s, int off, int workers, Stage &d, Compact &cs) {
    d = Stage{};
    cs = Compact{};
    d.x_plain = (const uint16_t *)s.x;
    d.K = (int32_t)s.K;
    d.KU = (int32_t)tiles_k(s.K);
    d.PT = (int32_t)ceil_div(d.KU, 2);
    d.nprod = s.n_products;
    d.cta_off = off;
    d.xform = s.xform;
    int nt_total = 0;
    for (int p = 0; p < MAX_PRODUCTS; ++p) {
        cs.ntc[p] = INT32_MAX;
        if (p >= s.n_products) continue;
        const q4b_chain_product &pr = s.products[p];
        Product &q = d.p[p];
        q.w = (const uint8_t *)pr.prepacked;
        q.y = (uint16_t *)pr.y;
        q.ll = nullptr;
        q.addend = pr.addend;
        q.N = (int32_t)pr.N;
        q.nt = (int32_t)tiles_n(pr.N);
        q.alpha = pr.alpha;
        q.act = act_of_flags(pr.flags);
        nt_total += q.nt;
        cs.w[p] = q.w;
        cs.ntc[p] = nt_total;
    }
    d.nt_total = nt_total;
    cs.nblk = (int32_t)(s.K / QK);
    cs.base = nt_total / workers;
    cs.extra = nt_total % workers;
    cs.off = off;
}

static int launch(const Stage *stages_dev, const Compact *ctab_dev, int n_stages, Ctl *ctl, int bf16, int64_t max_k,
                  const Stage &inline_stage, const Compact &inline_compact, bool cooperative, bool pdl, cudaStream_t st) {
    int sms = 0;
    if (int rc = prepare_device(&sms)) return rc;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)sms);
    cfg.blockDim = dim3(THREADS);
    const int nbuf = input_buffers(max_k, n_stages);
    if (nbuf == 0) return Q4B_ERR_TOO_LARGE;
    cfg.dynamicSmemBytes = (size_t)smem_bytes(max_k, n_stages, nbuf);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    int na = 0;
    if (cooperative) {
        attr[na].id = cudaLaunchAttributeCooperative;
        attr[na].val.cooperative = 1;
        ++na;
    } else if (pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    Q4B_CUDA_TRY(cudaLaunchKernelEx(&cfg, chain_kernel<CH, SLOTS>, stages_dev, ctab_dev, n_stages, ctl, bf16,
                                    (int)stage_blocks(max_k), nbuf, inline_stage, inline_compact));
    return Q4B_OK;
}

int wait_status(int *value) {
    int h = 0;
    Q4B_CUDA_TRY(cudaMemcpyFromSymbol(&h, g_chain_status, sizeof(int)));
    if (h != 0) {
        const int zero = 0;
        Q4B_CUDA_TRY(cudaMemcpyToSymbol(g_chain_status, &zero, sizeof(int)));
    }
    *value = h;
    return Q4B_OK;
}

// workspace layout: [Ctl | Stage x n | Compact x n | hand-over buffers of the products]
struct Layout {
    size_t stages_off, compact_off, ll_off;
};
static Layout layout_of(int n) {
    Layout l;
    l.stages_off = round_up(sizeof(Ctl));
    l.compact_off = l.stages_off + round_up((size_t)n * sizeof(Stage));
    l.ll_off = l.compact_off + round_up((size_t)n * sizeof(Compact));
    return l;
}
static size_t ll_bytes(int64_t N) { return round_up((size_t)ceil_div(N, 2) * 8); }

}  // namespace chain
}  // namespace q4b

using namespace q4b;
using namespace q4b::chain;

extern "C" int q4b_gemv_grouped(const void *x, int x_dtype, int64_t K, const q4b_chain_product *products, int n_products,
                                int flags, void *stream) {
    if (x == nullptr || products == nullptr || n_products < 1 || n_products > MAX_PRODUCTS) return Q4B_ERR_ARG;
    if (x_dtype != Q4B_F16 && x_dtype != Q4B_BF16) return Q4B_ERR_DTYPE;
    q4b_chain_stage s = {};
    s.x = x;
    s.K = K;
    s.n_products = n_products;
    for (int p = 0; p < n_products; ++p) s.products[p] = products[p];
    if (int rc = check_stage(s, 0)) return rc;
    if (input_buffers(K, 1) == 0) return Q4B_ERR_TOO_LARGE;
    int sms = 0;
    if (int rc = prepare_device(&sms)) return rc;
    Stage d;
    Compact cs;
    fill_stage(s, 0, 2 * sms, d, cs);
    return launch(nullptr, nullptr, 1, nullptr, x_dtype == Q4B_BF16, K, d, cs, false, (flags & Q4B_FLAG_PDL) != 0,
                  (cudaStream_t)stream);
}

extern "C" size_t q4b_chain_workspace_bytes(const q4b_chain_stage *stages, int n_stages) {
    if (stages == nullptr || n_stages < 1 || n_stages > Q4B_CHAIN_MAX_STAGES) return 0;
    size_t total = layout_of(n_stages).ll_off;
    for (int s = 0; s < n_stages; ++s)
        for (int p = 0; p < stages[s].n_products && p < MAX_PRODUCTS; ++p) total += ll_bytes(stages[s].products[p].N);
    return total;
}

extern "C" int q4b_chain_build(const q4b_chain_stage *stages, int n_stages, void *workspace, size_t workspace_bytes,
                               void *stream) {
    if (stages == nullptr || n_stages < 1 || workspace == nullptr) return Q4B_ERR_ARG;
    if (n_stages > Q4B_CHAIN_MAX_STAGES) return Q4B_ERR_TOO_LARGE;
    if (!aligned(workspace, ALIGN)) return Q4B_ERR_ALIGN;
    if (workspace_bytes < q4b_chain_workspace_bytes(stages, n_stages)) return Q4B_ERR_TOO_LARGE;
    int sms = 0;
    if (int rc = prepare_device(&sms)) return rc;
    const int workers = 2 * sms;
    const Layout l = layout_of(n_stages);
    uint8_t *base = (uint8_t *)workspace;
    std::unique_ptr<Stage[]> dev(new Stage[n_stages]);
    std::unique_ptr<Compact[]> ctab(new Compact[n_stages]);
    std::unique_ptr<size_t[]> ll_off(new size_t[(size_t)n_stages * MAX_PRODUCTS]());
    size_t next = l.ll_off;
    int64_t max_k = 0;
    for (int s = 0; s < n_stages; ++s) {
        if (int rc = check_stage(stages[s], s)) return rc;
        max_k = stages[s].K > max_k ? stages[s].K : max_k;
        for (int p = 0; p < stages[s].n_products; ++p) {
            ll_off[(size_t)s * MAX_PRODUCTS + p] = next;
            next += ll_bytes(stages[s].products[p].N);
        }
    }
    if (input_buffers(max_k, n_stages) == 0) return Q4B_ERR_TOO_LARGE;
    int off = 0;
    for (int s = 0; s < n_stages; ++s) {
        fill_stage(stages[s], off, workers, dev[s], ctab[s]);
        off = (off + ctab[s].extra) % workers;            // the next stage's runs start where this one's longer runs ended
        if (stages[s].x == nullptr) {
            const q4b_chain_stage &src = stages[stages[s].x_stage];
            if (stages[s].x_product >= src.n_products || src.products[stages[s].x_product].N != stages[s].K) return Q4B_ERR_SHAPE;
            dev[s].x_ll = (const unsigned long long *)(base + ll_off[(size_t)stages[s].x_stage * MAX_PRODUCTS + stages[s].x_product]);
            dev[stages[s].x_stage].p[stages[s].x_product].ll = (unsigned long long *)dev[s].x_ll;
            if (stages[s].xform == Q4B_CHAIN_X_SILU_MUL) {
                const q4b_chain_stage &src2 = stages[stages[s].x_stage2];
                if (stages[s].x_product2 >= src2.n_products || src2.products[stages[s].x_product2].N != stages[s].K) return Q4B_ERR_SHAPE;
                dev[s].x_ll2 = (const unsigned long long *)(base + ll_off[(size_t)stages[s].x_stage2 * MAX_PRODUCTS + stages[s].x_product2]);
                dev[stages[s].x_stage2].p[stages[s].x_product2].ll = (unsigned long long *)dev[s].x_ll2;
            }
        }
    }
    cudaStream_t st = (cudaStream_t)stream;
    // hand-over words start with flag 0, the epoch with 1: nothing is valid before it is written
    Q4B_CUDA_TRY(cudaMemsetAsync(base, 0, next, st));
    Ctl ctl = {};
    ctl.epoch = 1u;
    Q4B_CUDA_TRY(cudaMemcpyAsync(base, &ctl, sizeof(ctl), cudaMemcpyHostToDevice, st));
    Q4B_CUDA_TRY(cudaMemcpyAsync(base + l.stages_off, dev.get(), (size_t)n_stages * sizeof(Stage), cudaMemcpyHostToDevice, st));
    Q4B_CUDA_TRY(cudaMemcpyAsync(base + l.compact_off, ctab.get(), (size_t)n_stages * sizeof(Compact), cudaMemcpyHostToDevice, st));
    // the copies above read host memory that goes away when this call returns
    Q4B_CUDA_TRY(cudaStreamSynchronize(st));
    return Q4B_OK;
}

extern "C" int q4b_chain_run(const void *workspace, int n_stages, int x_dtype, int64_t max_k, int flags, void *stream) {
    (void)flags;
    if (workspace == nullptr || n_stages < 1 || max_k <= 0) return Q4B_ERR_ARG;
    if (n_stages > Q4B_CHAIN_MAX_STAGES) return Q4B_ERR_TOO_LARGE;
    if (x_dtype != Q4B_F16 && x_dtype != Q4B_BF16) return Q4B_ERR_DTYPE;
    if (max_k % QK) return Q4B_ERR_SHAPE;
    if (input_buffers(max_k, n_stages) == 0) return Q4B_ERR_TOO_LARGE;
    const Layout l = layout_of(n_stages);
    uint8_t *base = (uint8_t *)workspace;
    const Stage none = {};
    const Compact none_c = {};
    return launch((const Stage *)(base + l.stages_off), (const Compact *)(base + l.compact_off), n_stages, (Ctl *)base,
                  x_dtype == Q4B_BF16, max_k, none, none_c, true, false, (cudaStream_t)stream);
}

