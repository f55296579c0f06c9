// Decode path: Y[M, N] = X[M, K] . dequant(W) for 1 <= M <= 16, HBM-bound.
//
// Takes the role the reference gives to its 64x32-tile Metal kernel at small M
// (packages/metalcore/src/metalcore/native/quant_kernels.metal:1738-1886, launched by
// core_mps.mm:5917-5975), which has no GEMV specialisation.
//
// Each warp owns one 16-column tile and a contiguous range of its k tiles, which is one
// contiguous run of bytes in the column-tile-major prepacked layout.  The warp keeps a private
// ring in shared memory fed by bulk asynchronous copies (cp.async.bulk, completion counted on
// one mbarrier per ring slot): a slot holds CHUNK weight tiles plus the matching k-slice of the
// activation rows, so both arrive ahead of use and the bytes in flight per SM are set by the
// ring size, not by registers.  Lanes read 16 bytes of nibbles, 8 bytes of scales and 16 bytes
// of x per 32-k block from the slot (all conflict free), turn the nibbles into (q-8)
// fp16/bf16 pairs in registers, and feed them as the 16-row A operand of mma.sync.m16n8k16;
// up to 8 activation rows are the B operand, so M = 1..8 costs the same and M = 9..16 one more
// fragment.  The per-block scale multiplies the fp32 partial product of each 32-k block;
// accumulation is fp32 throughout.  Warps of a CTA that share a column tile split k and are
// reduced through shared memory.
//
// Every mbarrier wait is bounded: a wait that gives up sets g_wait_status and the warp stops
// consuming (its outputs are then wrong, which the status reports) instead of spinning.
#include <mutex>

#include "q4b_common.cuh"

namespace q4b {

constexpr int GEMV_WARPS = 8;
constexpr int GEMV_THREADS = GEMV_WARPS * 32;
constexpr int GEMV_SPIN_LIMIT = 1 << 22;            // try_wait polls before giving up (~0.1 s)

__device__ int g_wait_status = 0;                  // first bounded wait of this file that gave up

// Optional fused all-gather: when `world` > 0 the epilogue stores the result, instead of into y, at
// column offset col0 of the [M, ld]-shaped output of EVERY rank (peer-mapped pointers; plain
// stores over NVLink), so the column-parallel shards land gathered without a collective.
// Optional rank-G term of the group-wise INT4 format: when corr is not null the epilogue adds
// sum_g corr[g, n] * rowsums[m, g] (fp32; corr [G, N], rowsums [M, G]) before the one rounding, so that
// no [M, N] addend has to exist.
struct PeerOut {
    uint16_t *p[8];
    int world;
    int64_t col0, ld;
    const float *corr, *rowsums;
    int G;
    // ll_tag != 0: the peers' buffers hold 32-bit words and each store is (value | ll_tag), the tag being
    // the call's epoch in the upper half: a word validates itself, so the reader needs no barrier.
    uint32_t ll_tag;
    // ll_ctl != null: the call counter lives in device memory (so a captured launch can be replayed): call c
    // uses epoch c % 65535 + 1 and the buffer of parity c & 1, which starts ll_half words after p[r].
    const int *ll_ctl;
    int64_t ll_half;
};

// (tag, word offset of this call's buffer) of a self-validating store
__device__ __forceinline__ void ll_call(const PeerOut &peers, uint32_t &tag, int64_t &base) {
    tag = peers.ll_tag;
    base = 0;
    if (peers.ll_ctl != nullptr) {
        const int c = *reinterpret_cast<const volatile int *>(peers.ll_ctl);
        tag = (uint32_t)(c % 65535 + 1) << 16;
        base = (c & 1) ? peers.ll_half : 0;
    }
}


// Shared-memory geometry of one ring slot: CHUNK weight tiles, then the x rows.  The row
// stride is 64 bytes more than a multiple of 128 so that the eight (row, k-octet) pairs a
// quarter warp reads fall into eight different 16-byte bank groups.
template <int CHUNK> struct SlotGeom {
    static constexpr int W_BYTES = CHUNK * TILE_BYTES;
    static constexpr int X_ROW = CHUNK * TILE_K * 2;          // bytes of one activation row slice
    static constexpr int X_STRIDE = X_ROW + 64;
    static __host__ __device__ constexpr int slot_bytes(int m) { return W_BYTES + m * X_STRIDE; }
};

__device__ __forceinline__ uint32_t smem_addr_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("{ .reg .b64 t; mbarrier.arrive.expect_tx.shared::cta.b64 t, [%0], %1; }" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// On the lanes where `pred` holds: arm `bar` with the bytes of both copies and start them (weights,
// then the activation slice).  Predicated instead of branched, so the other lanes lose no time.
__device__ __forceinline__ void refill_pred(bool pred, uint32_t bar, uint32_t dst_w, const void *src_w, uint32_t wb,
                                            uint32_t dst_x, const void *src_x, uint32_t xb) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 t;\n\t"
        "setp.ne.u32 p, %0, 0;\n\t"
        "@p mbarrier.arrive.expect_tx.shared::cta.b64 t, [%1], %2;\n\t"
        "@p cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%3], [%4], %5, [%1];\n\t"
        "@p cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%6], [%7], %8, [%1];\n\t"
        "}" ::"r"((uint32_t)pred), "r"(bar), "r"(wb + xb), "r"(dst_w), "l"(src_w), "r"(wb), "r"(dst_x), "l"(src_x), "r"(xb)
        : "memory");
}

// d = a . b (first k-step of a block: the C operand is literal zero, no register is cleared)
template <bool BF16>
__device__ __forceinline__ void mma16816_first(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    if constexpr (BF16) {
        asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
            "{0f00000000,0f00000000,0f00000000,0f00000000};"
            : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    } else {
        asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
            "{0f00000000,0f00000000,0f00000000,0f00000000};"
            : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
}
// d += a . b
template <bool BF16>
__device__ __forceinline__ void mma16816_acc(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
    if constexpr (BF16) {
        asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    } else {
        asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
}

// One ring slot: CHUNK tiles (all of them when FULL, else the first tiles_here).  Every shared
// memory address is the slot base plus a compile-time offset plus a per-lane constant.
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 r;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "r"(addr));
    return r;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 r;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(r.x), "=r"(r.y) : "r"(addr));
    return r;
}

template <bool BF16, int MF, int CHUNK, bool FULL>
__device__ __forceinline__ void consume_slot(uint32_t qaddr, uint32_t daddr, const uint32_t (&xaddr)[MF],
                                             int tiles_here, float (&acc)[MF][4]) {
#pragma unroll
    for (int t = 0; t < CHUNK; ++t) {
        if (FULL || t < tiles_here) {
            const uint4 qw = lds128(qaddr + t * TILE_BYTES);
            const uint2 dw = lds64(daddr + t * TILE_BYTES);
#pragma unroll
            for (int kbl = 0; kbl < TILE_KB; ++kbl) {
                uint32_t hlo[4], hhi[4];
                dequant_word<BF16>(kbl ? qw.z : qw.x, hlo);     // column g
                dequant_word<BF16>(kbl ? qw.w : qw.y, hhi);     // column g + 8
                const uint32_t dpair = kbl ? dw.y : dw.x;       // (d of column g, d of column g+8)
                const float dlo = __half2float(__ushort_as_half((uint16_t)(dpair & 0xFFFFu)));
                const float dhi = __half2float(__ushort_as_half((uint16_t)(dpair >> 16)));
#pragma unroll
                for (int f = 0; f < MF; ++f) {
                    const uint4 xv = lds128(xaddr[f] + (t * TILE_K + kbl * QK) * 2);
                    float part[4];
                    mma16816_first<BF16>(part, hlo[0], hhi[0], hlo[1], hhi[1], xv.x, xv.y);
                    mma16816_acc<BF16>(part, hlo[2], hhi[2], hlo[3], hhi[3], xv.z, xv.w);
                    acc[f][0] = fmaf(dlo, part[0], acc[f][0]);
                    acc[f][1] = fmaf(dlo, part[1], acc[f][1]);
                    acc[f][2] = fmaf(dhi, part[2], acc[f][2]);
                    acc[f][3] = fmaf(dhi, part[3], acc[f][3]);
                }
            }
        }
    }
}

// Single activation row (M = 1).  With one row, seven of the eight mma columns would carry
// nothing, so the columns are given to eight different 32-k blocks instead: a group of four
// tiles (eight blocks) shares one accumulator, lane (g, c) feeding x only into column g while it
// multiplies block g (every other lane reads a page of zeros), so that accumulator column j ends
// up holding block j's partial product.  That leaves one scale fma per tile instead of eight,
// and lets the nibbles go in biased, as (OFF + q), with no per-pair subtraction: what has to come
// off, sum((OFF + 8) * x) of the column's block, is put into the accumulator by the tensor core
// itself, two mma per group whose A operand is the constant -(OFF + 8) and whose B operand
// holds block j's x in column j (each lane's own block, which it reads once per group).
//   q, d    lane's nibble slot in tile 0 / scales of tile c, in ring slot 0
//   xs[j]   where the lane reads the x of block j of a group: its slice if j == g, else zeros
//   xown    x of the lane's own block in group 0
//   soff    byte offset of the ring slot (a compile-time constant on the unrolled path)
template <bool BF16, int CHUNK, bool FULL>
__device__ __forceinline__ void m1_consume(uint32_t q, uint32_t d, const uint32_t (&xs)[8], uint32_t xown, uint32_t soff,
                                           int c, int tiles_here, float (&acc)[2]) {
    static_assert(CHUNK % 4 == 0, "groups of four tiles");
    constexpr int NG = CHUNK / 4;
    // -(OFF + 8) as packed pairs: k offsets 0,1,4,5 of a nibble word carry OFF = 1024 (fp16) and
    // the others 64; bf16 carries 128 everywhere
    constexpr uint32_t NEG_LO = BF16 ? 0xC308C308u : 0xE408E408u;      // -136 | -1032
    constexpr uint32_t NEG_HI = BF16 ? 0xC308C308u : 0xD480D480u;      // -136 | -72
    float part[NG][4];
#pragma unroll
    for (int grp = 0; grp < NG; ++grp) {
        const uint4 xo = lds128(xown + soff + grp * 4 * TILE_K * 2);
        mma16816_first<BF16>(part[grp], NEG_LO, NEG_LO, NEG_HI, NEG_HI, xo.x, xo.y);
        mma16816_acc<BF16>(part[grp], NEG_LO, NEG_LO, NEG_HI, NEG_HI, xo.z, xo.w);
    }
    // the groups' accumulator chains are independent: step them side by side
#pragma unroll
    for (int t4 = 0; t4 < 4; ++t4) {
#pragma unroll
        for (int grp = 0; grp < NG; ++grp) {
            const int t = grp * 4 + t4;
            if (FULL || t < tiles_here) {
                const uint4 qw = lds128(q + soff + t * TILE_BYTES);
#pragma unroll
                for (int kbl = 0; kbl < TILE_KB; ++kbl) {
                    const uint4 xv = lds128(xs[t4 * 2 + kbl] + soff + (t * TILE_K + kbl * QK) * 2);
                    uint32_t hlo[4], hhi[4];
                    dequant_word_biased<BF16>(kbl ? qw.z : qw.x, hlo);     // column g
                    dequant_word_biased<BF16>(kbl ? qw.w : qw.y, hhi);     // column g + 8
                    mma16816_acc<BF16>(part[grp], hlo[0], hhi[0], hlo[1], hhi[1], xv.x, xv.y);
                    mma16816_acc<BF16>(part[grp], hlo[2], hhi[2], hlo[3], hhi[3], xv.z, xv.w);
                }
            }
        }
    }
    // part[.][0], [1]: output column g, blocks kb0, kb1 of tile c; [2], [3]: column g+8
#pragma unroll
    for (int grp = 0; grp < NG; ++grp) {
        if (FULL || (grp * 4 + c) < tiles_here) {                      // tile c of the group exists
            const uint2 dq = lds64(d + soff + grp * 4 * TILE_BYTES);
            const float2 d0 = __half22float2(*reinterpret_cast<const __half2 *>(&dq.x));   // d(kb0, g), d(kb0, g+8)
            const float2 d1 = __half22float2(*reinterpret_cast<const __half2 *>(&dq.y));   // d(kb1, g), d(kb1, g+8)
            acc[0] = fmaf(d0.x, part[grp][0], fmaf(d1.x, part[grp][1], acc[0]));
            acc[1] = fmaf(d0.y, part[grp][2], fmaf(d1.y, part[grp][3], acc[1]));
        }
    }
}

template <bool BF16> __device__ __forceinline__ uint16_t out_bits(float v) {
    if constexpr (BF16) return __bfloat16_as_ushort(__float2bfloat16_rn(v));
    else return __half_as_ushort(__float2half_rn(v));
}

// KS = warps of a CTA that split k for the same column tile; the CTA covers 8/KS column tiles.
// CHUNK tiles per ring slot, SLOTS slots per warp.
template <bool BF16, int MF, int KS, int CHUNK, int SLOTS, bool GATHER>
__global__ void __launch_bounds__(GEMV_THREADS)
gemv_kernel(const uint16_t *__restrict__ x, int M, int64_t ldx, const uint8_t *__restrict__ prepacked, int64_t K,
            int64_t N, uint16_t *__restrict__ y, int64_t ldy, const float *__restrict__ addend, int64_t ld_add, int act,
            const PeerOut peers) {
    using G = SlotGeom<CHUNK>;
    constexpr int NTC = GEMV_WARPS / KS;
    extern __shared__ __align__(128) uint8_t ring_all[];
    __shared__ __align__(8) uint64_t bars[GEMV_WARPS][SLOTS];
    __shared__ float red[GEMV_WARPS][MF][TILE_N * 8];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, c = lane & 3;
    const int ks = warp % KS, ntl = warp / KS;
    const int NT = (int)tiles_n(N);
    const int KU = (int)tiles_k(K);
    const int nt = (int)blockIdx.x * NTC + ntl;
    const bool active = nt < NT;
    const int ku0 = KU * ks / KS, ku1 = KU * (ks + 1) / KS;
    const int ntiles = active ? ku1 - ku0 : 0;
    const int nchunks = (ntiles + CHUNK - 1) / CHUNK;
    const int slot_bytes = G::slot_bytes(M);

    uint8_t *ring = ring_all + (size_t)warp * SLOTS * slot_bytes;
    const uint32_t ring_s = smem_addr_u32(ring);
    const uint32_t bar_s = smem_addr_u32(&bars[warp][0]);
    const uint8_t *wsrc = prepacked + tile_offset(active ? nt : 0, ku0, KU);
    const int64_t kbase = (int64_t)ku0 * TILE_K;

    // Refill of ring slot `slot` with chunk `ci`.  Lane 0 arms the slot's barrier with the total
    // byte count and copies the weights; lanes 0..M-1 copy one activation row slice each.  The
    // barrier has a single arrival (lane 0's), so it cannot complete before it is armed, however
    // early the other lanes' copies land.
    auto chunk_w_bytes = [&](int ci) { return (uint32_t)(min(CHUNK, ntiles - ci * CHUNK) * TILE_BYTES); };
    auto chunk_x_bytes = [&](int ci) {
        return (uint32_t)(min((int64_t)CHUNK * TILE_K, K - (kbase + (int64_t)ci * CHUNK * TILE_K)) * 2);
    };
    auto issue_w = [&](int ci, int slot) {      // lane 0 only
        const uint32_t wb = chunk_w_bytes(ci);
        const uint32_t bar = bar_s + 8u * slot;
        mbar_expect_tx(bar, wb + chunk_x_bytes(ci) * (uint32_t)M);
        bulk_g2s(ring_s + (uint32_t)(slot * slot_bytes), wsrc + (size_t)ci * G::W_BYTES, wb, bar);
    };
    auto issue_x = [&](int ci, int slot) {      // lanes 0..M-1
        bulk_g2s(ring_s + (uint32_t)(slot * slot_bytes + G::W_BYTES + lane * G::X_STRIDE),
                 x + (size_t)lane * ldx + kbase + (int64_t)ci * CHUNK * TILE_K, chunk_x_bytes(ci), bar_s + 8u * slot);
    };

    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < SLOTS; ++s)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_s + 8u * s) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
#pragma unroll
        for (int s = 0; s < SLOTS; ++s)
            if (s < nchunks) issue_w(s, s);
    }
    if (K % TILE_K) {
        // Odd number of 32-k blocks: the last tile's pad block has zero weights, but what it is
        // multiplied with must be finite, so the x slices start out as zeros.
        for (int s = 0; s < SLOTS; ++s)
            for (int i = lane * 16; i < M * G::X_STRIDE; i += 32 * 16)
                *reinterpret_cast<uint4 *>(ring + s * slot_bytes + G::W_BYTES + i) = make_uint4(0u, 0u, 0u, 0u);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncwarp();
    // Weights never depend on earlier kernels of the stream; x and y do.  Under programmatic
    // dependent launch the weight copies above overlap the previous kernel's tail.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (lane < M) {
#pragma unroll
        for (int s = 0; s < SLOTS; ++s)
            if (s < nchunks) issue_x(s, s);
    }

    float acc[MF][4];
#pragma unroll
    for (int f = 0; f < MF; ++f)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[f][i] = 0.0f;

    // per-lane shared-memory addresses inside slot 0; other slots add a multiple of slot_bytes
    const uint32_t qaddr0 = ring_s + slot_of(g, c) * 16, daddr0 = ring_s + TILE_QS_BYTES + g * 8;
    uint32_t xaddr0[MF];
#pragma unroll
    for (int f = 0; f < MF; ++f) xaddr0[f] = ring_s + G::W_BYTES + min(f * 8 + g, M - 1) * G::X_STRIDE + c * 16;

    int slot = 0;
    uint32_t parity = 0, soff = 0;           // soff = slot * slot_bytes
    for (int ci = 0; ci < nchunks; ++ci) {
        const uint32_t bar = bar_s + 8u * slot;
        uint32_t done;
        asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (!done) {                     // slow path: bounded polling
            int spins = 0;
            while (!done && ++spins <= GEMV_SPIN_LIMIT)
                asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                             : "=r"(done) : "r"(bar), "r"(parity) : "memory");
            if (!done) atomicCAS(&g_wait_status, 0, 100);
        }
        if (!__all_sync(0xffffffffu, done != 0)) break;
        uint32_t xaddr[MF];
#pragma unroll
        for (int f = 0; f < MF; ++f) xaddr[f] = xaddr0[f] + soff;
        const int tiles_here = ntiles - ci * CHUNK;
        if (tiles_here >= CHUNK) consume_slot<BF16, MF, CHUNK, true>(qaddr0 + soff, daddr0 + soff, xaddr, CHUNK, acc);
        else consume_slot<BF16, MF, CHUNK, false>(qaddr0 + soff, daddr0 + soff, xaddr, tiles_here, acc);
        __syncwarp();                    // every lane has consumed the slot before it is refilled
        if (ci + SLOTS < nchunks) {
            if (lane == 0) issue_w(ci + SLOTS, slot);
            if (lane < M) issue_x(ci + SLOTS, slot);
        }
        soff += (uint32_t)slot_bytes;
        if (++slot == SLOTS) { slot = 0; soff = 0; parity ^= 1; }
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
        const int m = (o / TILE_N) % (MF * 8);
        const int tl = o / (TILE_N * MF * 8);
        const int f = m >> 3, m8 = m & 7;
        const int n = ((int)blockIdx.x * NTC + tl) * TILE_N + nl;
        if (m < M && n < N) {
            float s = 0.0f;
#pragma unroll
            for (int j = 0; j < KS; ++j) s += red[tl * KS + j][f][m8 * TILE_N + nl];
            if (addend != nullptr) s += addend[(size_t)m * ld_add + n];     // fp32 term added before the one rounding
            if (peers.corr != nullptr) {                                    // consecutive threads: consecutive n
                float t = 0.0f;
                for (int gi = 0; gi < peers.G; ++gi) t = fmaf(__ldg(peers.corr + (size_t)gi * N + n), __ldg(peers.rowsums + (size_t)m * peers.G + gi), t);
                s += t;
            }
            s = apply_act(s, act);
            const uint16_t bits = out_bits<BF16>(s);
            if constexpr (!GATHER) {
                y[(size_t)m * ldy + n] = bits;
            } else {
#pragma unroll
                for (int r = 0; r < 8; ++r)        // static indices: the pointers stay in the parameter bank
                    if (r < peers.world) {
                        const size_t at = (size_t)m * peers.ld + peers.col0 + n;
                        if (peers.ll_tag != 0 || peers.ll_ctl != nullptr) {
                            uint32_t tag;
                            int64_t base;
                            ll_call(peers, tag, base);
                            reinterpret_cast<uint32_t *>(peers.p[r])[base + at] = (uint32_t)bits | tag;
                        } else {
                            peers.p[r][at] = bits;
                        }
                    }
            }
        }
    }
}

template <bool BF16, int MF, int KS, int CHUNK, int SLOTS, bool GATHER>
static int launch_gemv_impl(const void *x, int M, int64_t ldx, const void *prepacked, int64_t K, int64_t N, void *y,
                            int64_t ldy, const float *addend, int64_t ld_add, int flags, cudaStream_t st, const PeerOut &po) {
    constexpr int NTC = GEMV_WARPS / KS;
    const int smem = GEMV_WARPS * SLOTS * SlotGeom<CHUNK>::slot_bytes(M);
    // opt in to > 48 KB of dynamic shared memory once per device and instantiation
    static bool attr_done[64] = {};
    static std::mutex attr_mu;
    int dev = 0;
    Q4B_CUDA_TRY(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> attr_lock(attr_mu);
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
        Q4B_CUDA_TRY(cudaFuncSetAttribute(gemv_kernel<BF16, MF, KS, CHUNK, SLOTS, GATHER>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          GEMV_WARPS * SLOTS * SlotGeom<CHUNK>::slot_bytes(MF * 8)));
        if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)ceil_div(tiles_n(N), NTC));
    cfg.blockDim = dim3(GEMV_THREADS);
    cfg.dynamicSmemBytes = (size_t)smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (flags & Q4B_FLAG_PDL) ? 1 : 0;
    Q4B_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemv_kernel<BF16, MF, KS, CHUNK, SLOTS, GATHER>, (const uint16_t *)x, M, ldx,
                                    (const uint8_t *)prepacked, K, N, (uint16_t *)y, ldy, addend, ld_add, act_of_flags(flags), po));
    return Q4B_OK;
}
// the fused all-gather is its own instantiation, so that the plain kernel carries none of it
template <bool BF16, int MF, int KS, int CHUNK, int SLOTS>
static int launch_gemv(const void *x, int M, int64_t ldx, const void *prepacked, int64_t K, int64_t N, void *y,
                       int64_t ldy, const float *addend, int64_t ld_add, int flags, cudaStream_t st, const PeerOut &po) {
    return po.world != 0
               ? launch_gemv_impl<BF16, MF, KS, CHUNK, SLOTS, true>(x, M, ldx, prepacked, K, N, y, ldy, addend, ld_add, flags, st, po)
               : launch_gemv_impl<BF16, MF, KS, CHUNK, SLOTS, false>(x, M, ldx, prepacked, K, N, y, ldy, addend, ld_add, flags, st, po);
}

// ---- single activation row ---------------------------------------------------------------
// Same decomposition as gemv_kernel (a warp per column tile and k range, a private ring per
// warp, warps of a CTA that share a column tile reduced through shared memory), with the slot
// loop unrolled over the ring so that every shared-memory address is a per-lane register plus a
// compile-time offset, and with refills that cost a handful of 32-bit instructions.
template <int CHUNK, int SLOTS> struct M1Geom {
    static constexpr int W_BYTES = CHUNK * TILE_BYTES;
    static constexpr int X_BYTES = CHUNK * TILE_K * 2;            // the chunk's slice of the activation row
    static constexpr int SLOT_BYTES = W_BYTES + X_BYTES;
    static constexpr int RING_BYTES = GEMV_WARPS * SLOTS * SLOT_BYTES;
    // Zero pages, one per ring position and SLOT_BYTES apart, so that "zero page + slot offset"
    // is a zero page again: a lane's eight x addresses then do not depend on the slot.
    static constexpr int ZERO_BYTES = (SLOTS - 1) * SLOT_BYTES + X_BYTES;
};

template <bool BF16, int KS, int CHUNK, int SLOTS, bool GATHER>
__global__ void __launch_bounds__(GEMV_THREADS)
gemv_m1_kernel(const uint16_t *__restrict__ x, const uint8_t *__restrict__ prepacked, int64_t K, int64_t N,
               uint16_t *__restrict__ y, const float *__restrict__ addend, int act, const PeerOut peers) {
    using G = M1Geom<CHUNK, SLOTS>;
    constexpr int NTC = GEMV_WARPS / KS;
    extern __shared__ __align__(128) uint8_t ring_all[];
    __shared__ __align__(16) uint8_t zero_region[G::ZERO_BYTES];
    __shared__ __align__(8) uint64_t bars[GEMV_WARPS][SLOTS];
    __shared__ float red[GEMV_WARPS][TILE_N];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, c = lane & 3;
    const int ks = warp % KS, ntl = warp / KS;
    const int NT = (int)tiles_n(N);
    const int KU = (int)tiles_k(K);
    const int nt = (int)blockIdx.x * NTC + ntl;
    const bool active = nt < NT;
    const int ku0 = KU * ks / KS, ku1 = KU * (ks + 1) / KS;
    const int ntiles = active ? ku1 - ku0 : 0;
    const int nfull = ntiles / CHUNK;                          // chunks with all CHUNK tiles
    const int nchunks = (ntiles + CHUNK - 1) / CHUNK;
    const int xelems = (int)(min((int64_t)ku1 * TILE_K, K) - (int64_t)ku0 * TILE_K);   // x this warp multiplies

    const uint32_t ring_s = smem_addr_u32(ring_all) + (uint32_t)(warp * SLOTS * G::SLOT_BYTES);
    const uint32_t bar_s = smem_addr_u32(&bars[warp][0]);
    const uint8_t *wsrc = prepacked + tile_offset(active ? nt : 0, ku0, KU);
    const uint16_t *xsrc = x + (int64_t)ku0 * TILE_K;

    // Refill of ring position `slot` with chunk `ci` (lane 0 only): the barrier is armed with the
    // bytes of both copies, so it cannot complete before the activation slice has landed too.
    auto chunk_tiles = [&](int ci) { return min(CHUNK, ntiles - ci * CHUNK); };
    auto chunk_x_bytes = [&](int ci) { return (uint32_t)(min(CHUNK * TILE_K, xelems - ci * CHUNK * TILE_K) * 2); };
    auto issue_w = [&](int ci, int slot) {
        const uint32_t wb = (uint32_t)(chunk_tiles(ci) * TILE_BYTES);
        mbar_expect_tx(bar_s + 8u * slot, wb + chunk_x_bytes(ci));
        bulk_g2s(ring_s + (uint32_t)(slot * G::SLOT_BYTES), wsrc + (size_t)ci * G::W_BYTES, wb, bar_s + 8u * slot);
    };
    auto issue_x = [&](int ci, int slot) {
        bulk_g2s(ring_s + (uint32_t)(slot * G::SLOT_BYTES + G::W_BYTES), xsrc + (size_t)ci * CHUNK * TILE_K,
                 chunk_x_bytes(ci), bar_s + 8u * slot);
    };

    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < SLOTS; ++s)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_s + 8u * s) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
#pragma unroll
        for (int s = 0; s < SLOTS; ++s)
            if (s < nchunks) issue_w(s, s);
    }
    // zero pages (what the other seven mma columns read)
    for (int i = threadIdx.x * 16; i < SLOTS * G::X_BYTES; i += GEMV_THREADS * 16)
        *reinterpret_cast<uint4 *>(zero_region + (i / G::X_BYTES) * G::SLOT_BYTES + (i % G::X_BYTES)) =
            make_uint4(0u, 0u, 0u, 0u);
    if (K % TILE_K) {
        // Odd number of 32-k blocks: the last tile's pad block has zero weights, but what it is
        // multiplied with must be finite, so the x slices start out as zeros.
        for (int s = 0; s < SLOTS; ++s)
            for (int i = lane * 16; i < G::X_BYTES; i += 32 * 16)
                *reinterpret_cast<uint4 *>(ring_all + (size_t)(warp * SLOTS + s) * G::SLOT_BYTES + G::W_BYTES + i) =
                    make_uint4(0u, 0u, 0u, 0u);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    // Weights never depend on earlier kernels of the stream; x and y do.  Under programmatic
    // dependent launch the weight copies above overlap the previous kernel's tail.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < SLOTS; ++s)
            if (s < nchunks) issue_x(s, s);
    }

    // per-lane shared-memory addresses inside ring position 0
    const uint32_t q0 = ring_s + slot_of(g, c) * 16;
    const uint32_t d0 = ring_s + c * TILE_BYTES + TILE_QS_BYTES + g * 8;
    const uint32_t xslice = ring_s + G::W_BYTES + c * 16;
    const uint32_t xown = ring_s + G::W_BYTES + ((g >> 1) * TILE_K + (g & 1) * QK + c * 8) * 2;
    const uint32_t zero_s = smem_addr_u32(zero_region) + c * 16;
    uint32_t xs[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) xs[j] = (g == j) ? xslice : zero_s;

    float acc[2] = {0.0f, 0.0f};
    auto wait_slot = [&](uint32_t bar, uint32_t parity) -> bool {
        uint32_t done;
        asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (!done) {                     // slow path: bounded polling
            int spins = 0;
            while (!done && ++spins <= GEMV_SPIN_LIMIT)
                asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                             : "=r"(done) : "r"(bar), "r"(parity) : "memory");
            if (!done) atomicCAS(&g_wait_status, 0, 101);
        }
        return __all_sync(0xffffffffu, done != 0);
    };

    {
        uint32_t parity = 0;
        int ci = 0;
        bool ok = true;
        const int nfast = xelems / (CHUNK * TILE_K);           // chunks whose weights and x slice are both whole
        const uint8_t *wnext = wsrc + (size_t)SLOTS * G::W_BYTES;      // chunk ci + SLOTS
        const uint16_t *xnext = xsrc + (size_t)SLOTS * CHUNK * TILE_K;
        while (ok && ci < nfull) {
#pragma unroll
            for (int s = 0; s < SLOTS; ++s) {
                if (ok && ci < nfull) {
                    ok = wait_slot(bar_s + 8u * s, parity);
                    if (ok) {
                        m1_consume<BF16, CHUNK, true>(q0, d0, xs, xown, (uint32_t)(s * G::SLOT_BYTES), c, CHUNK, acc);
                        __syncwarp();            // every lane has read the slot before it is refilled
                        const uint32_t dst = ring_s + (uint32_t)(s * G::SLOT_BYTES);
                        if (ci + SLOTS < nfast)
                            refill_pred(lane == 0, bar_s + 8u * s, dst, wnext, G::W_BYTES, dst + G::W_BYTES, xnext, G::X_BYTES);
                        else if (ci + SLOTS < nchunks)
                            refill_pred(lane == 0, bar_s + 8u * s, dst, wnext, (uint32_t)(chunk_tiles(ci + SLOTS) * TILE_BYTES),
                                        dst + G::W_BYTES, xnext, chunk_x_bytes(ci + SLOTS));
                        wnext += G::W_BYTES;
                        xnext += CHUNK * TILE_K;
                        ++ci;
                    }
                }
            }
            parity ^= 1;
        }
        if (ok && nchunks > nfull) {             // the k range's last, partial chunk
            const int s = nfull % SLOTS;
            if (wait_slot(bar_s + 8u * s, (uint32_t)((nfull / SLOTS) & 1)))
                m1_consume<BF16, CHUNK, false>(q0, d0, xs, xown, (uint32_t)(s * G::SLOT_BYTES), c, ntiles - nfull * CHUNK, acc);
        }
    }

    // each lane of a quad summed different blocks of output columns g and g+8
    float a0 = acc[0], a1 = acc[1];
    a0 += __shfl_xor_sync(0xffffffffu, a0, 1);
    a1 += __shfl_xor_sync(0xffffffffu, a1, 1);
    a0 += __shfl_xor_sync(0xffffffffu, a0, 2);
    a1 += __shfl_xor_sync(0xffffffffu, a1, 2);
    if (c == 0) {
        red[warp][g] = a0;
        red[warp][g + 8] = a1;
    }
    __syncthreads();
    if (threadIdx.x < NTC * TILE_N) {
        const int tl = threadIdx.x / TILE_N, nl = threadIdx.x % TILE_N;
        const int n = ((int)blockIdx.x * NTC + tl) * TILE_N + nl;
        if (n < N) {
            float sum = 0.0f;
#pragma unroll
            for (int j = 0; j < KS; ++j) sum += red[tl * KS + j][nl];
            if (addend != nullptr) sum += addend[n];           // fp32 term added before the one rounding
            if (peers.corr != nullptr) {                       // consecutive threads: consecutive n
                float t = 0.0f;
                for (int gi = 0; gi < peers.G; ++gi) t = fmaf(__ldg(peers.corr + (size_t)gi * N + n), __ldg(peers.rowsums + gi), t);
                sum += t;
            }
            const uint16_t bits = out_bits<BF16>(apply_act(sum, act));
            if constexpr (!GATHER) {
                y[n] = bits;
            } else {
#pragma unroll
                for (int r = 0; r < 8; ++r)        // static indices: the pointers stay in the parameter bank
                    if (r < peers.world) {
                        if (peers.ll_tag != 0 || peers.ll_ctl != nullptr) {
                            uint32_t tag;
                            int64_t base;
                            ll_call(peers, tag, base);
                            reinterpret_cast<uint32_t *>(peers.p[r])[base + peers.col0 + n] = (uint32_t)bits | tag;
                        } else {
                            peers.p[r][peers.col0 + n] = bits;
                        }
                    }
            }
        }
    }
}

template <bool BF16, int KS, int CHUNK, int SLOTS, bool GATHER>
static int launch_gemv_m1_impl(const void *x, const void *prepacked, int64_t K, int64_t N, void *y, const float *addend,
                               int flags, cudaStream_t st, const PeerOut &po) {
    using G = M1Geom<CHUNK, SLOTS>;
    constexpr int NTC = GEMV_WARPS / KS;
    // opt in to > 48 KB of dynamic shared memory once per device and instantiation
    static bool attr_done[64] = {};
    static std::mutex attr_mu;
    int dev = 0;
    Q4B_CUDA_TRY(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> attr_lock(attr_mu);
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
        Q4B_CUDA_TRY(cudaFuncSetAttribute(gemv_m1_kernel<BF16, KS, CHUNK, SLOTS, GATHER>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, G::RING_BYTES));
        if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)ceil_div(tiles_n(N), NTC));
    cfg.blockDim = dim3(GEMV_THREADS);
    cfg.dynamicSmemBytes = (size_t)G::RING_BYTES;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (flags & Q4B_FLAG_PDL) ? 1 : 0;
    Q4B_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemv_m1_kernel<BF16, KS, CHUNK, SLOTS, GATHER>, (const uint16_t *)x,
                                    (const uint8_t *)prepacked, K, N, (uint16_t *)y, addend, act_of_flags(flags), po));
    return Q4B_OK;
}
template <bool BF16, int KS, int CHUNK, int SLOTS>
static int launch_gemv_m1(const void *x, const void *prepacked, int64_t K, int64_t N, void *y, const float *addend,
                          int flags, cudaStream_t st, const PeerOut &po) {
    return po.world != 0 ? launch_gemv_m1_impl<BF16, KS, CHUNK, SLOTS, true>(x, prepacked, K, N, y, addend, flags, st, po)
                               : launch_gemv_m1_impl<BF16, KS, CHUNK, SLOTS, false>(x, prepacked, K, N, y, addend, flags, st, po);
}

// Ring geometry by row count: shared memory per CTA = 8 warps x SLOTS x (CHUNK x 576 + M x row).
//   M <= 4 : 8 tiles x 2 slots or 4 tiles x 3 slots (see below)
//   M <= 8 : 4 tiles x 2 slots (100 KB)          M <= 16 : 2 tiles x 2 slots (98 KB)
int device_sm_count();

// Single-row launches: k-split and ring geometry by the number of column tiles NT.  A chain of
// decode launches runs fastest when each is one wave of CTAs (the next launch's CTAs then load
// their weights while this one computes, and no late wave starts cold), made of as few and as
// long-lived CTAs as still fill the SMs:
//   NT <= 2 SMs : k-split 8, 8 tiles x 2 slots (2 CTAs per SM)     NT <= 4 SMs : k-split 4, same ring
//   NT <= 6 SMs : k-split 4, 4 tiles x 3 slots (3 CTAs per SM)     beyond      : k-split 4, 4 x 2 (4 per SM)
static int m1_ksplit(int64_t NT, int sms) { return NT <= 2LL * sms ? 8 : 4; }
static int m1_geometry(int64_t NT, int ks, int sms) {
    const int64_t grid = ceil_div(NT, GEMV_WARPS / ks);
    if (grid <= 2LL * sms) return 82;
    if (grid <= 3LL * sms) return 43;
    return 42;
}

template <bool BF16, int KS>
static int launch_gemv_m(const void *x, int M, int64_t ldx, const void *prepacked, int64_t K, int64_t N, void *y,
                         int64_t ldy, const float *addend, int64_t ld_add, int flags, cudaStream_t st, const PeerOut &po) {
    if (M == 1) {
        // one row: the eight mma columns carry eight 32-k blocks (see m1_consume)
        int geom = m1_geometry(tiles_n(N), KS, device_sm_count());
        switch (geom) {
            case 43: return launch_gemv_m1<BF16, KS, 4, 3>(x, prepacked, K, N, y, addend, flags, st, po);
            case 42: return launch_gemv_m1<BF16, KS, 4, 2>(x, prepacked, K, N, y, addend, flags, st, po);
            case 44: return launch_gemv_m1<BF16, KS, 4, 4>(x, prepacked, K, N, y, addend, flags, st, po);
            default: return launch_gemv_m1<BF16, KS, 8, 2>(x, prepacked, K, N, y, addend, flags, st, po);
        }
    }
    // Several rows: slot bytes grow with M (the slot carries the rows' x slices), so the ring gets
    // shorter as M grows.  geom = <tiles per slot><slots>; measured best per M over the Llama-shaped
    // layers: two rows like one row (one wave of CTAs where the ring allows it), 3..8 rows 4 tiles
    // x 2 slots (4 CTAs per SM), more rows 2 x 2.
    int geom = M <= 8 ? 42 : 22;
    if (M == 2) geom = m1_geometry(tiles_n(N), KS, device_sm_count());
    if (M <= 8) {
        switch (geom) {
            case 82: return launch_gemv<BF16, 1, KS, 8, 2>(x, M, ldx, prepacked, K, N, y, ldy, addend, ld_add, flags, st, po);
            case 43: return launch_gemv<BF16, 1, KS, 4, 3>(x, M, ldx, prepacked, K, N, y, ldy, addend, ld_add, flags, st, po);
            case 23: return launch_gemv<BF16, 1, KS, 2, 3>(x, M, ldx, prepacked, K, N, y, ldy, addend, ld_add, flags, st, po);
            case 22: return launch_gemv<BF16, 1, KS, 2, 2>(x, M, ldx, prepacked, K, N, y, ldy, addend, ld_add, flags, st, po);
            default: return launch_gemv<BF16, 1, KS, 4, 2>(x, M, ldx, prepacked, K, N, y, ldy, addend, ld_add, flags, st, po);
        }
    }
    if (geom == 23) return launch_gemv<BF16, 2, KS, 2, 3>(x, M, ldx, prepacked, K, N, y, ldy, addend, ld_add, flags, st, po);
    if (geom == 42) return launch_gemv<BF16, 2, KS, 4, 2>(x, M, ldx, prepacked, K, N, y, ldy, addend, ld_add, flags, st, po);
    return launch_gemv<BF16, 2, KS, 2, 2>(x, M, ldx, prepacked, K, N, y, ldy, addend, ld_add, flags, st, po);
}

template <bool BF16>
static int launch_gemv_ks(int ksplit, const void *x, int M, int64_t ldx, const void *prepacked, int64_t K, int64_t N,
                          void *y, int64_t ldy, const float *addend, int64_t ld_add, int flags, cudaStream_t st, const PeerOut &po) {
    switch (ksplit) {
        case 8: return launch_gemv_m<BF16, 8>(x, M, ldx, prepacked, K, N, y, ldy, addend, ld_add, flags, st, po);
        case 4: return launch_gemv_m<BF16, 4>(x, M, ldx, prepacked, K, N, y, ldy, addend, ld_add, flags, st, po);
        case 2: return launch_gemv_m<BF16, 2>(x, M, ldx, prepacked, K, N, y, ldy, addend, ld_add, flags, st, po);
        default: return launch_gemv_m<BF16, 1>(x, M, ldx, prepacked, K, N, y, ldy, addend, ld_add, flags, st, po);
    }
}


// Reader side of the self-validating words: every thread polls its words until they carry this call's tag
// (bounded: code 700 and zeros on giving up), then writes the plain values.  SLOTS > 1: the row holds SLOTS
// partial results side by side (one per rank), summed here in fp32 in slot order and rounded once.
// A peer may be late for reasons that have nothing to do with the GPU (a host thread that was descheduled, a
// first call that still loads its module), so this bound is seconds, not the fraction of a second of the
// waits inside one kernel.
constexpr long long LL_WAIT_CYCLES = 1LL << 32;      // ~2.3 s
// ctl != null: ctl[0] is the call counter (see PeerOut), ctl[1] counts the blocks that are done; the words
// read are set back to 0 (no epoch), so nothing stale survives a call, and the last block out bumps ctl[0].
template <bool BF16, bool SUM>
__global__ void __launch_bounds__(256)
ll_unpack_kernel(uint32_t *ll, int rows, int64_t cols, int64_t ld_ll, int slots, uint32_t tag, uint16_t *__restrict__ out,
                 int64_t ld_out, int *ctl, int64_t ll_half) {
    if (ctl != nullptr) {
        const int c = *reinterpret_cast<const volatile int *>(ctl);
        tag = (uint32_t)(c % 65535 + 1) << 16;
        if (c & 1) ll += ll_half;
    }
    const int64_t total = (int64_t)rows * cols;
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += (int64_t)gridDim.x * 256) {
        const int64_t m = i / cols, n = i % cols;
        float acc = 0.0f;
        uint32_t last = 0;
        for (int sl = 0; sl < slots; ++sl) {
            uint32_t *w = ll + m * ld_ll + (int64_t)sl * cols + n;
            uint32_t v;
            long long t0 = 0;
            for (int it = 0;; ++it) {
                asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(w) : "memory");
                if ((v & 0xFFFF0000u) == tag) break;
                if ((it & 15) == 15) {
                    const long long now = clock64();
                    if (t0 == 0) t0 = now;
                    else if (now - t0 > LL_WAIT_CYCLES) {
                        atomicCAS(&g_wait_status, 0, 700);
                        v = 0;
                        break;
                    }
                    __nanosleep(100);
                }
            }
            last = v & 0xFFFFu;
            if (ctl != nullptr) *w = 0;
            if (SUM) acc += BF16 ? __bfloat162float(__ushort_as_bfloat16((uint16_t)last)) : __half2float(__ushort_as_half((uint16_t)last));
        }
        out[m * ld_out + n] = SUM ? out_bits<BF16>(acc) : (uint16_t)last;
    }
    if (ctl != nullptr) {
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence();
            if (atomicAdd(&ctl[1], 1) == (int)gridDim.x - 1) {      // the last block out: the next call's counter
                ctl[1] = 0;
                __threadfence();
                atomicAdd(&ctl[0], 1);
            }
        }
    }
}

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
    return q4b_gemv_addend(x, x_dtype, M, ldx, prepacked, K, N, nullptr, 0, y, ldy, flags, stream);
}

// argument checks and launch plan shared by the plain and the gathering entry points
static int gemv_dispatch(const void *x, int x_dtype, int64_t M, int64_t ldx, const void *prepacked, int64_t K, int64_t N,
                         const float *addend, int64_t ld_add, void *y, int64_t ldy, int flags, void *stream,
                         const PeerOut &po) {
    // ld_add == 0: the addend is one row of N values added to every row of the result (a bias)
    if (addend != nullptr && ld_add != 0 && ld_add < N) return Q4B_ERR_ARG;
    if (x == nullptr || prepacked == nullptr || y == nullptr) return Q4B_ERR_ARG;
    if (M < 1 || K <= 0 || N <= 0 || ldx < K || ldy < N) return Q4B_ERR_ARG;
    if (M > 16 || K % QK || tiles_k(K) > (1 << 24)) return Q4B_ERR_SHAPE;
    if (x_dtype != Q4B_F16 && x_dtype != Q4B_BF16) return Q4B_ERR_DTYPE;
    if (act_of_flags(flags) == 3) return Q4B_ERR_ARG;
    if (!aligned(x, 16) || (ldx % 8) || !aligned(prepacked, 16) || !aligned(y, 2)) return Q4B_ERR_ALIGN;
    // k-split (see m1_ksplit for one row), never more splits than k-tiles
    const int64_t NT = tiles_n(N), KU = tiles_k(K);
    int ks = M == 1 ? m1_ksplit(NT, device_sm_count()) : 8;             // several rows: always 8 (measured)
    while (ks > 1 && KU < ks) ks /= 2;
    cudaStream_t st = (cudaStream_t)stream;
    return x_dtype == Q4B_BF16 ? launch_gemv_ks<true>(ks, x, (int)M, ldx, prepacked, K, N, y, ldy, addend, ld_add, flags, st, po)
                               : launch_gemv_ks<false>(ks, x, (int)M, ldx, prepacked, K, N, y, ldy, addend, ld_add, flags, st, po);
}

extern "C" int q4b_gemv_addend(const void *x, int x_dtype, int64_t M, int64_t ldx, const void *prepacked, int64_t K,
                               int64_t N, const float *addend, int64_t ld_add, void *y, int64_t ldy, int flags,
                               void *stream) {
    return gemv_dispatch(x, x_dtype, M, ldx, prepacked, K, N, addend, ld_add, y, ldy, flags, stream, PeerOut{});
}

// The group-wise INT4 product for up to 16 rows with its zero-point term formed in the epilogue from the
// rows' group sums (rowsums [M, G] fp32, from q4b_int4g_rowsums) and corr [G, N]; bias: one fp32 row or NULL.
extern "C" int q4b_int4g_gemv(const void *x, int x_dtype, int64_t M, int64_t ldx, const void *prepacked, int64_t K, int64_t N,
                              const float *corr, const float *rowsums, int64_t group, const float *bias, void *y, int64_t ldy,
                              int flags, void *stream) {
    if (corr == nullptr || rowsums == nullptr || group < 1 || K < 1) return Q4B_ERR_ARG;
    const int64_t G = ceil_div(K, group);
    if (G > 65535) return Q4B_ERR_SHAPE;
    PeerOut po = {};
    po.corr = corr;
    po.rowsums = rowsums;
    po.G = (int)G;
    return gemv_dispatch(x, x_dtype, M, ldx, prepacked, K, N, bias, 0, y, ldy, flags, stream, po);
}

static int launch_ll_unpack(const void *ll, int64_t rows, int64_t cols, int64_t ld_ll, int slots, uint32_t tag, int x_dtype, void *out,
                            int64_t ld_out, int *ctl, int64_t ll_half, cudaStream_t st) {
    const int64_t total = rows * cols;
    const unsigned grid = (unsigned)(ceil_div(total, 256) < 1184 ? ceil_div(total, 256) : 1184);
    uint32_t *w = (uint32_t *)const_cast<void *>(ll);
    if (slots == 1)
        ll_unpack_kernel<false, false><<<grid, 256, 0, st>>>(w, (int)rows, cols, ld_ll, 1, tag, (uint16_t *)out, ld_out, ctl, ll_half);
    else if (x_dtype == Q4B_BF16)
        ll_unpack_kernel<true, true><<<grid, 256, 0, st>>>(w, (int)rows, cols, ld_ll, slots, tag, (uint16_t *)out, ld_out, ctl, ll_half);
    else
        ll_unpack_kernel<false, true><<<grid, 256, 0, st>>>(w, (int)rows, cols, ld_ll, slots, tag, (uint16_t *)out, ld_out, ctl, ll_half);
    Q4B_LAUNCH_CHECK();
    return Q4B_OK;
}

// The gather without barriers: the peers' buffers are uint32 [rows, ld_out] and every store carries the call's
// epoch (1..65535) in its upper half; q4b_gather_ll_unpack on each rank waits, word by word and bounded, for
// all words of the epoch and writes the plain result.  The caller alternates between two buffers from call
// to call (stream order then guarantees that nobody still reads the buffer being overwritten).
extern "C" int q4b_gemv_gather_ll(const void *x, int x_dtype, int64_t M, int64_t ldx, const void *prepacked, int64_t K,
                                  int64_t N, void *const *ll_ranks, int world, int64_t col0, int64_t ld_out, int epoch, int flags,
                                  void *stream) {
    if (ll_ranks == nullptr || world < 1 || world > 8 || col0 < 0 || ld_out < col0 + N) return Q4B_ERR_ARG;
    if (epoch < 1 || epoch > 65535) return Q4B_ERR_ARG;
    for (int r = 0; r < world; ++r)
        if (ll_ranks[r] == nullptr || !aligned(ll_ranks[r], 4)) return Q4B_ERR_ARG;
    PeerOut po = {};
    for (int r = 0; r < world; ++r) po.p[r] = (uint16_t *)ll_ranks[r];
    po.world = world;
    po.col0 = col0;
    po.ld = ld_out;
    po.ll_tag = (uint32_t)epoch << 16;
    return gemv_dispatch(x, x_dtype, M, ldx, prepacked, K, N, nullptr, 0, ll_ranks[0], ld_out, flags, stream, po);
}

// slots == 1: out[m, n] = value of ll[m, n].  slots > 1: out[m, n] = sum over s of ll[m, s * cols + n], fp32, slot
// order, one rounding to x_dtype (the partial products of a row-parallel layer).
extern "C" int q4b_gather_ll_unpack(const void *ll, int64_t rows, int64_t cols, int64_t ld_ll, int slots, int epoch, int x_dtype,
                                    void *out, int64_t ld_out, void *stream) {
    if (ll == nullptr || out == nullptr || rows < 1 || rows > 16 || cols < 1 || slots < 1 || slots > 8) return Q4B_ERR_ARG;
    if (ld_ll < (int64_t)slots * cols || ld_out < cols || epoch < 1 || epoch > 65535) return Q4B_ERR_ARG;
    if (x_dtype != Q4B_F16 && x_dtype != Q4B_BF16) return Q4B_ERR_DTYPE;
    return launch_ll_unpack(ll, rows, cols, ld_ll, slots, (uint32_t)epoch << 16, x_dtype, out, ld_out, nullptr, 0, (cudaStream_t)stream);
}

// The exchange with the call counter in device memory (ctl: two ints, zero at set-up; the two buffers of a
// rank are ll_half words apart, ll_ranks / ll_local point at the first): nothing changes from call to call on
// the host side, so a captured launch can be replayed.  The unpack sets the words it read back to zero.
extern "C" int q4b_gemv_exchange_dev(const void *x, int x_dtype, int64_t M, int64_t ldx, const void *prepacked, int64_t K, int64_t N,
                                     void *const *ll_ranks, int world, int64_t col0, int64_t ld_out, void *ll_local, int64_t ll_half,
                                     int slots, int *ctl, void *out, int64_t ld_y, int flags, void *stream) {
    if (ll_ranks == nullptr || world < 1 || world > 8 || col0 < 0 || ld_out < col0 + N || ctl == nullptr || ll_half < 16 * ld_out)
        return Q4B_ERR_ARG;
    if (ll_local == nullptr || out == nullptr || slots < 1 || slots > 8 || M < 1 || M > 16) return Q4B_ERR_ARG;
    for (int r = 0; r < world; ++r)
        if (ll_ranks[r] == nullptr || !aligned(ll_ranks[r], 4)) return Q4B_ERR_ARG;
    PeerOut po = {};
    for (int r = 0; r < world; ++r) po.p[r] = (uint16_t *)ll_ranks[r];
    po.world = world;
    po.col0 = col0;
    po.ld = ld_out;
    po.ll_ctl = ctl;
    po.ll_half = ll_half;
    if (int rc = gemv_dispatch(x, x_dtype, M, ldx, prepacked, K, N, nullptr, 0, ll_ranks[0], ld_out, flags, stream, po)) return rc;
    const int64_t cols = slots > 1 ? N : ld_out;
    if (ld_out < (int64_t)slots * cols || ld_y < cols) return Q4B_ERR_ARG;
    return launch_ll_unpack(ll_local, M, cols, ld_out, slots, 0, x_dtype, out, ld_y, ctl, ll_half, (cudaStream_t)stream);
}

// Both steps of the barrier-free exchange in one call: the product stored into every rank's words, then the
// wait-and-unpack of this rank's own words (ll_local = this rank's entry of ll_ranks) into out.
// slots == 1: a gather (out is [M, ld_out] wide, col0 = this rank's first column); slots > 1: the reduction of
// `slots` partial results (ld_out = slots * N, col0 = rank * N; out is [M, N]).
extern "C" int q4b_gemv_exchange(const void *x, int x_dtype, int64_t M, int64_t ldx, const void *prepacked, int64_t K, int64_t N,
                                 void *const *ll_ranks, int world, int64_t col0, int64_t ld_out, const void *ll_local, int slots,
                                 int epoch, void *out, int64_t ld_y, int flags, void *stream) {
    if (int rc = q4b_gemv_gather_ll(x, x_dtype, M, ldx, prepacked, K, N, ll_ranks, world, col0, ld_out, epoch, flags, stream)) return rc;
    const int64_t cols = slots > 1 ? N : ld_out;
    return q4b_gather_ll_unpack(ll_local, M, cols, ld_out, slots, epoch, x_dtype, out, ld_y, stream);
}

extern "C" int q4b_gemv_gather(const void *x, int x_dtype, int64_t M, int64_t ldx, const void *prepacked, int64_t K,
                               int64_t N, void *const *y_ranks, int world, int64_t col0, int64_t ld_out, int flags,
                               void *stream) {
    if (y_ranks == nullptr || world < 1 || world > 8 || col0 < 0 || ld_out < col0 + N) return Q4B_ERR_ARG;
    for (int r = 0; r < world; ++r)
        if (y_ranks[r] == nullptr || !aligned(y_ranks[r], 2)) return Q4B_ERR_ARG;
    PeerOut po = {};
    for (int r = 0; r < world; ++r) po.p[r] = (uint16_t *)y_ranks[r];
    po.world = world;
    po.col0 = col0;
    po.ld = ld_out;
    // y itself is not written in this mode; the first rank pointer stands in for the argument checks
    return gemv_dispatch(x, x_dtype, M, ldx, prepacked, K, N, nullptr, 0, y_ranks[0], ld_out, flags, stream, po);
}
