// Thin wrappers around the sm_100a PTX used by the tensor-memory kernels: mbarriers with bounded
// waits, bulk and tensor copies, tcgen05 (alloc-free parts), cluster helpers, operand descriptors.
#pragma once

#include <cuda.h>

#include "q4b_common.cuh"

namespace q4b {
namespace ptx {

constexpr long long WAIT_LIMIT_CYCLES = 1LL << 28;   // ~0.15 s; far above any legitimate wait

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
// Bounded wait: false when another role aborted or when this wait ran out, in which case it records
// `code` in *status (first writer wins) and raises the CTA-wide abort flag.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int *status, int code,
                                          long long limit_cycles = WAIT_LIMIT_CYCLES) {
    if (mbar_try_wait(bar, parity)) return true;
    long long t0 = 0;
    for (int it = 1;; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 63) == 0) {
            if (*abort_flag) return false;
            const long long now = clock64();
            if (t0 == 0) t0 = now;
            else if (now - t0 > limit_cycles) {
                *abort_flag = 1;
                atomicCAS(status, 0, code);
                return false;
            }
        }
    }
}
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int *abort_flag, int *status, int code) {
    return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag, status, code));
}
// true on one lane of the (converged) warp
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{ .reg .pred p; elect.sync _|p, 0xffffffff; selp.u32 %0, 1, 0, p; }" : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[tmem] . B[smem descriptor]
__device__ __forceinline__ void tc_mma_ts_f16(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc,
                                              uint32_t accumulate) {
    asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p; }"
                 ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// 16 registers <-> 16 consecutive columns of the thread's own tensor-memory lane
__device__ __forceinline__ void tc_st_32x32b_x16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void tc_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// the float at the same shared-memory offset in CTA `rank` of the cluster
__device__ __forceinline__ float ld_cluster_f32(uint32_t local_addr, uint32_t rank) {
    uint32_t remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}
// four floats at the same (16-byte aligned) shared-memory offset in CTA `rank` of the cluster
__device__ __forceinline__ float4 ld_cluster_f32x4(uint32_t local_addr, uint32_t rank) {
    uint32_t remote;
    float4 v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote) : "memory");
    return v;
}
// K-major operand tile stored as rows of 128 bytes (64 16-bit elements) with the 128-byte swizzle:
// 8-row groups 1024 bytes apart.  A k16 step inside the tile adds 32 bytes (2 units) to the address.
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

// One k-tile of a 128-column panel, packed in shared memory at `wst` (eight 576-byte tiles, `run` bytes
// apart), dequantised into 32 columns of tensor memory at `taddr` as the tcgen05 A operand: a warp covers
// one lane quadrant, thread = output column, (q - 8) * d rounded once to the activations' type.
// woff[c] / doff: the thread's byte offsets of nibble word c and of its scale inside the k-tile.
template <bool BF16>
__device__ __forceinline__ void dequant_tile_to_tmem(uint32_t wst, const uint32_t (&woff)[4], uint32_t doff, uint32_t taddr) {
    uint32_t w[2][4];
#pragma unroll
    for (int kb = 0; kb < 2; ++kb)
#pragma unroll
        for (int c = 0; c < 4; ++c)
            asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w[kb][c]) : "r"(wst + woff[c] + kb * 8));
    uint32_t dbits[2];
    asm volatile("ld.shared.u16 %0, [%1];" : "=r"(dbits[0]) : "r"(wst + doff));
    asm volatile("ld.shared.u16 %0, [%1];" : "=r"(dbits[1]) : "r"(wst + doff + 4));
#pragma unroll
    for (int kb = 0; kb < 2; ++kb) {
        const uint32_t d2 = scale_pair<BF16>((uint16_t)dbits[kb]);
        uint32_t regs[16];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            uint32_t h[4];
            dequant_word<BF16>(w[kb][c], h);
#pragma unroll
            for (int e = 0; e < 4; ++e) regs[4 * c + e] = BF16 ? bmul2_bits(h[e], d2) : hmul2_bits(h[e], d2);
        }
        tc_st_32x32b_x16(taddr + (uint32_t)(kb * 16), regs);
    }
}

}  // namespace ptx

// Tensor map of the activations X [M, K] (K contiguous, leading dimension ldx) for copies of
// 64 k x `rows` rows with the 128-byte swizzle; rows beyond M read as zero.  Defined in q4b_gemm.cu.
int encode_x_tensor_map(CUtensorMap *map, const void *x, int bf16, int64_t M, int64_t K, int64_t ldx, int rows);

}  // namespace q4b
