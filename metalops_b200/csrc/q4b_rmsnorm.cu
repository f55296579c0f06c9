// RMSNorm in front of a quantised linear layer: y[m, :] = T(float(x[m, :]) * rstd[m] * float(w[:])),
// rstd = rsqrt(mean(x^2) + eps), sums in fp32.
//
// First step of the reference's fused_rmsnorm_linear_int4 (core_mps.mm:3017-3103), which runs its
// rmsnorm_fwd_half kernel (training_kernels.metal:425-485) and its INT4 matmul back to back on one
// command encoder with the normalised activations rounded to half in between; the same two steps
// are issued here on one stream.  HBM-bound and tiny next to the matmul it feeds (2 x M x K x 2 bytes).
#include "q4b_common.cuh"

namespace q4b {

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// one CTA per row; the row is read twice (the second time from L1/L2)
template <typename T>
__global__ void __launch_bounds__(256)
rmsnorm_kernel(const T *__restrict__ x, int64_t ldx, const T *__restrict__ w, int64_t K, float eps, T *__restrict__ y,
               int64_t ldy) {
    __shared__ float partial[8];
    __shared__ float s_rstd;
    const T *xr = x + (size_t)blockIdx.x * ldx;
    T *yr = y + (size_t)blockIdx.x * ldy;
    float sum = 0.0f;
    for (int64_t i = threadIdx.x; i < K; i += blockDim.x) {
        const float v = to_f32<T>(xr[i]);
        sum += v * v;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
        float total = 0.0f;
        for (int i = 0; i < (int)(blockDim.x >> 5); ++i) total += partial[i];     // fixed order: repeatable
        s_rstd = rsqrtf(total / (float)K + eps);
    }
    __syncthreads();
    const float rstd = s_rstd;
    for (int64_t i = threadIdx.x; i < K; i += blockDim.x)
        yr[i] = from_f32<T>(to_f32<T>(xr[i]) * rstd * to_f32<T>(w[i]));
}

}  // namespace q4b

using namespace q4b;

extern "C" int q4b_rmsnorm(const void *x, int dtype, int64_t M, int64_t K, int64_t ldx, const void *weight, float eps,
                           void *y, int64_t ldy, void *stream) {
    if (x == nullptr || weight == nullptr || y == nullptr) return Q4B_ERR_ARG;
    if (M < 1 || K < 1 || ldx < K || ldy < K || M > (1LL << 31) - 1) return Q4B_ERR_ARG;
    if (dtype != Q4B_F16 && dtype != Q4B_BF16) return Q4B_ERR_DTYPE;
    if (q4b_device_ok() != Q4B_OK) return Q4B_ERR_ARCH;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == Q4B_F16)
        rmsnorm_kernel<__half><<<(unsigned)M, 256, 0, st>>>((const __half *)x, ldx, (const __half *)weight, K, eps, (__half *)y, ldy);
    else
        rmsnorm_kernel<__nv_bfloat16><<<(unsigned)M, 256, 0, st>>>((const __nv_bfloat16 *)x, ldx, (const __nv_bfloat16 *)weight, K,
                                                                  eps, (__nv_bfloat16 *)y, ldy);
    Q4B_LAUNCH_CHECK();
    return Q4B_OK;
}
