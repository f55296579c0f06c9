// Entry points of the tensor-core matmul (more rows than the decode kernels take) and the status of the
// library's bounded waits.
//
// Replaces the reference's dispatch to its simdgroup kernel matmul_ggml_q4_0
// (packages/metalcore/src/metalcore/native/core_mps.mm:5917-5975, kernel quant_kernels.metal:1738-1886).
// Both kernels behind q4b_gemm keep the dequantised weights in tensor memory as the tcgen05 A operand:
//   M <= 128   q4b_gemm_tmem.cu: a CTA per 128-column panel and k range (clusters split k), whose cost per
//              k-tile does not depend on M, unless the weight has more panels than two per SM;
//   otherwise  q4b_gemm_wt.cu: persistent CTAs over items of 128 columns x up to 256 rows x all of k.
#include <cuda.h>

#include <mutex>

#include "q4b_sm100_ptx.cuh"

namespace q4b {

int device_sm_count();
int gemm_tmem_launch(const void *x, int bf16, int M, int64_t ldx, const void *prepacked, int64_t K, int64_t N,
                     const float *addend, int64_t ld_add, void *y, int64_t ldy, int flags, cudaStream_t st,
                     const void *corr_op = nullptr, const void *xr = nullptr, int KX = 0);
int gemm_wt_launch(const void *x, int bf16, int M, int64_t ldx, const void *prepacked, int64_t K, int64_t N, const float *addend,
                   int64_t ld_add, void *y, int64_t ldy, int flags, cudaStream_t st, const void *corr_op = nullptr,
                   const void *xr = nullptr, int KX = 0);
int gemv_wait_status(int *value);
int gemm_tmem_wait_status(int *value);
int gemm_wt_wait_status(int *value);
namespace chain { int wait_status(int *value); }
int selftest_wait_status(int *value);

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

int encode_x_tensor_map(CUtensorMap *map, const void *x, int bf16, int64_t M, int64_t K, int64_t ldx, int rows) {
    EncodeTiledFn enc = get_encode_fn();
    if (enc == nullptr) return Q4B_ERR_CUDA;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
    const cuuint64_t strides[1] = {(cuuint64_t)ldx * 2};
    const cuuint32_t box[2] = {(cuuint32_t)TILE_K, (cuuint32_t)rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = enc(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(x),
                           dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? Q4B_OK : Q4B_ERR_ARG;
}

// argument checks shared by q4b_gemm_addend and q4b_gemm_wt_addend
static int check_gemm_args(const void *x, int x_dtype, int64_t M, int64_t ldx, const void *prepacked, int64_t K, int64_t N,
                           const float *addend, int64_t ld_add, const void *y, int64_t ldy, int flags) {
    // ld_add == 0: the addend is one row of N values added to every row of the result (a bias)
    if (addend != nullptr && ld_add != 0 && ld_add < N) return Q4B_ERR_ARG;
    if (x == nullptr || prepacked == nullptr || y == nullptr) return Q4B_ERR_ARG;
    if (M < 1 || K <= 0 || N <= 0 || ldx < K || ldy < N) return Q4B_ERR_ARG;
    if (act_of_flags(flags) == 3) return Q4B_ERR_ARG;
    if (K % QK || M > (1 << 30) || N > (1 << 30) || K > (1 << 30)) return Q4B_ERR_SHAPE;
    if (x_dtype != Q4B_F16 && x_dtype != Q4B_BF16) return Q4B_ERR_DTYPE;
    if (!aligned(x, 16) || (ldx % 8) || !aligned(prepacked, 16) || !aligned(y, 2)) return Q4B_ERR_ALIGN;
    if (q4b_device_ok() != Q4B_OK) return Q4B_ERR_ARCH;
    return Q4B_OK;
}

}  // namespace q4b

using namespace q4b;

extern "C" int q4b_gemm(const void *x, int x_dtype, int64_t M, int64_t ldx, const void *prepacked, int64_t K,
                        int64_t N, void *y, int64_t ldy, int flags, void *stream) {
    return q4b_gemm_addend(x, x_dtype, M, ldx, prepacked, K, N, nullptr, 0, y, ldy, flags, stream);
}

extern "C" int q4b_gemm_addend(const void *x, int x_dtype, int64_t M, int64_t ldx, const void *prepacked, int64_t K,
                               int64_t N, const float *addend, int64_t ld_add, void *y, int64_t ldy, int flags,
                               void *stream) {
    if (int rc = check_gemm_args(x, x_dtype, M, ldx, prepacked, K, N, addend, ld_add, y, ldy, flags)) return rc;
    if (M <= 128 && ceil_div(tiles_n(N), 8) <= 2 * device_sm_count())
        return gemm_tmem_launch(x, x_dtype == Q4B_BF16, (int)M, ldx, prepacked, K, N, addend, ld_add, y, ldy, flags,
                                (cudaStream_t)stream);
    return gemm_wt_launch(x, x_dtype == Q4B_BF16, (int)M, ldx, prepacked, K, N, addend, ld_add, y, ldy, flags, (cudaStream_t)stream);
}

// The persistent kernel whatever M: same arguments and checks as q4b_gemm_addend.
extern "C" int q4b_gemm_wt_addend(const void *x, int x_dtype, int64_t M, int64_t ldx, const void *prepacked, int64_t K,
                                  int64_t N, const float *addend, int64_t ld_add, void *y, int64_t ldy, int flags,
                                  void *stream) {
    if (int rc = check_gemm_args(x, x_dtype, M, ldx, prepacked, K, N, addend, ld_add, y, ldy, flags)) return rc;
    return gemm_wt_launch(x, x_dtype == Q4B_BF16, (int)M, ldx, prepacked, K, N, addend, ld_add, y, ldy, flags, (cudaStream_t)stream);
}

// The group-wise INT4 product with its zero-point term folded into the contraction (the kernels behind
// q4b_gemm, picked by M as there; any M >= 1): KX further k-tiles multiply fold_rows [M, 64 KX] by fold_operand [N, 64 KX] (both
// bf16, from q4b_int4g_fold_rows / q4b_int4g_fold_operand).  bias: one fp32 row of N values, or NULL.
extern "C" int q4b_int4g_gemm_fold(const void *x, int x_dtype, int64_t M, int64_t ldx, const void *prepacked, int64_t K, int64_t N,
                                   const void *fold_operand, const void *fold_rows, int KX, const float *bias, void *y,
                                   int64_t ldy, int flags, void *stream) {
    if (int rc = check_gemm_args(x, x_dtype, M, ldx, prepacked, K, N, bias, 0, y, ldy, flags)) return rc;
    if (fold_operand == nullptr || fold_rows == nullptr || KX < 1 || KX > 4096) return Q4B_ERR_ARG;
    if (!aligned(fold_operand, 16) || !aligned(fold_rows, 16)) return Q4B_ERR_ALIGN;
    if (M <= 128 && ceil_div(tiles_n(N), 8) <= 2 * device_sm_count())
        return gemm_tmem_launch(x, x_dtype == Q4B_BF16, (int)M, ldx, prepacked, K, N, bias, 0, y, ldy, flags, (cudaStream_t)stream,
                                fold_operand, fold_rows, KX);
    return gemm_wt_launch(x, x_dtype == Q4B_BF16, (int)M, ldx, prepacked, K, N, bias, 0, y, ldy, flags, (cudaStream_t)stream,
                          fold_operand, fold_rows, KX);
}

// Synchronises the stream, then reads and clears the status words of every kernel with bounded waits.
extern "C" int q4b_wait_status(void *stream, int *detail) {
    Q4B_CUDA_TRY(cudaStreamSynchronize((cudaStream_t)stream));
    int h = 0, hv = 0;
    if (int rc = gemv_wait_status(&hv)) return rc;
    if (h == 0) h = hv;
    if (int rc = gemm_tmem_wait_status(&hv)) return rc;
    if (h == 0) h = hv;
    if (int rc = gemm_wt_wait_status(&hv)) return rc;
    if (h == 0) h = hv;
    if (int rc = chain::wait_status(&hv)) return rc;
    if (h == 0) h = hv;
    if (int rc = selftest_wait_status(&hv)) return rc;
    if (h == 0) h = hv;
    if (detail) *detail = h;
    return h != 0 ? Q4B_ERR_TIMEOUT : Q4B_OK;
}
