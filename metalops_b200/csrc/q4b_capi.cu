// C-ABI glue: status strings, device checks, the M-based dispatcher and the host-buffer
// convenience entry.  The kernels live in q4b_quantize.cu, q4b_gemv.cu, q4b_gemm_tmem.cu and q4b_gemm_wt.cu.
#include <cstdio>
#include <cstring>
#include <mutex>

#include "q4b_common.cuh"
#include "q4b_sm100_ptx.cuh"

namespace q4b {

static thread_local char g_cuda_err[256] = "";

void set_cuda_error(cudaError_t e) {
    const char *name = cudaGetErrorName(e);
    const char *text = cudaGetErrorString(e);
    snprintf(g_cuda_err, sizeof(g_cuda_err), "%s: %s", name ? name : "?", text ? text : "?");
    // configuration errors are sticky in cudaGetLastError only; clear so the next launch is clean
    (void)cudaGetLastError();
}

// Per-device facts, read once.  Guarded by a mutex: callers may use several host threads.
struct DevInfo {
    bool known = false;
    int sms = 0;
    int major = 0;
};
static DevInfo g_dev[64];
static std::mutex g_dev_mu;

static const DevInfo *dev_info() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lk(g_dev_mu);
    DevInfo &d = g_dev[dev];
    if (!d.known) {
        if (cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return nullptr;
        if (cudaDeviceGetAttribute(&d.major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return nullptr;
        d.known = true;
    }
    return &d;
}

int device_sm_count() {
    const DevInfo *d = dev_info();
    return d ? d->sms : 148;
}

}  // namespace q4b

using namespace q4b;

extern "C" const char *q4b_strerror(int status) {
    switch (status) {
        case Q4B_OK: return "ok";
        case Q4B_ERR_ARG: return "invalid argument (null pointer, non-positive size or unknown enum)";
        case Q4B_ERR_SHAPE: return "unsupported shape (K must be a multiple of 32; see the entry point's limits)";
        case Q4B_ERR_DTYPE: return "unsupported dtype for this entry point";
        case Q4B_ERR_ALIGN: return "pointer or leading dimension is not aligned as the entry point requires";
        case Q4B_ERR_ARCH: return "the current device is not compute capability 10.x (B200, sm_100a)";
        case Q4B_ERR_CUDA: return "a CUDA runtime call failed (see q4b_last_cuda_error)";
        case Q4B_ERR_TIMEOUT: return "a bounded device-side wait gave up";
        case Q4B_ERR_TOO_LARGE: return "problem exceeds a fixed internal buffer";
        default: return "unknown q4b status";
    }
}

extern "C" const char *q4b_last_cuda_error(void) { return g_cuda_err; }

extern "C" int q4b_version(void) { return 100; }

extern "C" int q4b_device_ok(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) {
        (void)cudaGetLastError();
        return Q4B_ERR_ARCH;
    }
    const DevInfo *d = dev_info();
    if (d == nullptr) return Q4B_ERR_CUDA;
    return d->major == 10 ? Q4B_OK : Q4B_ERR_ARCH;
}

extern "C" int q4b_matmul(const void *x, int x_dtype, int64_t M, int64_t ldx, const void *prepacked, int64_t K,
                          int64_t N, void *y, int64_t ldy, int flags, void *stream) {
    return q4b_matmul_addend(x, x_dtype, M, ldx, prepacked, K, N, nullptr, 0, y, ldy, flags, stream);
}

extern "C" int q4b_matmul_addend(const void *x, int x_dtype, int64_t M, int64_t ldx, const void *prepacked, int64_t K,
                                 int64_t N, const float *addend, int64_t ld_add, void *y, int64_t ldy, int flags,
                                 void *stream) {
    // Up to 8 rows: decode kernels.  9..16 rows: decode kernel for small weights, else the
    // tensor-memory kernel behind q4b_gemm (measured crossover: the decode kernel re-reads x per
    // column tile, which at 16 rows is 3.5x the weight bytes).  More rows: q4b_gemm.
    if (M >= 1 && (M <= 8 || (M <= 16 && K * N < (1LL << 25))))
        return q4b_gemv_addend(x, x_dtype, M, ldx, prepacked, K, N, addend, ld_add, y, ldy, flags, stream);
    return q4b_gemm_addend(x, x_dtype, M, ldx, prepacked, K, N, addend, ld_add, y, ldy, flags, stream);
}

extern "C" int q4b_matmul_host(const void *x_host, void *x_dev, int x_dtype, int64_t M, const void *prepacked,
                               int64_t K, int64_t N, void *y_dev, void *y_host, int flags, void *stream) {
    if (x_host == nullptr || x_dev == nullptr || y_dev == nullptr || y_host == nullptr) return Q4B_ERR_ARG;
    if (M < 1 || K <= 0 || N <= 0) return Q4B_ERR_ARG;
    if (x_dtype != Q4B_F16 && x_dtype != Q4B_BF16) return Q4B_ERR_DTYPE;
    cudaStream_t st = (cudaStream_t)stream;
    Q4B_CUDA_TRY(cudaMemcpyAsync(x_dev, x_host, (size_t)M * K * 2, cudaMemcpyHostToDevice, st));
    // the copy above writes x, so the kernel must not start before it: no early launch here
    int rc = q4b_matmul(x_dev, x_dtype, M, K, prepacked, K, N, y_dev, N, flags & ~Q4B_FLAG_PDL, stream);
    if (rc != Q4B_OK) return rc;
    Q4B_CUDA_TRY(cudaMemcpyAsync(y_host, y_dev, (size_t)M * N * 2, cudaMemcpyDeviceToHost, st));
    return Q4B_OK;
}

// ---------------------------------------------------------------------------------------------
// q4b_matmul_host_noalloc: the same host-buffer product, for callers that cannot allocate device
// memory.  The two device staging buffers that q4b_matmul_host takes from its caller live in
// this file-scope array instead.  Every GPU that loads the library carries the array until the
// process exits, so it is kept modest.
// ---------------------------------------------------------------------------------------------
namespace q4b {

constexpr size_t NOALLOC_SCRATCH_BYTES = Q4B_NOALLOC_MAX_BYTES;
static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_SCRATCH_BYTES];

// In host code `g_noalloc_scratch` only names the symbol; it is not a device address.  The real
// address is asked for once per device, with that device current, and kept here.
static unsigned char *g_noalloc_ptr[64] = {};
static std::mutex g_noalloc_mu;

static int noalloc_scratch(unsigned char **out) {
    int dev = 0;
    Q4B_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return Q4B_ERR_ARG;
    std::lock_guard<std::mutex> lk(g_noalloc_mu);
    if (g_noalloc_ptr[dev] == nullptr) {
        void *p = nullptr;
        Q4B_CUDA_TRY(cudaGetSymbolAddress(&p, g_noalloc_scratch));
        if (p == nullptr) return Q4B_ERR_CUDA;
        g_noalloc_ptr[dev] = static_cast<unsigned char *>(p);
    }
    *out = g_noalloc_ptr[dev];
    return Q4B_OK;
}

}  // namespace q4b

extern "C" int q4b_matmul_host_noalloc(const void *x_host, int x_dtype, int64_t M, const void *prepacked, int64_t K,
                                       int64_t N, void *y_host, void *stream) {
    if (x_host == nullptr || prepacked == nullptr || y_host == nullptr) return Q4B_ERR_ARG;
    if (M < 1 || K <= 0 || N <= 0) return Q4B_ERR_ARG;
    if (x_dtype != Q4B_F16 && x_dtype != Q4B_BF16) return Q4B_ERR_DTYPE;
    if (K % QK) return Q4B_ERR_SHAPE;
    // X staging first, Y staging after it, both on 256-byte boundaries
    const size_t x_bytes = ((size_t)M * (size_t)K * 2 + 255) & ~(size_t)255;
    const size_t y_bytes = ((size_t)M * (size_t)N * 2 + 255) & ~(size_t)255;
    if (x_bytes > NOALLOC_SCRATCH_BYTES || y_bytes > NOALLOC_SCRATCH_BYTES - x_bytes) return Q4B_ERR_TOO_LARGE;
    unsigned char *scratch = nullptr;
    if (int rc = noalloc_scratch(&scratch)) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    void *x_dev = scratch, *y_dev = scratch + x_bytes;
    // Nothing in the scratch has to start at zero: the copy overwrites all of X's staging and the
    // kernel writes every element of Y's before the copy back reads it.
    Q4B_CUDA_TRY(cudaMemcpyAsync(x_dev, x_host, (size_t)M * K * 2, cudaMemcpyHostToDevice, st));
    int rc = q4b_matmul(x_dev, x_dtype, M, K, prepacked, K, N, y_dev, N, Q4B_FLAG_NONE, stream);
    if (rc != Q4B_OK) return rc;
    Q4B_CUDA_TRY(cudaMemcpyAsync(y_host, y_dev, (size_t)M * N * 2, cudaMemcpyDeviceToHost, st));
    return Q4B_OK;
}

// ---------------------------------------------------------------------------------------------
// q4b_selftest_wait_timeout: makes a bounded wait run out without harming anything.  One warp
// initialises a shared-memory barrier that nobody will ever arrive at and waits on it with the
// kernels' own bounded wait (ptx::mbar_wait) and a limit of `limit_cycles`; the wait gives up,
// records code 900 and the kernel returns.  q4b_wait_status then reports Q4B_ERR_TIMEOUT / 900.
// ---------------------------------------------------------------------------------------------
namespace q4b {

__device__ int g_selftest_status = 0;

__global__ void selftest_wait_kernel(long long limit_cycles) {
    __shared__ __align__(8) unsigned long long bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        ptx::mbar_init(ptx::smem_u32(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    ptx::mbar_wait(ptx::smem_u32(&bar), 0, &abort_flag, &g_selftest_status, 900, limit_cycles);
}

int selftest_wait_status(int *value) {
    int h = 0;
    Q4B_CUDA_TRY(cudaMemcpyFromSymbol(&h, g_selftest_status, sizeof(int)));
    if (h != 0) {
        const int zero = 0;
        Q4B_CUDA_TRY(cudaMemcpyToSymbol(g_selftest_status, &zero, sizeof(int)));
    }
    *value = h;
    return Q4B_OK;
}

}  // namespace q4b

extern "C" int q4b_selftest_wait_timeout(int64_t limit_cycles, void *stream) {
    if (limit_cycles < 1 || limit_cycles > (1LL << 24)) return Q4B_ERR_ARG;      // at most ~10 ms
    selftest_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((long long)limit_cycles);
    Q4B_LAUNCH_CHECK();
    return Q4B_OK;
}
