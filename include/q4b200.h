/*
 * q4b200 — C ABI of the B200 (sm_100a) block_q4_0 INT4 matmul library.
 *
 * This is the boundary a host binding loads instead of metalcore's pybind11 extension
 * `metalcore_backend` (packages/metalcore/src/metalcore/native/core_mps.mm:6866-6952) for
 * the q4_0 path.  Plain pointers and sizes only; every pointer is a DEVICE pointer unless the
 * name says host.  All calls are asynchronous on the given stream (a cudaStream_t passed as
 * void*; NULL = the legacy default stream), never synchronise, never allocate device memory
 * and return 0 or a q4b_status code.  The device used is the calling thread's current device.
 *
 * Tensor layouts
 *   blocks     uint8 [K/32, N, 18]  interchange format, bit-exact with the reference's
 *              quantize_ggml_q4_0 (quantization.py:307-371): fp16 scale d (little endian),
 *              then 16 bytes, byte j = q[2j] | q[2j+1] << 4.
 *   prepacked  uint8 [ceil(N/16), ceil(K/64), 576]  internal streaming format, one 576-byte
 *              tile per 16 output columns x 64 k, column-tile-major (all k tiles of a column
 *              tile are contiguous).  Same information as `blocks` (18 bytes per 32 weights),
 *              rearranged so that a lane's mma fragment is one 128-bit word plus one 64-bit
 *              word of scales.  q4b_prepacked_bytes gives its size; the buffer must be
 *              16-byte aligned.  Tile layout:
 *                bytes [0,512): 32 slots of 16 bytes; the slot of column-in-octet g (0..7) and
 *                  k-octet c (0..3) is p = (g/2)*8 + (g%2)*4 + (c ^ (g/2)) and holds four
 *                  32-bit words: blocks (kb0,g),(kb0,g+8),(kb0+1,g),(kb0+1,g+8), each word =
 *                  the 8 nibbles q[8c..8c+7] of that block
 *                  stored as q0|q2<<4|q4<<8|q6<<12|q1<<16|q3<<20|q5<<24|q7<<28;
 *                bytes [512,576): 8 rows g of four fp16 scales d(kb0,g), d(kb0,g+8),
 *                  d(kb0+1,g), d(kb0+1,g+8).
 *              Padding blocks (k >= K or n >= N) have d = 0 and q = 8.
 */
#ifndef Q4B200_H
#define Q4B200_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define Q4B_API __attribute__((visibility("default")))
#else
#define Q4B_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    Q4B_OK = 0,
    Q4B_ERR_ARG = 1,      /* null pointer, negative size, unknown enum value            */
    Q4B_ERR_SHAPE = 2,    /* K not a multiple of 32, size beyond the supported range    */
    Q4B_ERR_DTYPE = 3,    /* dtype not supported by this entry point                    */
    Q4B_ERR_ALIGN = 4,    /* pointer or leading dimension not aligned as documented     */
    Q4B_ERR_ARCH = 5,     /* current device is not compute capability 10.x              */
    Q4B_ERR_CUDA = 6,     /* a CUDA runtime call failed; see q4b_last_cuda_error        */
    Q4B_ERR_TIMEOUT = 7,  /* a bounded device-side wait gave up (read via q4b_wait_status) */
    Q4B_ERR_TOO_LARGE = 8 /* problem exceeds a fixed internal buffer                    */
} q4b_status;

typedef enum { Q4B_F32 = 0, Q4B_F16 = 1, Q4B_BF16 = 2 } q4b_dtype;

/* layout of the floating-point weight given to q4b_quantize */
typedef enum {
    Q4B_LAYOUT_KN = 0,    /* [K, N], N contiguous: the reference's quantize_ggml_q4_0 input */
    Q4B_LAYOUT_NK = 1     /* [N, K], K contiguous: torch.nn.Linear.weight as stored         */
} q4b_layout;

/* flags for the matmul entry points */
enum {
    Q4B_FLAG_NONE = 0,
    /* Launch with programmatic dependent launch: the kernel may start fetching WEIGHTS while
     * earlier work on the stream is still running, and waits for that work before it reads x
     * or writes y.  Only valid when nothing still in flight on the stream writes `prepacked`. */
    Q4B_FLAG_PDL = 1,
    /* bits 2 and 4 are not used */
    /* Activation applied to the fp32 result (after the addend, before the one rounding), as the
     * reference's fused kernels matmul_int4_silu / matmul_int4_gelu do (quant_kernels.metal:880-1144):
     * SiLU v / (1 + exp(-v)), or GELU in its tanh form.  At most one of the two. */
    Q4B_FLAG_ACT_SILU = 8,
    Q4B_FLAG_ACT_GELU = 16
};

Q4B_API const char *q4b_strerror(int status);
/* text of the last CUDA runtime error seen by this thread inside the library ("" if none) */
Q4B_API const char *q4b_last_cuda_error(void);
Q4B_API int q4b_version(void);
/* Q4B_OK when the current device can run the kernels (compute capability 10.x) */
Q4B_API int q4b_device_ok(void);

/* bytes of the prepacked buffer for a [K, N] weight; 0 if K is not a multiple of 32 */
Q4B_API size_t q4b_prepacked_bytes(int64_t K, int64_t N);

/*
 * Quantize + pack.  Replaces the torch pipeline of quantize_ggml_q4_0
 * (quantization.py:307-371; the reference has no native kernel for it).  `w` is [K, N] or
 * [N, K] per `layout`, dense (leading dimension = inner extent), dtype f32 / f16 / bf16; the
 * arithmetic rounds after every step in that dtype exactly as the reference's torch ops do,
 * so `blocks_out` is bit-identical to the reference.  Either output may be NULL.
 */
Q4B_API int q4b_quantize(const void *w, int w_dtype, int64_t K, int64_t N, int layout,
                 void *blocks_out, void *prepacked_out, void *stream);

/* interchange blocks -> prepacked tiles, and back (both exact, no arithmetic) */
Q4B_API int q4b_repack(const void *blocks, int64_t K, int64_t N, void *prepacked_out, void *stream);
Q4B_API int q4b_unpack(const void *prepacked, int64_t K, int64_t N, void *blocks_out, void *stream);

/*
 * blocks -> dense W [K, N] of out_dtype: W = (q - 8) * float(d) in fp32, then cast.
 * Replaces dequantize_ggml_q4_0 (quantization.py:374-419).
 */
Q4B_API int q4b_dequantize(const void *blocks, int64_t K, int64_t N, void *w_out, int out_dtype,
                   void *stream);

/*
 * Y[M, N] = X[M, K] . dequant(W), fp32 accumulation, Y of the same dtype as X (f16 or bf16).
 * Replaces matmul_ggml_q4_0_metal (core_mps.mm:5917-5975) and the Metal kernel
 * matmul_ggml_q4_0 (quant_kernels.metal:1738-1886).  X rows are K contiguous elements with
 * leading dimension ldx (elements, multiple of 8, X 16-byte aligned); Y has leading
 * dimension ldy (elements).
 *
 *   q4b_gemv   decode path, 1 <= M <= 16: streams the prepacked tiles once (bulk asynchronous
 *              copies into per-warp rings, 128-bit reads), dequantises in registers,
 *              warp-level mma + split-K reduction in the CTA.
 *   q4b_gemm   prefill path, any M >= 1 (intended for M >= 17): the packed weights are
 *              dequantised to bf16/fp16 straight into tensor memory and are the A operand of
 *              tcgen05.mma, X tiles arrive by TMA, accumulators in tensor memory.  Up to 128
 *              rows a CTA per 128-column panel and k range; above, persistent CTAs over items
 *              of 128 columns x up to 256 rows.
 *   q4b_matmul picks q4b_gemv for M <= 8, and for 9 <= M <= 16 when the weight has fewer than
 *              2^25 elements; otherwise q4b_gemm.
 * A flags word with both activation bits set is rejected with Q4B_ERR_ARG.
 */
Q4B_API int q4b_gemv(const void *x, int x_dtype, int64_t M, int64_t ldx, const void *prepacked,
             int64_t K, int64_t N, void *y, int64_t ldy, int flags, void *stream);
Q4B_API int q4b_gemm(const void *x, int x_dtype, int64_t M, int64_t ldx, const void *prepacked,
             int64_t K, int64_t N, void *y, int64_t ldy, int flags, void *stream);
Q4B_API int q4b_matmul(const void *x, int x_dtype, int64_t M, int64_t ldx, const void *prepacked,
               int64_t K, int64_t N, void *y, int64_t ldy, int flags, void *stream);

/*
 * The same products with an optional fp32 term added before the single rounding to the output
 * dtype: Y = round(X . dequant(W) + addend), addend [M, N] fp32 with leading dimension ld_add
 * (NULL = none; ld_add = 0: one row of N values added to every row, i.e. a bias).  Used for the group-wise format's zero-point term and for a fused bias
 * (the reference adds its bias after the matmul, quantization.py:602-603).
 */
Q4B_API int q4b_gemv_addend(const void *x, int x_dtype, int64_t M, int64_t ldx, const void *prepacked,
                            int64_t K, int64_t N, const float *addend, int64_t ld_add, void *y,
                            int64_t ldy, int flags, void *stream);
Q4B_API int q4b_gemm_addend(const void *x, int x_dtype, int64_t M, int64_t ldx, const void *prepacked,
                            int64_t K, int64_t N, const float *addend, int64_t ld_add, void *y,
                            int64_t ldy, int flags, void *stream);
Q4B_API int q4b_matmul_addend(const void *x, int x_dtype, int64_t M, int64_t ldx,
                              const void *prepacked, int64_t K, int64_t N, const float *addend,
                              int64_t ld_add, void *y, int64_t ldy, int flags, void *stream);
/* The same product forced onto the persistent prefill kernel (items of 128 columns x up to 256 rows x
 * all of k; any M >= 1), which q4b_gemm_addend uses above 128 rows. */
Q4B_API int q4b_gemm_wt_addend(const void *x, int x_dtype, int64_t M, int64_t ldx, const void *prepacked,
                               int64_t K, int64_t N, const float *addend, int64_t ld_add, void *y,
                               int64_t ldy, int flags, void *stream);

/*
 * Group-wise asymmetric INT4 format of the reference (quantization.py:26-239; its Metal
 * quantizer quantize_to_int4, quant_kernels.metal:634-690 / core_mps.mm:4655-4705, and matmul
 * dispatcher matmul_int4_metal, core_mps.mm:5612-5776):
 *   packed uint8 [K/2, N] (byte r of column n = q[2r] | q[2r+1] << 4), scales and zeros
 *   [ceil(K/group), N] in the weight's dtype, W = (q - zero) * scale.
 *
 * q4b_int4g_quantize    bit-exact with quantize_int4: per (group, column) min/max,
 *                       scale = max((max-min)/15, 1e-8), zero = -min/scale,
 *                       q = clamp(round(w/scale + zero), 0, 15), every step rounded in w's dtype.
 *                       K and group even.  scales/zeros are written in w's dtype.
 * q4b_int4g_dequantize  ((q - zero) * scale) in fp32, cast to out_dtype (dequantize_int4).
 * q4b_int4g_prepack     converts to the streaming tile layout used by the matmul kernels
 *                       (block scale d = fp16(scale), needs group % 32 == 0 and K % 32 == 0) and
 *                       writes corr [ceil(K/group), N] fp32 = 8*d - zero*scale, the per-group
 *                       constant that the symmetric tiles leave out.
 *                       A scale outside fp16's range cannot be a block scale: the kernel notes it
 *                       and q4b_int4g_prepack_status (which synchronises the stream) reports it.
 * q4b_int4g_addend      addend[m, n] = sum_g corr[g, n] * sum_{k in g} x[m, k] + bias[n]  (fp32
 *                       [M, N]; bias fp32 [N] or NULL), to be passed to q4b_matmul_addend with the
 *                       prepacked tiles.  Any M.  rowsums_ws: q4b_int4g_rowsums_bytes(M, K, group)
 *                       bytes of device memory (the rows' group sums, [M, ceil(K/group)] fp32),
 *                       written by a first kernel and read by the second.
 * q4b_int4g_matmul_generic  the same product straight from the [K/2, N] format for the shapes the
 *                       streaming tiles do not cover (K or group not a multiple of 32), as the
 *                       reference's Python loop accepts them (quantization.py:207-239): fp32
 *                       accumulation on the CUDA cores, any even K, any group.
 */
Q4B_API int q4b_int4g_quantize(const void *w, int w_dtype, int64_t K, int64_t N, int64_t group,
                               void *packed_out, void *scales_out, void *zeros_out, void *stream);
Q4B_API int q4b_int4g_dequantize(const void *packed, const void *scales, const void *zeros,
                                 int sz_dtype, int64_t K, int64_t N, int64_t group, void *w_out,
                                 int out_dtype, void *stream);
Q4B_API int q4b_int4g_prepack(const void *packed, const void *scales, const void *zeros,
                              int sz_dtype, int64_t K, int64_t N, int64_t group,
                              void *prepacked_out, float *corr_out, void *stream);
Q4B_API int q4b_int4g_prepack_status(void *stream, int *out_of_range);
Q4B_API size_t q4b_int4g_rowsums_bytes(int64_t M, int64_t K, int64_t group);
Q4B_API int q4b_int4g_addend(const void *x, int x_dtype, int64_t M, int64_t ldx, const float *corr,
                             const float *bias, int64_t K, int64_t N, int64_t group, float *rowsums_ws,
                             float *addend_out, void *stream);
/*
 * The zero-point term folded into the contraction of the tensor-core kernels (those behind q4b_gemm,
 * picked by M in the same way): instead of an [M, N] fp32 addend, KX = q4b_int4g_fold_ktiles(K, group) further k-tiles multiply
 *   fold_rows    [M, 64 KX] bf16, from X per call (q4b_int4g_fold_rows: the rows' group sums), by
 *   fold_operand [N, 64 KX] bf16, from corr once per weight (q4b_int4g_fold_operand).
 * Both factors are split into three bf16 terms and the six largest products kept, so the term keeps
 * fp32-like accuracy (what is dropped is below 2^-24 of it).  q4b_int4g_gemm_fold runs the product;
 * bias is one fp32 row of N values or NULL.
 */
Q4B_API int q4b_int4g_fold_ktiles(int64_t K, int64_t group);
Q4B_API int q4b_int4g_fold_operand(const float *corr, int64_t K, int64_t N, int64_t group, void *operand_out,
                                   void *stream);
Q4B_API int q4b_int4g_fold_rows(const void *x, int x_dtype, int64_t M, int64_t ldx, int64_t K, int64_t group,
                                void *rows_out, void *stream);
Q4B_API int q4b_int4g_gemm_fold(const void *x, int x_dtype, int64_t M, int64_t ldx, const void *prepacked,
                                int64_t K, int64_t N, const void *fold_operand, const void *fold_rows, int KX,
                                const float *bias, void *y, int64_t ldy, int flags, void *stream);
/*
 * Up to 16 rows (the decode kernels): q4b_int4g_rowsums writes the rows' group sums [M, ceil(K/group)] fp32
 * (q4b_int4g_rowsums_bytes), and q4b_int4g_gemv forms sum_g corr[g, n] * rowsums[m, g] in its epilogue,
 * in fp32, before the one rounding; bias is one fp32 row of N values or NULL.
 */
Q4B_API int q4b_int4g_rowsums(const void *x, int x_dtype, int64_t M, int64_t ldx, int64_t K, int64_t group,
                              float *rowsums_out, void *stream);
Q4B_API int q4b_int4g_gemv(const void *x, int x_dtype, int64_t M, int64_t ldx, const void *prepacked, int64_t K,
                           int64_t N, const float *corr, const float *rowsums, int64_t group, const float *bias,
                           void *y, int64_t ldy, int flags, void *stream);
Q4B_API int q4b_int4g_matmul_generic(const void *x, int x_dtype, int64_t M, int64_t ldx,
                                     const void *packed, const void *scales, const void *zeros,
                                     int sz_dtype, int64_t K, int64_t N, int64_t group, void *y,
                                     int64_t ldy, void *stream);

/*
 * Weights from other GGML tools, and the reference's group-wise INT8 weights.
 *
 * q4b_import_ggml    block_q4_0 data as those tools store it: rows of K/32 blocks per output
 *                    feature, [N, K/32, 18], byte j of a block = value j | value (j + 16) << 4 (the
 *                    order the reference's own helper reads, quant_kernels.metal:1714-1731; format
 *                    provenance quantization.py:292-304)  ->  this library's blocks [K/32, N, 18].
 * q4b_quantize_ggml  quantizes with those tools' scale rule instead of the reference's amax / 7:
 *                    d = (value of largest magnitude in the block) / -8, q = clamp(round(w / d) + 8,
 *                    0, 15), all-zero block: d = 0, q = 8; fp32 arithmetic, ties to even.  Writes
 *                    blocks (required) and optionally the streaming layout.  The matmul kernels
 *                    accept either rule (negative d included).
 * q4b_int8g_matmul   Y = X . ((w_q - zero) * scale) for int8 w_q [K, N] and scales / zeros
 *                    [ceil(K/group), N] of dtype sz_dtype: matmul_int8 of the reference
 *                    (quantization.py:242-286, quant_kernels.metal:40-109, core_mps.mm:4516-4574).
 *                    fp32 accumulation on the CUDA cores, X and Y f16 or bf16; any M (tiled eight
 *                    rows at a time), w_int8 4-byte aligned.
 */
Q4B_API int q4b_import_ggml(const void *raw, int64_t K, int64_t N, void *blocks_out, void *stream);
Q4B_API int q4b_quantize_ggml(const void *w, int w_dtype, int64_t K, int64_t N, int layout,
                              void *blocks_out, void *prepacked_out, void *stream);
Q4B_API int q4b_int8g_matmul(const void *x, int x_dtype, int64_t M, int64_t ldx, const void *w_int8,
                             const void *scales, const void *zeros, int sz_dtype, int64_t K, int64_t N,
                             int64_t group, void *y, int64_t ldy, void *stream);

/*
 * Single-row decode (M = 1) over a list of stages in ONE persistent launch (no reference
 * counterpart: the reference launches its 64x32-tile kernel once per product,
 * core_mps.mm:5917-5975, quant_kernels.metal:1738-1886).
 *
 * A stage is 1..Q4B_CHAIN_MAX_PRODUCTS products that share one input row of K elements
 * (q|k|v, gate|up):  y_p = act(alpha_p * (x . dequant(W_p)) + addend_p).  Its input is either a
 * device pointer whose contents are ready when the launch starts (x != NULL), or the output of an
 * EARLIER stage's product (x == NULL; x_stage, x_product), optionally transformed on the way in:
 * Q4B_CHAIN_X_SILU_MUL takes x = silu(a) * b from two earlier outputs (the gated MLP).  Outputs
 * are always also written to y for the caller.
 *
 * Arithmetic: x is held as 15-bit fixed point per 32-k block (scale max|x|/16383), the dot
 * product with the 4-bit weights is exact in int32 on the tensor cores (mma.sync s8), scales are
 * applied in fp32, fixed summation order (bitwise repeatable); relative error about 1e-4.
 *
 *   q4b_gemv_grouped           one stage, input in plain memory, no workspace.
 *   q4b_chain_workspace_bytes  size of the device workspace of a chain (0 on bad arguments).
 *   q4b_chain_build            validates the list, writes the device-side work list and the
 *                              hand-over buffers into `workspace` (256-byte aligned) and waits for
 *                              its copies; do it once, outside any stream capture.
 *   q4b_chain_run              one launch over the whole list; n_stages, x_dtype (f16/bf16, of
 *                              every input and output) and max_k (largest K of the list) as
 *                              given to the build.  Launches of one workspace must not overlap on
 *                              the GPU; weights, outputs and addends must stay where they were.
 * K a multiple of 32 and at most about 32768 (the input row must fit in shared memory,
 * Q4B_ERR_TOO_LARGE beyond).  Hand-over waits are bounded like every other wait (q4b_wait_status
 * codes 500-502).
 */
#define Q4B_CHAIN_MAX_PRODUCTS 4
#define Q4B_CHAIN_MAX_STAGES 256
enum { Q4B_CHAIN_X_PLAIN = 0, Q4B_CHAIN_X_SILU_MUL = 1 };
typedef struct {
    const void *prepacked;  /* [K, N] weights in the streaming layout                        */
    void *y;                /* [N] output, dtype of the chain                                 */
    const float *addend;    /* optional fp32 [N] added before the rounding (bias), or NULL   */
    int64_t N;
    float alpha;            /* scale of the product, applied in fp32                          */
    int flags;              /* Q4B_FLAG_ACT_SILU / Q4B_FLAG_ACT_GELU or 0                     */
} q4b_chain_product;
typedef struct {
    const void *x;          /* [K] input in device memory, or NULL: taken from an earlier stage */
    int x_stage, x_product; /* with x == NULL: which earlier output is the input              */
    int x_stage2, x_product2; /* with Q4B_CHAIN_X_SILU_MUL: the second operand b              */
    int xform;              /* Q4B_CHAIN_X_*                                                  */
    int n_products;
    int64_t K;
    q4b_chain_product products[Q4B_CHAIN_MAX_PRODUCTS];
} q4b_chain_stage;
Q4B_API int q4b_gemv_grouped(const void *x, int x_dtype, int64_t K, const q4b_chain_product *products,
                             int n_products, int flags, void *stream);
Q4B_API size_t q4b_chain_workspace_bytes(const q4b_chain_stage *stages, int n_stages);
Q4B_API int q4b_chain_build(const q4b_chain_stage *stages, int n_stages, void *workspace,
                            size_t workspace_bytes, void *stream);
Q4B_API int q4b_chain_run(const void *workspace, int n_stages, int x_dtype, int64_t max_k, int flags,
                          void *stream);

/*
 * Decode product with a fused all-gather (column-parallel layers over several GPUs of one box; no
 * reference counterpart, the reference is single-device): q4b_gemv, but each rank's kernel stores
 * its [M, N] result at column offset col0 of the [M, ld_out] output of EVERY rank, through
 * peer-mapped device pointers y_ranks[0..world-1] (a HOST array; plain stores over NVLink), instead
 * of into a local y.  The caller provides the peer mapping (e.g. torch symmetric memory) and the
 * barrier after which the gathered outputs may be read.  1 <= M <= 16, world <= 8.
 */
Q4B_API int q4b_gemv_gather(const void *x, int x_dtype, int64_t M, int64_t ldx,
                            const void *prepacked, int64_t K, int64_t N, void *const *y_ranks,
                            int world, int64_t col0, int64_t ld_out, int flags, void *stream);
/*
 * The same gather without barriers: the peers' buffers are uint32 [rows, ld_out] and every store carries
 * the call's epoch (1..65535) in its upper half, so each word validates itself.  q4b_gather_ll_unpack, on
 * every rank, waits word by word (bounded; q4b_wait_status code 700) for the epoch and writes the plain
 * values; with slots > 1 it adds the `slots` partial results that sit side by side in a row (fp32, slot
 * order, one rounding): the reduction of a row-parallel layer.  Alternate between two buffers from call
 * to call: stream order then guarantees that nobody still reads the buffer being overwritten.
 */
Q4B_API int q4b_gemv_gather_ll(const void *x, int x_dtype, int64_t M, int64_t ldx, const void *prepacked,
                               int64_t K, int64_t N, void *const *ll_ranks, int world, int64_t col0,
                               int64_t ld_out, int epoch, int flags, void *stream);
Q4B_API int q4b_gather_ll_unpack(const void *ll, int64_t rows, int64_t cols, int64_t ld_ll, int slots, int epoch,
                                 int x_dtype, void *out, int64_t ld_out, void *stream);
/* both steps in one call: the product stored into every rank's words, then this rank's wait-and-unpack of
 * its own buffer ll_local into out (slots == 1: gather, out [M, ld_out]; slots > 1: sum of the partial
 * results, ld_out = slots * N, out [M, N]) */
Q4B_API int q4b_gemv_exchange(const void *x, int x_dtype, int64_t M, int64_t ldx, const void *prepacked, int64_t K,
                              int64_t N, void *const *ll_ranks, int world, int64_t col0, int64_t ld_out,
                              const void *ll_local, int slots, int epoch, void *out, int64_t ld_y, int flags,
                              void *stream);
/* The same with the call counter in device memory, so that nothing changes on the host from call to call
 * and a captured launch can be replayed: ctl points at two ints (zero at set-up, one pair per rank), call c
 * uses epoch c % 65535 + 1 and the buffer of parity c & 1; a rank's two buffers are ll_half words apart and
 * ll_ranks / ll_local point at the first.  The unpack kernel sets the words it read back to zero (nothing
 * stale survives a call) and its last block increments the counter. */
Q4B_API int q4b_gemv_exchange_dev(const void *x, int x_dtype, int64_t M, int64_t ldx, const void *prepacked,
                                  int64_t K, int64_t N, void *const *ll_ranks, int world, int64_t col0,
                                  int64_t ld_out, void *ll_local, int64_t ll_half, int slots, int *ctl, void *out,
                                  int64_t ld_y, int flags, void *stream);

/*
 * RMSNorm in front of a quantised linear layer, the first step of the reference's
 * fused_rmsnorm_linear_int4 (core_mps.mm:3017-3103; kernel training_kernels.metal:425-485):
 * y[m, :] = T(float(x[m, :]) * rsqrt(mean(x[m, :]^2) + eps) * float(weight[:])), sums in fp32.
 * x, weight and y share `dtype` (Q4B_F16 or Q4B_BF16); y may not alias x.
 */
Q4B_API int q4b_rmsnorm(const void *x, int dtype, int64_t M, int64_t K, int64_t ldx,
                        const void *weight, float eps, void *y, int64_t ldy, void *stream);

/*
 * The matmul kernels bound every mbarrier wait; a wait that gives up makes the kernel set a
 * status word on the device and stop early (its output is then incomplete).  This call
 * synchronises the stream, reads that word and clears it: Q4B_OK, or Q4B_ERR_TIMEOUT with
 * *detail (may be NULL) = which wait gave up (100-101 decode kernels, 401-407 small-batch
 * tensor-memory kernel, 500-504 persistent single-row kernel, 601-608 persistent prefill kernel,
 * 700 barrier-free gather, 900 self-test).
 * It never traps or faults the device.
 */
Q4B_API int q4b_wait_status(void *stream, int *detail);
/*
 * Launches a one-warp kernel whose bounded wait (the kernels' own wait routine, on a barrier
 * nobody arrives at) runs out after `limit_cycles` (1 .. 2^24) and returns: q4b_wait_status then
 * reports Q4B_ERR_TIMEOUT with detail 900.  For testing the error path; nothing faults or hangs.
 */
Q4B_API int q4b_selftest_wait_timeout(int64_t limit_cycles, void *stream);

/*
 * Host-buffer convenience used for end-to-end timing: x_host and y_host are (ideally pinned)
 * HOST pointers; x_dev / y_dev are caller-provided device staging buffers of M*K and M*N
 * elements.  Enqueues H2D copy of X, q4b_matmul, D2H copy of Y on `stream`.
 */
Q4B_API int q4b_matmul_host(const void *x_host, void *x_dev, int x_dtype, int64_t M,
                    const void *prepacked, int64_t K, int64_t N, void *y_dev, void *y_host,
                    int flags, void *stream);

/*
 * Host-buffer product for callers that cannot allocate device memory.  (This entry point has no
 * counterpart in the reference: metalcore always lets its extension allocate.)
 *
 * Who needs it: code that runs where cudaMalloc is forbidden or unaffordable — a plugin called
 * inside somebody else's real-time or inference loop that must not touch the allocator, a host
 * that has handed all device memory to one arena and gives none back, a process that may not
 * take the allocator's device-wide lock.  q4b_matmul_host asks such a caller for two device
 * staging buffers; here they come out of a fixed array that is part of the library image.
 *
 * x_host [M, K] and y_host [M, N] are HOST pointers (dense, x_dtype f16 or bf16), `prepacked` is
 * the usual device pointer.  Enqueues H2D copy of X, q4b_matmul, D2H copy of Y on `stream`.
 *
 * Limits and rules:
 *   - round_up(M*K*2, 256) + round_up(M*N*2, 256) must not exceed Q4B_NOALLOC_MAX_BYTES, else
 *     the call returns Q4B_ERR_TOO_LARGE and enqueues nothing.  Every GPU on which the library
 *     is loaded holds those Q4B_NOALLOC_MAX_BYTES of global memory until the process exits.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress,
 *     with that device current) and keeps it; make that first call outside any stream capture.
 *   - All calls on a device share the one array, and it keeps the previous call's bytes.
 *     Nothing in it needs clearing (X's part is overwritten whole, Y's part is written whole
 *     before it is read), but two calls whose work overlaps on the GPU — different streams, or
 *     different host threads — race on it.  Serialise them on one stream.
 *   - No cudaMalloc, cudaFree or allocating library routine is called, on any call.
 */
#define Q4B_NOALLOC_MAX_BYTES (4u << 20)
Q4B_API int q4b_matmul_host_noalloc(const void *x_host, int x_dtype, int64_t M,
                                    const void *prepacked, int64_t K, int64_t N, void *y_host,
                                    void *stream);

#ifdef __cplusplus
}
#endif
#endif /* Q4B200_H */
