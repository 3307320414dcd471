/*
 * C ABI of the B200 (sm_100a) matrix-multiply-accumulate library.
 *
 * rocWMMA itself is a header-only C++ device library: its drop-in boundary is
 * the source-level API under include/rocwmma/.  What a host program links
 * against are the kernels built on that API; this header declares their
 * launchers.  Each entry point cites the reference kernel or host routine whose
 * calling convention it follows (paths inside the rocWMMA source tree).
 *
 * Conventions shared by every entry point
 *   - plain pointers and sizes only; device pointers are owned by the caller and
 *     are neither retained nor freed;
 *   - `stream` is a cudaStream_t passed as void* (NULL = default stream); calls
 *     are asynchronous with respect to the host unless stated otherwise;
 *   - the return value is B200WMMA_OK or a negative B200WMMA_ERR_* code; nothing
 *     ever calls exit() (the reference samples do: samples/common.hpp:34-46);
 *   - there is no CPU fallback: without a CUDA device every compute entry point
 *     returns B200WMMA_ERR_CUDA.
 */
#ifndef ROCWMMA_B200_C_API_H
#define ROCWMMA_B200_C_API_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define B200WMMA_API __attribute__((visibility("default")))
#else
#define B200WMMA_API
#endif

/* Element types (rocWMMA docs/api-reference/api-reference-guide.rst:80-153). */
enum b200wmma_dtype
{
    B200WMMA_F16  = 0, /* float16_t                                     */
    B200WMMA_BF16 = 1, /* bfloat16_t                                    */
    B200WMMA_E4M3 = 2, /* float8_t, OCP e4m3                            */
    B200WMMA_I8   = 3, /* int8_t                                        */
    B200WMMA_F32  = 4, /* float32_t, full fp32 products                 */
    B200WMMA_XF32 = 5, /* xfloat32_t: fp32 storage, low 13 bits zero    */
    B200WMMA_F64  = 6, /* float64_t                                     */
    B200WMMA_I32  = 7, /* int32_t (outputs of int8 GEMM)                */
    B200WMMA_E5M2 = 8  /* bfloat8_t, OCP e5m2                           */
};

/* Memory layouts (rocwmma.hpp:74-81, 106-110). */
enum b200wmma_layout
{
    B200WMMA_ROW_MAJOR = 0,
    B200WMMA_COL_MAJOR = 1
};

enum b200wmma_status
{
    B200WMMA_OK               = 0,
    B200WMMA_ERR_INVALID_ARG  = -1, /* null pointer, zero or indivisible size          */
    B200WMMA_ERR_UNSUPPORTED  = -2, /* type / layout combination not built             */
    B200WMMA_ERR_ALIGNMENT    = -3, /* pointer or leading dimension not 16-byte aligned */
    B200WMMA_ERR_CUDA         = -4, /* a CUDA runtime or driver call failed            */
    B200WMMA_ERR_DEVICE_WAIT  = -5, /* a bounded wait inside a kernel ran out          */
    B200WMMA_ERR_TOO_LARGE    = -6  /* size beyond a documented maximum                */
};

B200WMMA_API int         b200wmma_version(void);
B200WMMA_API const char* b200wmma_status_string(int status);

/*
 * D = alpha * A * B + beta * C with ONE fragment tile per warp, written on the
 * per-warp fragment API exactly like the reference's simple GEMM samples
 * (kernel: samples/simple_hgemm.cpp:81-139, simple_sgemm.cpp:81, simple_dgemm.cpp:81;
 * argument order: test/gemm/gemm_kernel_base.hpp:102-114).
 * A is m x k, B is k x n, C and D are m x n and share `layout_cd`.
 * `block` selects the fragment shape: 16 -> 16x16x16, 32 -> 32x32x16
 * (32x32x32 for 8-bit inputs).  m and n must be multiples of `block`, k of the
 * fragment's BlockK.  Type pairs (in -> out): F16->F32, F16->F16, BF16->F32,
 * BF16->BF16, E4M3->F32, I8->I32, F32->F32, XF32->F32, F64->F64.
 * alpha and beta are converted to the compute type (int32 for I8).
 */
B200WMMA_API int b200wmma_gemm_simple(int in_dtype, int out_dtype, uint32_t m, uint32_t n, uint32_t k,
                         const void* a, const void* b, const void* c, void* d, uint32_t lda,
                         uint32_t ldb, uint32_t ldc, uint32_t ldd, double alpha, double beta,
                         int layout_a, int layout_b, int layout_cd, int block, void* stream);

/*
 * The same kernel for a full rocWMMA type triple Ti / To / Tc
 * (docs/api-reference/api-reference-guide.rst:80-153; the reference's test kernels take
 * the compute type and BlockK as template parameters, test/gemm/gemm_kernel_base.hpp:57-75).
 * compute_dtype is the type of the accumulator fragment, of alpha and beta and of the
 * scaling arithmetic; a negative value selects the usual one (F32; I32 for I8; F64 for
 * F64), which makes the call identical to b200wmma_gemm_simple.  Besides the triples of
 * b200wmma_gemm_simple: F16/F16/F16 (tensor-core fp16 accumulation), BF16/BF16/BF16
 * (accumulator fragment rounded to bf16 after every BlockK step, as rocWMMA does for
 * 16-bit compute types, internal/mfma_impl.hpp:101-156), I8/I8/I32, E5M2/F32/F32.
 * block_k is the K extent of the A and B fragments: 0 for the usual one (16; 32 for 8-bit
 * types in 32 x 32 tiles), else 8 (16-bit types only: the reference's minimum for 32 x 32
 * blocks, test/gemm/gemm_predicates_base.hpp:137-209), 16, 32 or 64 for 8- and 16-bit types
 * (128 too with 16 x 16 tiles), 4, 8 or 32 for F32 / XF32, 4 or 8 for F64; k must be a
 * multiple of it.  Fragments whose BlockK is below the K extent of the full-depth tensor-core
 * instruction run on its half-depth form (m16n8k8 for 16-bit, m16n8k4 for tf32).
 */
B200WMMA_API int b200wmma_gemm_simple_ex(int in_dtype, int out_dtype, int compute_dtype, uint32_t m,
                            uint32_t n, uint32_t k, const void* a, const void* b, const void* c,
                            void* d, uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd,
                            double alpha, double beta, int layout_a, int layout_b, int layout_cd,
                            int block, int block_k, void* stream);

/*
 * D = alpha * A * B + beta * C through the block-cooperative path: TMA-staged
 * shared-memory ring, tcgen05.mma with accumulators in tensor memory, persistent
 * tiles.  Takes the place of the reference's macro-tile GEMM
 * (samples/perf_hgemm.cpp:518-714, perf_sgemm.cpp:472, perf_dgemm.cpp:464; same
 * argument order as above).  C and D are row-major.  When beta == 0, c may be
 * NULL and is never read.  Type pairs: F16->F16, F16->F32, BF16->F32, BF16->BF16,
 * XF32->F32, F32->F32, I8->I32, E4M3->BF16, E4M3->F32, E5M2->BF16, E5M2->F32; F64->F64 runs on the warp-level
 * double-precision tensor path with a shared-memory pipeline.
 * Requirements: a, b, c, d 16-byte aligned; lda, ldb, ldc, ldd times the element
 * size multiples of 16 bytes.  Any m, n, k >= 1 (edge tiles are zero-filled on
 * load and masked on store).  Every layout combination of A and B is read in
 * place (row-major A / column-major B as K-major tensor-core operands,
 * column-major A / row-major B as MN-major ones), except for 32- and 64-bit
 * inputs (XF32, F64): those transpose column-major A / row-major B into a
 * per-device scratch buffer first (allocated on first use, grown on demand; such
 * calls on different streams of one device must not overlap).  F32->F32 (the reference's
 * perf_sgemm: full fp32 products) runs as three TF32 products over split copies
 * (hi + lo) of A and B, which also live in that scratch buffer (2 (m + n) k floats), for every
 * layout; its A and B need no 16-byte alignment.  The first call on a device allocates a few
 * bytes of status memory.
 */
B200WMMA_API int b200wmma_gemm(int in_dtype, int out_dtype, uint32_t m, uint32_t n, uint32_t k, const void* a,
                  const void* b, const void* c, void* d, uint32_t lda, uint32_t ldb, uint32_t ldc,
                  uint32_t ldd, double alpha, double beta, int layout_a, int layout_b,
                  void* stream);

/*
 * Same computation with HOST buffers: copies A, B (and C when beta != 0) to the
 * device, runs b200wmma_gemm, copies D back and waits for it.  Device staging
 * buffers are cached per device and grown on demand; b200wmma_shutdown frees
 * them.  This is the call the reference's host driver makes around its kernel
 * (hipMemcpy in / launch / hipMemcpy out, samples/perf_hgemm.cpp:782-890).
 * One call per device at a time: the staging buffers, copy streams and events
 * are per device, and the call holds a per-device lock from start to finish, so
 * a second host thread calling it for the same device waits for the first.
 */
B200WMMA_API int b200wmma_gemm_host(int in_dtype, int out_dtype, uint32_t m, uint32_t n, uint32_t k,
                       const void* a, const void* b, const void* c, void* d, uint32_t lda,
                       uint32_t ldb, uint32_t ldc, uint32_t ldd, double alpha, double beta,
                       int layout_a, int layout_b, void* stream);

/*
 * b200wmma_gemm for callers that cannot allocate device memory.  (This entry point has
 * no counterpart in the reference.)
 *
 * Who needs it: a process whose own allocator has already claimed the whole GPU (an
 * inference server or a training framework with a caching pool), where a cudaMalloc
 * issued behind its back can fail or push it over its budget; and code on a latency
 * budget, since cudaFree (and, depending on the driver, cudaMalloc) waits for the whole
 * device and so stalls every stream that is running.  b200wmma_gemm calls cudaMalloc on
 * its first use on a device (for the word its kernels report abandoned waits in); this
 * variant calls neither cudaMalloc, cudaFree nor any other allocating routine.  It brings
 * column-major A / row-major B into the K-major form with a transposition pass of its
 * own, whose scratch is a fixed array inside the library image.
 *
 * Same arguments, same checks, same arithmetic and same results as b200wmma_gemm, for
 * these type pairs: F16->F16, F16->F32, BF16->F32, BF16->BF16, XF32->F32, I8->I32,
 * E4M3->BF16, E4M3->F32, E5M2->BF16, E5M2->F32.  Not offered (B200WMMA_ERR_UNSUPPORTED):
 * F32->F32, whose hi / lo split of A and B needs 2 (m + n) k floats of scratch for every
 * layout, and F64->F64.  Every argument is validated before anything is enqueued.
 * Differences:
 *   - limit: the transposed copies, m * k' elements of A (if column-major) plus n * k'
 *     of B (if row-major), k' = k rounded up to 16 bytes, must fit in 8 MiB together;
 *     larger problems are refused with B200WMMA_ERR_TOO_LARGE.  Native layouts need no
 *     scratch and have no size limit.  The array occupies 8 MiB on every GPU that loads
 *     the library, for the life of the process.
 *   - the first call on each device looks up the device address of that array.  Make
 *     that first call during set-up, before any stream capture is begun.
 *   - all calls on a device share the one array and it keeps the previous call's
 *     contents; the entry point rewrites everything it later reads, so no clearing is
 *     needed, but two calls whose kernels can overlap on the GPU (different streams)
 *     race on it.  Keep calls on one device in one stream, or order them with events.
 *   - a kernel that gives up on a bounded wait still exits cleanly, but the event is
 *     not reported through b200wmma_check_device (that flag lives in allocated memory).
 */
B200WMMA_API int b200wmma_gemm_noalloc(int in_dtype, int out_dtype, uint32_t m, uint32_t n,
                                       uint32_t k, const void* a, const void* b, const void* c,
                                       void* d, uint32_t lda, uint32_t ldb, uint32_t ldc,
                                       uint32_t ldd, double alpha, double beta, int layout_a,
                                       int layout_b, void* stream);

/*
 * y_out = alpha * A * x + beta * y_in, A column-major m x k with leading
 * dimension lda >= m (reference: samples/simple_sgemv.cpp:103-155, host routine
 * :46-67; simple_dgemv.cpp).  dtype F32 or F64.  y_out may alias y_in.
 * Each row is summed in ascending column order with a rounded multiply and a
 * rounded add per term, exactly like the host routine, so results are
 * bit-identical to it.  Needs no scratch memory.
 */
B200WMMA_API int b200wmma_gemv(int dtype, uint32_t m, uint32_t k, const void* a, const void* x,
                  const void* y_in, void* y_out, double alpha, double beta, uint32_t lda,
                  void* stream);

/*
 * DLRM dot-interaction forward (reference: samples/simple_dlrm.cpp:184-284,
 * host routine test/reference_impl.hpp:83-119).  input [batch][m][k],
 * output [batch][k + m(m-1)/2]: the first k values are row 0 of the sample, then
 * the strict lower triangle of X X^T in row-major (i, j<i) order.  dtype F16
 * (fp32 accumulation).  m <= 32, k a multiple of 16 and <= 256.  Unlike the
 * reference no m*m*batch scratch buffer is needed.  The first DLRM call on a
 * device allocates and zeroes a 2 KB ring of work counters (a synchronising
 * step: make that call outside stream capture); later calls only launch.
 * Each stream of a device owns one of 64 self-resetting counters, shared by
 * all DLRM launches (forward and backward) of that stream, which run one after
 * the other; any number of launches may be queued.  A 65th distinct stream on
 * one device makes the call wait for the device once and start the table over.
 * A DLRM launch captured into a CUDA graph keeps the counter of the stream it
 * was captured on: do not replay such a graph concurrently with DLRM work on
 * that stream.
 */
B200WMMA_API int b200wmma_dlrm_fwd(int dtype, const void* input, void* output, uint32_t m, uint32_t k,
                      uint32_t batch, void* stream);

/*
 * DLRM dot-interaction backward (reference: samples/simple_dlrm.cpp:290-441,
 * host routine test/reference_impl.hpp:121-179).  upstream [batch][k + m(m-1)/2];
 * mlp_grad [batch][k] = first k upstream values; grad [batch][m][k] = G X with G
 * the symmetric zero-diagonal matrix unpacked from the rest of upstream.
 */
B200WMMA_API int b200wmma_dlrm_bwd(int dtype, const void* input, const void* upstream, void* grad,
                      void* mlp_grad, uint32_t m, uint32_t k, uint32_t batch, void* stream);

/*
 * Waits for `stream` and reports whether any kernel of this library gave up on a
 * bounded device-side wait since the last call (B200WMMA_ERR_DEVICE_WAIT), then
 * clears the flag.  `detail`, when not NULL, receives a code naming the wait.
 */
B200WMMA_API int b200wmma_check_device(void* stream, uint32_t* detail);

/* Frees every per-device cache (staging buffers, scratch, tensor maps). */
B200WMMA_API int b200wmma_shutdown(void);

#ifdef __cplusplus
}
#endif

#endif /* ROCWMMA_B200_C_API_H */
