/*
 * ftcuda/ftcuda.h -- thin C ABI between the host pipeline and the CUDA
 * (sm_100a) platform subtree.
 *
 * Everything the C++ host layers (family, primitives, plan) need from the GPU
 * goes through these entry points: plain pointers, integers and fixed-size
 * structs, integer return codes, no C++ types, no exceptions. The platform
 * subtree behind it replaces the reference's HIP subtree:
 *   ftcuda_current_device   <- getCurrentDeviceId / hipGetDevice
 *                              (src/constraints.cpp:15-26)
 *   ftcuda_gemm_supports    <- the platform half of Fp32Gemm::isApplicable
 *                              (src/primitive/hygon/gemm/fp32_gemm.cpp:27-62)
 *   ftcuda_gemm_configure   <- Fp32Gemm::configure (fp32_gemm.cpp:66-77)
 *   ftcuda_gemm_launch      <- launchFp32Gemm (src/primitive/hygon/gemm/fp32_gemm.hip:35-51)
 *   ftcuda_trace_push/pop   <- roctxRangePushA/Pop (src/trace.cpp:14-28)
 *
 * Return code: 0 = success; nonzero = failure with a NUL-terminated reason
 * written to the caller's message buffer (when one is given).
 */
#ifndef FTCUDA_FTCUDA_H_
#define FTCUDA_FTCUDA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__) || defined(__clang__)
#    define FTCUDA_API __attribute__((visibility("default")))
#else
#    define FTCUDA_API
#endif

/* Kernel families. Each id is one Primitive of the GEMM family. */
enum {
    /* Exact FP32: SIMT FFMA tiles, TMA-staged when the layout allows it, with a
     * predicated path for any strides. No workspace. */
    FTCUDA_GEMM_SIMT = 0,
    /* 3xTF32 split-precision on tcgen05 tensor cores with TMEM accumulators. */
    FTCUDA_GEMM_TF32X3 = 1,
    /* 3xTF32 with the K range split across CTAs; partial tiles go to the
     * workspace and a second kernel reduces them and applies alpha/beta. */
    FTCUDA_GEMM_TF32X3_SPLITK = 2,
    /* Exact FP32 for very few rows of A: streams B once at HBM rate. */
    FTCUDA_GEMM_SKINNY = 3,
    /* Exact FP32 SIMT with the K range split across CTAs (workspace). */
    FTCUDA_GEMM_SIMT_SPLITK = 4,
    /* 3xTF32 for few rows of A (m <= 64): B fills the tensor core's 128-row
     * dimension (D^T = B^T A^T), K split over a thread-block cluster. No workspace. */
    FTCUDA_GEMM_TF32X3_ROWS = 5,
    FTCUDA_GEMM_KERNEL_COUNT = 6,
};

/* One GEMM D = alpha * A * B + beta * C in terms of raw memory. Strides are in
 * elements. c may be NULL (no beta * C term). c == d (in place) is allowed. */
typedef struct {
    const float* a;
    const float* b;
    const float* c;
    float* d;
    float alpha;
    float beta;
    uint64_t m;
    uint64_t n;
    uint64_t k;
    int64_t a_row_stride, a_col_stride;
    int64_t b_row_stride, b_col_stride;
    int64_t c_row_stride, c_col_stride;
    int64_t d_row_stride, d_col_stride;
    int32_t device;
} FtcudaGemmDesc;

/* A configured launch: kernel choice, grid, pre-encoded TMA descriptors and
 * kernel arguments. Opaque to the host code, trivially copyable, 64-byte
 * aligned (a CUtensorMap inside needs that). */
typedef struct {
    uint64_t words[160];
} __attribute__((aligned(64))) FtcudaGemmLaunch;

/* Calling thread's current CUDA device. */
FTCUDA_API int ftcuda_current_device(int32_t* device, char* message, size_t message_capacity);

/* Number of SMs of a device (cached per device after the first query). */
FTCUDA_API int ftcuda_device_sm_count(int32_t device, int32_t* sm_count, char* message, size_t message_capacity);

/* 0 when kernel family `kernel` can run `desc`; otherwise nonzero and a reason.
 * Pure host arithmetic on the descriptor: needs no device. */
FTCUDA_API int ftcuda_gemm_supports(int kernel, const FtcudaGemmDesc* desc, char* message, size_t message_capacity);

/* Fills `launch` for `kernel` on desc->device (tile shape, grid, TMA
 * descriptors). Needs no device work beyond attribute queries. */
FTCUDA_API int ftcuda_gemm_configure(int kernel, const FtcudaGemmDesc* desc, FtcudaGemmLaunch* launch, char* message,
                                     size_t message_capacity);

/* Workspace a configured launch needs, in bytes. */
FTCUDA_API uint64_t ftcuda_gemm_workspace_bytes(const FtcudaGemmLaunch* launch);

/* Enqueues the configured launch on `stream` (a cudaStream_t) and returns
 * without synchronising. No allocation, no descriptor encoding. */
FTCUDA_API int ftcuda_gemm_launch(const FtcudaGemmLaunch* launch, void* workspace, uint64_t workspace_bytes,
                                  void* stream, char* message, size_t message_capacity);

/*
 * Exact-FP32 split-K GEMM that needs no workspace from the caller and allocates
 * nothing. It has no counterpart in the reference, whose only kernel needs no
 * scratch memory at all.
 *
 * It exists for callers that cannot supply or allocate a workspace: code
 * running after a framework has taken all device memory into its own pool,
 * latency-critical loops that must avoid the device-wide synchronisation
 * inside cudaMalloc/cudaFree, and bindings that always pass a null workspace.
 * The partial sums of the K slices live in a 16 MiB array inside the library
 * image (one copy on every GPU that loads the library, kept until exit;
 * ftcuda_gemm_splitk_static_capacity returns its size in bytes).
 *
 *   - desc->device must be the calling thread's current device.
 *   - slices * m * n * 4 bytes must fit the array with at least two slices,
 *     i.e. m * n <= 2 Mi elements; larger outputs are refused with a message.
 *   - The first call on a device resolves the array's device address
 *     (cudaGetSymbolAddress); make that first call outside of stream capture.
 *   - All calls on a GPU share the array. Nothing in it has to be cleared
 *     between calls (every element read is written first in the same call),
 *     but calls that can overlap on the GPU race on it: serialise them, for
 *     instance on one stream.
 * Same arithmetic as FTCUDA_GEMM_SIMT_SPLITK: FP32 FFMA per slice, slices summed
 * in order. Returns 0, or nonzero with a reason in `message`.
 */
FTCUDA_API int ftcuda_gemm_splitk_static(const FtcudaGemmDesc* desc, void* stream, char* message,
                                         size_t message_capacity);
FTCUDA_API uint64_t ftcuda_gemm_splitk_static_capacity(void);

/*
 * K-sharded GEMM over several GPUs without a separate reduction pass (no
 * counterpart in the reference, which is single-device): `launch` was
 * configured for FTCUDA_GEMM_TF32X3 or FTCUDA_GEMM_TF32X3_SPLITK on this GPU's
 * shard of K; instead of writing d, the kernel ADDS alpha * (A B) into the
 * buffers of the rows' owners: row r goes to owner r / rows_per_owner, whose
 * buffer owner_rows[owner] is a dense FP32 [rows_per_owner][n] matrix. The
 * buffers may live on other GPUs (peer-mapped addresses, e.g. symmetric
 * memory); the additions are single FP32 atomics travelling over NVLink. The
 * caller initialises every buffer (zeros, or beta * C) and orders that before
 * the launch, and the launches of all GPUs before the first read, with
 * barriers of its own. c and beta of the descriptor are ignored. The workspace
 * is optional: without one (NULL, or fewer bytes than
 * ftcuda_gemm_workspace_bytes) every K slice of the split-K family adds its
 * tile directly, one launch, nothing stored; with one the slices are combined
 * on this GPU first and every element crosses NVLink once (two launches); a
 * launch that asks for no workspace (ftcuda_gemm_workspace_bytes == 0) never
 * writes to one. The order of the additions is not fixed, so the last bits of the result can
 * differ from run to run.
 */
FTCUDA_API int ftcuda_gemm_launch_scatter(const FtcudaGemmLaunch* launch, void* workspace, uint64_t workspace_bytes,
                                          float* const* owner_rows, int32_t owners, uint64_t rows_per_owner, void* stream,
                                          char* message, size_t message_capacity);

/*
 * Grouped GEMM: D_g = alpha * A_g * B_g + beta * C_g for num_groups independent problems, each given
 * as an ordinary descriptor (alpha, beta and device equal in all of them). The reference declares the
 * operation in its public API (include/flash_train/common.h:248-266 there) but ships no Primitive for
 * it; these entry points are what this build's GroupedABCDGemm Primitives stand on. Groups with
 * m * n == 0 are skipped.
 *   FTCUDA_GROUPED_GEMM_EXACT   exact FP32 (FFMA): one launch of the FTCUDA_GEMM_SIMT family per
 *                               non-empty group; any layout, K = 0 included; no workspace.
 *   FTCUDA_GROUPED_GEMM_TF32X3  one persistent launch of the 3xTF32 tensor-core kernel over the
 *                               output tiles of all groups. Every non-empty group must suit
 *                               FTCUDA_GEMM_TF32X3 (K >= 128, TMA-eligible A and B) and all groups
 *                               must share one operand layout class. The per-group table (TMA
 *                               descriptors, output views) is copied into the workspace by every
 *                               launch: ftcuda_grouped_gemm_workspace_bytes says how large it is.
 * configure returns a heap object through *launch; destroy frees it (NULL is allowed).
 */
enum {
    FTCUDA_GROUPED_GEMM_EXACT        = 0,
    FTCUDA_GROUPED_GEMM_TF32X3       = 1,
    FTCUDA_GROUPED_GEMM_KERNEL_COUNT = 2,
};
typedef struct FtcudaGroupedGemmLaunch FtcudaGroupedGemmLaunch;
FTCUDA_API int ftcuda_grouped_gemm_supports(int kernel, const FtcudaGemmDesc* groups, uint32_t num_groups, char* message,
                                            size_t message_capacity);
FTCUDA_API int ftcuda_grouped_gemm_configure(int kernel, const FtcudaGemmDesc* groups, uint32_t num_groups,
                                             FtcudaGroupedGemmLaunch** launch, char* message, size_t message_capacity);
FTCUDA_API uint64_t ftcuda_grouped_gemm_workspace_bytes(const FtcudaGroupedGemmLaunch* launch);
FTCUDA_API int ftcuda_grouped_gemm_launch(const FtcudaGroupedGemmLaunch* launch, void* workspace, uint64_t workspace_bytes,
                                          void* stream, char* message, size_t message_capacity);
FTCUDA_API void ftcuda_grouped_gemm_destroy(FtcudaGroupedGemmLaunch* launch);

/*
 * Per-device status word (no counterpart in the reference, whose kernel has no device-side waits).
 * Every wait inside the kernels is bounded; a kernel whose wait ran out stops its pipeline, frees
 * its tensor memory, returns, and leaves a nonzero code in a word of mapped host memory. The next
 * ftcuda_gemm_launch / ftcuda_gemm_launch_scatter on that device reports the code as a failure ONCE and
 * clears it, so later launches proceed (the context is intact: nothing trapped). ftcuda_device_status
 * reads the word without clearing it (0 = healthy; *code is 0 for a device no launch was configured
 * on yet), ftcuda_device_status_reset clears it.
 */
FTCUDA_API int ftcuda_device_status(int32_t device, int32_t* code, char* message, size_t message_capacity);
FTCUDA_API int ftcuda_device_status_reset(int32_t device, char* message, size_t message_capacity);

/*
 * Self test of the bounded wait: launches one warp on `stream` that waits, with a budget of
 * `budget_ns` nanoseconds (at most one second), on a barrier nothing ever arrives on, and then
 * records code 2 in the device's status word -- the path a kernel takes when a partner role has
 * stopped, without a trap, a fault or an unbounded spin. `device` must be current.
 */
FTCUDA_API int ftcuda_selftest_bounded_wait(int32_t device, uint64_t budget_ns, void* stream, char* message,
                                            size_t message_capacity);

/*
 * Measured FP32 FFMA rate of `device` (which must be current) in TFLOP/s: a register-only kernel of
 * independent FFMA chains, 2048 threads per SM, best of three launches timed with CUDA events on the
 * default stream; blocks until done. The yardstick the exact-FP32 kernels are held against.
 */
FTCUDA_API int ftcuda_measure_ffma_tflops(int32_t device, double* tflops, char* message, size_t message_capacity);

/* Number of device kernels ftcuda_gemm_launch has enqueued from this process;
 * benchmarks read it to report how many launches a timed region made. */
FTCUDA_API uint64_t ftcuda_launch_count(void);

/* NVTX range on the calling thread; push returns nonzero when a range was
 * opened (pop only then). */
FTCUDA_API int ftcuda_trace_push(const char* name);
FTCUDA_API void ftcuda_trace_pop(void);
FTCUDA_API void ftcuda_trace_mark(const char* name);

#ifdef __cplusplus
}
#endif

#endif
