// Internal interface of the CUDA platform subtree: the in-memory form of a
// configured launch and the per-kernel-family host entry points that the
// C ABI in ftcuda_gemm.cu dispatches to.
#ifndef FTCUDA_GEMM_KERNELS_HPP_
#define FTCUDA_GEMM_KERNELS_HPP_

#include <cuda.h>
#include <cuda_runtime_api.h>

#include <cstddef>
#include <cstdint>
#include <vector>

#include "ftcuda/ftcuda.h"

namespace ftcuda {

// How an operand tile reaches the kernel.
enum Variant : int {
    kVariantGeneric  = 0,  // predicated loads, any strides (SIMT only)
    kVariantTmaAk    = 1,  // TMA; A rows contiguous along K (row-major A)
    kVariantTmaAm    = 2,  // TMA; A contiguous along M (transposed view of a K x M buffer)
    kVariantSmall    = 3,  // SIMT only: 32 x 32 tiles with register prefetch, for outputs too small to fill the SMs otherwise
    kVariantMaskA    = 15,
    kVariantFlagBk   = 16,  // tensor kernel: B contiguous along K (transposed view of an N x K buffer)
    kVariantFlagCluster = 64,  // tensor kernel: the K slices of a tile form a thread-block cluster (one launch)
    kVariantFlagEarlyStart = 128,  // ... launched with programmatic stream serialization (set-up overlaps the predecessor's tail)
};

// One operand copied into the workspace before the launch (see LaunchState::staged).
struct StagedOperand {
    const float* source;
    std::int64_t row_stride, col_stride;  // of the source, in elements
    std::uint64_t rows, cols;
    std::uint64_t pitch;                   // elements between rows of the copy, a multiple of four
    std::uint64_t offset;                  // byte offset of the copy in the workspace, a multiple of 256
};

// What ftcuda_gemm_configure stores inside an FtcudaGemmLaunch.
struct LaunchState {
    alignas(64) CUtensorMap map_a;
    alignas(64) CUtensorMap map_b;
    FtcudaGemmDesc desc;
    std::int32_t kernel;
    std::int32_t variant;
    std::uint32_t grid_x, grid_y, grid_z;
    std::uint32_t block;
    std::uint32_t smem_bytes;
    std::uint32_t splits;          // K slices (1 = no split)
    std::uint32_t k_per_split;     // K elements per slice, a multiple of the K tile
    std::uint32_t chunk_k_blocks;  // tensor kernel: K blocks accumulated in TMEM between drains
    std::uint32_t row_tile;        // skinny kernel: rows of A kept per thread
    std::uint32_t band_m_tiles;    // tensor kernel: M tiles walked together (fixed when the launch is configured)
    std::uint64_t workspace_bytes;
    int* device_status;            // mapped host word the kernels report a timed-out wait in
    volatile int* host_status;
    // Operand staging (tensor-core families): an A or B whose layout TMA cannot describe (a transposed
    // view with an odd pitch, a misaligned base, two non-unit strides) is first copied, by a small
    // kernel, into the head of the workspace as a dense row-major matrix with a 16-byte row pitch; the
    // TMA descriptors were made for that copy and get its address in front of every launch.
    std::uint32_t staged;          // bit 0: A is staged, bit 1: B
    StagedOperand stage[2];
    std::uint64_t stage_bytes;     // bytes at the head of the workspace taken by the copies
};
static_assert(sizeof(LaunchState) <= sizeof(FtcudaGemmLaunch), "launch blob too small");
static_assert(alignof(FtcudaGemmLaunch) >= 64, "launch blob must be 64-byte aligned");

inline std::uint64_t ceilDiv(std::uint64_t x, std::uint64_t y) { return (x + y - 1) / y; }

// Writes a message (if a buffer is given) and returns `code`.
int fail(char* message, std::size_t capacity, int code, const char* format, ...);

// ---- runtime helpers (ftcuda_runtime.cu) ----

// SM count of `device`, cached. Returns false (with message) on a CUDA error.
bool deviceSmCount(int device, int* sm_count, char* message, std::size_t capacity);
// Per-device status word in mapped pinned host memory; nonzero after a kernel
// gave up on a wait. Returns false (with message) on a CUDA error.
bool deviceStatusWord(int device, int** device_pointer, volatile int** host_pointer, char* message,
                      std::size_t capacity);
// Reads the status word of a launch's device and clears it: a timed-out wait is reported once.
inline int takeDeviceStatus(volatile int* host_status) {
    if (host_status == nullptr) { return 0; }
    const int code = *host_status;
    if (code != 0) { *host_status = 0; }
    return code;
}
// Shared-memory swizzle of a tiled copy. kSwizzle128: 16-byte chunks of a 128-byte
// row XOR-ed with row % 8. kSwizzle128Atom32: 32-byte chunks XOR-ed with row % 4
// (the layout the tensor cores want for an MN-major operand of 32-bit elements).
enum TensorMapSwizzle : int { kSwizzleNone = 0, kSwizzle128 = 1, kSwizzle128Atom32 = 2 };
// Encodes a 2-D FP32 tiled TMA descriptor: `inner` contiguous elements per row,
// `outer` rows, `row_pitch_bytes` between rows, box = box_inner x box_outer.
bool encodeTensorMap2d(CUtensorMap* map, const void* base, std::uint64_t inner, std::uint64_t outer,
                       std::uint64_t row_pitch_bytes, std::uint32_t box_inner, std::uint32_t box_outer,
                       int swizzle, char* message, std::size_t capacity);
void countLaunches(std::uint64_t launches);

// True when `base`/strides describe a matrix TMA can fetch with `contiguous`
// as the unit-stride dimension: unit stride there, 16-byte aligned base,
// row pitch a positive multiple of 16 bytes that fits 2^40, extents < 2^32.
bool tmaEligible(const void* base, std::int64_t contiguous_stride, std::int64_t other_stride,
                 std::uint64_t contiguous_extent, std::uint64_t other_extent);

// ---- operand staging (gemm_stage.cu) ----
// Decides which operands of `desc` kernel family `kernel` cannot fetch by TMA as they are, records
// them in `state` (staged, stage[], stage_bytes) and rewrites state.desc to describe the copies
// (dense row-major, placeholder addresses of the right alignment). Returns a reason when an operand
// can be neither fetched nor staged, else nullptr. Pure host arithmetic.
const char* planStaging(int kernel, const FtcudaGemmDesc& desc, LaunchState& state);
// Enqueues the copies into `workspace` and points the launch's TMA descriptors at them.
cudaError_t runStaging(LaunchState& local, void* workspace, cudaStream_t stream, char* message, std::size_t capacity);

// ---- kernel families ----
// supports*: nullptr when the family can run the problem, else the reason.
// configure*: fills `state` (desc, kernel already set); 0 on success.
// launch*: enqueues; returns the CUDA error of the launch.

namespace tf32x3 {
struct TensorParams;
}
// 3xTF32 for few rows of A with the operands' roles swapped (gemm_tf32x3_rows.cu).
const char* supportsTensorRows(const FtcudaGemmDesc& desc);
int configureTensorRows(LaunchState& state, char* message, std::size_t capacity);
cudaError_t launchTensorRows(const LaunchState& state, cudaStream_t stream);

const char* supportsSimt(const FtcudaGemmDesc& desc, bool split_k);
int configureSimt(LaunchState& state, bool split_k, char* message, std::size_t capacity);
cudaError_t launchSimt(const LaunchState& state, void* workspace, cudaStream_t stream);
// Fills grid, block and K slicing of the predicated (any layout) SIMT kernel for
// about `splits` K slices. Pure arithmetic on state.desc: no device call.
void planSimtGenericSplitK(LaunchState& state, std::uint32_t splits);

const char* supportsSkinny(const FtcudaGemmDesc& desc);
int configureSkinny(LaunchState& state, char* message, std::size_t capacity);
cudaError_t launchSkinny(const LaunchState& state, cudaStream_t stream);

const char* supportsTensor(const FtcudaGemmDesc& desc, bool split_k);
int configureTensor(LaunchState& state, bool split_k, char* message, std::size_t capacity);
cudaError_t launchTensor(const LaunchState& state, void* workspace, cudaStream_t stream);
// The tensor kernel with its results added into per-owner row buffers (see ftcuda_gemm_launch_scatter).
// With a workspace (and K slices) the slices are combined locally first and every element travels once.
cudaError_t launchTensorScatter(const LaunchState& state, void* workspace, float* const* owner_rows, std::uint32_t owners,
                                std::uint32_t rows_per_owner, cudaStream_t stream);
cudaError_t launchSplitKReduceScatter(const FtcudaGemmDesc& desc, const float* partials, std::uint32_t splits,
                                      float* const* owner_rows, std::uint32_t owners, std::uint32_t rows_per_owner,
                                      cudaStream_t stream);

// ---- grouped launches (ftcuda_grouped_gemm_*): many independent GEMMs behind one call ----

// What ftcuda_grouped_gemm_configure builds (a heap object behind the opaque handle).
struct GroupedLaunchState {
    std::int32_t kernel = 0;
    std::int32_t device = 0;
    // FTCUDA_GROUPED_GEMM_EXACT: one configured launch of the exact-FP32 family per non-empty group.
    std::vector<LaunchState> per_group;
    // FTCUDA_GROUPED_GEMM_TF32X3: the table the persistent kernel walks -- one GroupEntry per non-empty
    // group, then the group index of every work item -- exactly as it is copied into the workspace.
    std::vector<unsigned char> table;
    std::uint32_t entries = 0;
    std::uint32_t items   = 0;
    std::uint32_t grid    = 0;
    std::uint32_t a_m_contiguous = 0, b_k_contiguous = 0;
    float alpha = 0.0F, beta = 0.0F;
    std::uint64_t workspace_bytes = 0;
    int* device_status            = nullptr;
    volatile int* host_status     = nullptr;
};

// The persistent tensor-core kernel over the tiles of all groups (gemm_tf32x3.cu).
const char* supportsTensorGrouped(const FtcudaGemmDesc* groups, std::uint32_t count);
int configureTensorGrouped(GroupedLaunchState& state, const FtcudaGemmDesc* groups, std::uint32_t count, char* message,
                           std::size_t capacity);
cudaError_t launchTensorGrouped(const GroupedLaunchState& state, void* workspace, cudaStream_t stream);

// D = alpha * sum_s partial[s] + beta * C over `splits` dense m x n partials.
cudaError_t launchSplitKReduce(const FtcudaGemmDesc& desc, const float* partials, std::uint32_t splits,
                               cudaStream_t stream);

}  // namespace ftcuda

#endif
