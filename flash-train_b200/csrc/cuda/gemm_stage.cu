// Operand staging for the tensor-core kernel families.
//
// Those kernels fetch A and B with TMA, which wants a unit stride in one dimension, a 16-byte
// aligned base and a row pitch that is a multiple of 16 bytes. A transposed view of a k x m buffer
// with an odd m (the tail shapes m = 17, 255, 4097), a view into the middle of a row, or a matrix
// with two non-unit strides has none of that, and without staging such a problem falls to the
// predicated SIMT kernel (4097 x 4096 x 4096 with A transposed: 4.67 ms against 0.66 ms). Staging
// copies the operand once per launch into the head of the workspace as a dense row-major matrix
// with a padded pitch -- m k 4 bytes read and written, about 5 % of the GEMM's time at that shape --
// and the GEMM kernel runs on the copy unchanged. The Primitive then asks for a workspace.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cudaTypedefs.h>

#include <cstdint>

#include "gemm_kernels.hpp"

namespace ftcuda {
namespace {

constexpr std::uint64_t kStageAlignment = 256;

struct RepackParams {
    const float* source;
    std::int64_t row_stride, col_stride;
    std::uint64_t rows, cols;
    float* copy;
    std::uint64_t pitch;
};

// 32 x 32 elements per CTA. When the source runs fastest along its rows index (a transposed view)
// the tile goes through shared memory so that both the loads and the stores of a warp touch
// consecutive addresses; otherwise it is a straight strided copy.
__global__ void __launch_bounds__(256) repackMatrix(const RepackParams p) {
    __shared__ float tile[32][33];
    const std::uint64_t row0 = static_cast<std::uint64_t>(blockIdx.x) * 32;
    const std::uint64_t col0 = static_cast<std::uint64_t>(blockIdx.y) * 32;
    const int tx             = threadIdx.x & 31;
    const int ty             = threadIdx.x >> 5;  // 0..7
    const std::int64_t rs    = p.row_stride < 0 ? -p.row_stride : p.row_stride;
    const std::int64_t cs    = p.col_stride < 0 ? -p.col_stride : p.col_stride;
    if (rs < cs) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const std::uint64_t row = row0 + tx;
            const std::uint64_t col = col0 + ty + 8 * j;
            tile[ty + 8 * j][tx] = (row < p.rows && col < p.cols)
                                       ? p.source[static_cast<std::int64_t>(row) * p.row_stride + static_cast<std::int64_t>(col) * p.col_stride]
                                       : 0.0F;
        }
        __syncthreads();
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const std::uint64_t row = row0 + ty + 8 * j;
            const std::uint64_t col = col0 + tx;
            if (row < p.rows && col < p.cols) { p.copy[row * p.pitch + col] = tile[tx][ty + 8 * j]; }
        }
        return;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const std::uint64_t row = row0 + ty + 8 * j;
        const std::uint64_t col = col0 + tx;
        if (row < p.rows && col < p.cols) {
            p.copy[row * p.pitch + col] =
                p.source[static_cast<std::int64_t>(row) * p.row_stride + static_cast<std::int64_t>(col) * p.col_stride];
        }
    }
}

PFN_cuTensorMapReplaceAddress_v12000 addressReplacer() {
    static const PFN_cuTensorMapReplaceAddress_v12000 replacer = [] {
        void* entry                            = nullptr;
        cudaDriverEntryPointQueryResult result = cudaDriverEntryPointSymbolNotFound;
        if (cudaGetDriverEntryPoint("cuTensorMapReplaceAddress", &entry, cudaEnableDefault, &result) != cudaSuccess ||
            result != cudaDriverEntryPointSuccess) {
            entry = nullptr;
        }
        return reinterpret_cast<PFN_cuTensorMapReplaceAddress_v12000>(entry);
    }();
    return replacer;
}

bool eitherWay(const float* base, std::int64_t row_stride, std::int64_t col_stride, std::uint64_t rows, std::uint64_t cols) {
    return tmaEligible(base, col_stride, row_stride, cols, rows) || tmaEligible(base, row_stride, col_stride, rows, cols);
}

// An address with the alignment of the future copy, inside the operand's own allocation (the
// descriptors are encoded with it when the launch is configured and re-pointed before every launch).
const float* placeholder(const float* source) {
    return reinterpret_cast<const float*>(reinterpret_cast<std::uintptr_t>(source) & ~static_cast<std::uintptr_t>(15));
}

}  // namespace

const char* planStaging(int kernel, const FtcudaGemmDesc& desc, LaunchState& state) {
    state.staged      = 0;
    state.stage_bytes = 0;
    if (desc.m * desc.n == 0 || desc.k == 0) { return nullptr; }
    // The few-rows kernel takes A contiguous along K only; the large-tile kernels take either orientation.
    const bool a_fetchable = kernel == FTCUDA_GEMM_TF32X3_ROWS ? tmaEligible(desc.a, desc.a_col_stride, desc.a_row_stride, desc.k, desc.m)
                                                               : eitherWay(desc.a, desc.a_row_stride, desc.a_col_stride, desc.m, desc.k);
    const bool b_fetchable = eitherWay(desc.b, desc.b_row_stride, desc.b_col_stride, desc.k, desc.n);
    const struct {
        bool needed;
        const float* source;
        std::int64_t row_stride, col_stride;
        std::uint64_t rows, cols;
    } operands[2] = {{!a_fetchable, desc.a, desc.a_row_stride, desc.a_col_stride, desc.m, desc.k},
                     {!b_fetchable, desc.b, desc.b_row_stride, desc.b_col_stride, desc.k, desc.n}};
    std::uint64_t offset = 0;
    for (int which = 0; which < 2; ++which) {
        if (!operands[which].needed) { continue; }
        if (operands[which].source == nullptr) { return which == 0 ? "A has no address" : "B has no address"; }
        if (reinterpret_cast<std::uintptr_t>(operands[which].source) % alignof(float) != 0) {
            return which == 0 ? "A is not float-aligned" : "B is not float-aligned";
        }
        if (operands[which].rows >= (1ULL << 31) || ceilDiv(operands[which].cols, 32) > 65535) {
            return which == 0 ? "A can be neither fetched by TMA nor staged (too large)" : "B can be neither fetched by TMA nor staged (too large)";
        }
        StagedOperand& staged = state.stage[which];
        staged.source         = operands[which].source;
        staged.row_stride     = operands[which].row_stride;
        staged.col_stride     = operands[which].col_stride;
        staged.rows           = operands[which].rows;
        staged.cols           = operands[which].cols;
        staged.pitch          = ceilDiv(operands[which].cols, 4) * 4;
        staged.offset         = offset;
        offset += ceilDiv(staged.rows * staged.pitch * sizeof(float), kStageAlignment) * kStageAlignment;
        state.staged |= 1U << which;
    }
    state.stage_bytes = offset;
    if ((state.staged & 1U) != 0) {
        state.desc.a            = placeholder(desc.a);
        state.desc.a_row_stride = static_cast<std::int64_t>(state.stage[0].pitch);
        state.desc.a_col_stride = 1;
    }
    if ((state.staged & 2U) != 0) {
        state.desc.b            = placeholder(desc.b);
        state.desc.b_row_stride = static_cast<std::int64_t>(state.stage[1].pitch);
        state.desc.b_col_stride = 1;
    }
    return nullptr;
}

cudaError_t runStaging(LaunchState& local, void* workspace, cudaStream_t stream, char* message, std::size_t capacity) {
    const PFN_cuTensorMapReplaceAddress_v12000 replace = addressReplacer();
    if (replace == nullptr) {
        fail(message, capacity, 1, "the CUDA driver does not provide cuTensorMapReplaceAddress");
        return cudaErrorNotSupported;
    }
    // The workspace's own alignment is the caller's; the copies sit at 256-byte boundaries inside it.
    const std::uintptr_t base = (reinterpret_cast<std::uintptr_t>(workspace) + kStageAlignment - 1) & ~(kStageAlignment - 1);
    for (int which = 0; which < 2; ++which) {
        if ((local.staged & (1U << which)) == 0) { continue; }
        const StagedOperand& staged = local.stage[which];
        RepackParams p{};
        p.source     = staged.source;
        p.row_stride = staged.row_stride;
        p.col_stride = staged.col_stride;
        p.rows       = staged.rows;
        p.cols       = staged.cols;
        p.copy       = reinterpret_cast<float*>(base + staged.offset);
        p.pitch      = staged.pitch;
        const dim3 grid(static_cast<unsigned>(ceilDiv(staged.rows, 32)), static_cast<unsigned>(ceilDiv(staged.cols, 32)), 1);
        repackMatrix<<<grid, 256, 0, stream>>>(p);
        const cudaError_t error = cudaGetLastError();
        if (error != cudaSuccess) { return error; }
        countLaunches(1);
        CUtensorMap* map = which == 0 ? &local.map_a : &local.map_b;
        if (replace(map, p.copy) != CUDA_SUCCESS) {
            fail(message, capacity, 1, "cuTensorMapReplaceAddress failed");
            return cudaErrorInvalidValue;
        }
    }
    return cudaSuccess;
}

}  // namespace ftcuda
