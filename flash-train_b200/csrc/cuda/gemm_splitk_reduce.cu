// Second pass of the split-K kernels: D = alpha * sum_s partial[s] + beta * C.
// The partials are dense row-major m x n slabs written by the first pass; the
// slabs are summed in slice order in FP32, so the result does not depend on
// which CTA finished first. HBM-bound: (splits + 1 [+ 1 with C]) * m * n * 4
// bytes of traffic.
#include <cuda_runtime.h>

#include <cstdint>

#include "gemm_kernels.hpp"
#include "ptx.cuh"

namespace ftcuda {
namespace {

struct ReduceParams {
    const float* partials;
    const float* c;
    float* d;
    std::int64_t c_row_stride, c_col_stride;
    std::int64_t d_row_stride, d_col_stride;
    std::uint64_t m, n;
    std::uint32_t splits;
    float alpha, beta;
    bool vectorised;
};

__global__ void __launch_bounds__(256) splitKReduce(const ReduceParams p) {
    // Launched with programmatic stream serialization: the CTAs may be resident before the kernel
    // that writes the partial sums has completed, and wait here for it.
    gridDependencyWait();
    const std::uint64_t slab   = p.m * p.n;
    const std::uint64_t stride = static_cast<std::uint64_t>(gridDim.x) * blockDim.x;
    std::uint64_t index        = static_cast<std::uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (p.vectorised) {
        // n % 4 == 0 and dense, 16-byte aligned C and D: four columns per thread.
        const std::uint64_t quads = slab / 4;
        for (; index < quads; index += stride) {
            const std::uint64_t element = index * 4;
            float4 sum                  = *reinterpret_cast<const float4*>(p.partials + element);
            for (std::uint32_t s = 1; s < p.splits; ++s) {
                const float4 next = *reinterpret_cast<const float4*>(p.partials + s * slab + element);
                sum.x += next.x;
                sum.y += next.y;
                sum.z += next.z;
                sum.w += next.w;
            }
            const std::uint64_t row = element / p.n;
            const std::uint64_t col = element % p.n;
            float4 value = make_float4(p.alpha * sum.x, p.alpha * sum.y, p.alpha * sum.z, p.alpha * sum.w);
            if (p.c != nullptr) {
                const float4 addend = *reinterpret_cast<const float4*>(p.c + row * p.c_row_stride + col);
                value.x += p.beta * addend.x;
                value.y += p.beta * addend.y;
                value.z += p.beta * addend.z;
                value.w += p.beta * addend.w;
            }
            *reinterpret_cast<float4*>(p.d + row * p.d_row_stride + col) = value;
        }
        return;
    }
    for (; index < slab; index += stride) {
        float sum = p.partials[index];
        for (std::uint32_t s = 1; s < p.splits; ++s) { sum += p.partials[s * slab + index]; }
        const std::int64_t row = static_cast<std::int64_t>(index / p.n);
        const std::int64_t col = static_cast<std::int64_t>(index % p.n);
        float value            = p.alpha * sum;
        if (p.c != nullptr) { value += p.beta * p.c[row * p.c_row_stride + col * p.c_col_stride]; }
        p.d[row * p.d_row_stride + col * p.d_col_stride] = value;
    }
}

// Scatter form: the combined value of every element is ADDED (one FP32 atomic) into the buffer of the
// row's owner, a dense [rows_per_owner][n] matrix that may live on another GPU.
struct ScatterReduceParams {
    const float* partials;
    float* owner_rows[8];
    std::uint64_t m, n, rows_per_owner;
    std::uint32_t splits;
    float alpha;
};

__global__ void __launch_bounds__(256) splitKReduceScatter(const ScatterReduceParams p) {
    const std::uint64_t slab   = p.m * p.n;
    const std::uint64_t stride = static_cast<std::uint64_t>(gridDim.x) * blockDim.x;
    for (std::uint64_t index = static_cast<std::uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; index < slab; index += stride) {
        float sum = p.partials[index];
        for (std::uint32_t s = 1; s < p.splits; ++s) { sum += p.partials[s * slab + index]; }
        const std::uint64_t row   = index / p.n;
        const std::uint64_t col   = index % p.n;
        const std::uint64_t owner = row / p.rows_per_owner;
        // System scope: several GPUs add into the same peer-mapped element at once.
        atomicAdd_system(p.owner_rows[owner] + (row - owner * p.rows_per_owner) * p.n + col, p.alpha * sum);
    }
}

bool denseAligned(const float* base, std::int64_t row_stride, std::int64_t col_stride) {
    return col_stride == 1 && row_stride % 4 == 0 && reinterpret_cast<std::uintptr_t>(base) % 16 == 0;
}

}  // namespace

cudaError_t launchSplitKReduce(const FtcudaGemmDesc& desc, const float* partials, std::uint32_t splits,
                               cudaStream_t stream) {
    ReduceParams p{};
    p.partials     = partials;
    p.c            = desc.c;
    p.d            = desc.d;
    p.c_row_stride = desc.c_row_stride;
    p.c_col_stride = desc.c_col_stride;
    p.d_row_stride = desc.d_row_stride;
    p.d_col_stride = desc.d_col_stride;
    p.m            = desc.m;
    p.n            = desc.n;
    p.splits       = splits;
    p.alpha        = desc.alpha;
    p.beta         = desc.beta;
    p.vectorised   = desc.n % 4 == 0 && reinterpret_cast<std::uintptr_t>(partials) % 16 == 0 &&
                   denseAligned(desc.d, desc.d_row_stride, desc.d_col_stride) &&
                   (desc.c == nullptr || denseAligned(desc.c, desc.c_row_stride, desc.c_col_stride));
    const std::uint64_t items  = p.vectorised ? desc.m * desc.n / 4 : desc.m * desc.n;
    std::uint64_t blocks       = ceilDiv(items, 256);
    if (blocks > 148 * 16) { blocks = 148 * 16; }
    if (blocks == 0) { blocks = 1; }
    cudaLaunchConfig_t config{};
    config.gridDim   = dim3(static_cast<unsigned>(blocks), 1, 1);
    config.blockDim  = dim3(256, 1, 1);
    config.stream    = stream;
    cudaLaunchAttribute attribute{};
    attribute.id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute.val.programmaticStreamSerializationAllowed = 1;
    config.attrs                                         = &attribute;
    config.numAttrs                                      = 1;
    return cudaLaunchKernelEx(&config, splitKReduce, p);
}

}  // namespace ftcuda

namespace ftcuda {

cudaError_t launchSplitKReduceScatter(const FtcudaGemmDesc& desc, const float* partials, std::uint32_t splits,
                                      float* const* owner_rows, std::uint32_t owners, std::uint32_t rows_per_owner,
                                      cudaStream_t stream) {
    ScatterReduceParams p{};
    p.partials       = partials;
    p.m              = desc.m;
    p.n              = desc.n;
    p.rows_per_owner = rows_per_owner;
    p.splits         = splits;
    p.alpha          = desc.alpha;
    for (std::uint32_t i = 0; i < owners && i < 8; ++i) { p.owner_rows[i] = owner_rows[i]; }
    const std::uint64_t elements = desc.m * desc.n;
    std::uint64_t blocks         = (elements + 255) / 256;
    if (blocks > 148ULL * 16) { blocks = 148ULL * 16; }
    if (blocks == 0) { return cudaSuccess; }
    splitKReduceScatter<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace ftcuda
