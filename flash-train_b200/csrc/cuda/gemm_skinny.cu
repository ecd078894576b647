// Exact-FP32 GEMM for very few rows of A (m <= 32): D = alpha * A * B + beta * C
// where the whole cost is reading B once. HBM-bound; algorithmic traffic
// 4 * (k * n + m * k + m * n [+ m * n]) bytes, of which k * n dominates.
//
// Each CTA owns a strip of 32 columns of B and walks all of K. A warp-wide
// 128-bit load covers 4 rows of B x 32 columns (lane = row-in-group * 8 +
// column-quad), so every request is four full 128-byte lines; eight such loads
// are kept in flight per warp. The values of A are broadcast loads that hit
// L1. The eight warps of a CTA take interleaved K rows; their partial sums
// meet in a fixed order (shuffles across the 4 row groups of a warp, then
// shared memory across warps), so results are deterministic. Sums are FP32
// FFMA; the order over K differs from a sequential loop only by that fixed
// partition.
#include <cuda_runtime.h>

#include <cstdint>

#include "gemm_kernels.hpp"

namespace ftcuda {
namespace {

constexpr int kStripColumns = 32;
constexpr int kWarps        = 8;
constexpr int kRowsPerStep  = 4 * kWarps;  // K rows consumed per CTA step

struct SkinnyParams {
    const float* a;
    const float* b;
    const float* c;
    float* d;
    std::int64_t a_row_stride, a_col_stride;
    std::int64_t b_row_stride;  // B columns are unit stride
    std::int64_t c_row_stride, c_col_stride;
    std::int64_t d_row_stride, d_col_stride;
    std::uint32_t m, n, k;
    float alpha, beta;
};

template<int kRows>
__global__ void __launch_bounds__(kWarps * 32) skinnyGemm(const SkinnyParams p) {
    // Loads of B kept in flight per thread; fewer when the accumulators are many.
    constexpr int kUnroll = kRows >= 16 ? 4 : 8;
    __shared__ float4 across_warps[kWarps][kRows][8];
    const int warp      = threadIdx.x >> 5;
    const int lane      = threadIdx.x & 31;
    const int row_group = lane >> 3;  // which of the 4 K rows of a warp-wide load
    const int quad      = lane & 7;   // which 4 columns of the strip
    const std::uint32_t col = blockIdx.x * kStripColumns + quad * 4;
    const bool col_ok       = col < p.n;  // n % 4 == 0, so a quad is all in or all out

    float4 acc[kRows];
#pragma unroll
    for (int i = 0; i < kRows; ++i) { acc[i] = make_float4(0.0F, 0.0F, 0.0F, 0.0F); }

    const std::uint32_t first = warp * 4 + row_group;
    for (std::uint32_t k0 = first; k0 < p.k; k0 += kRowsPerStep * kUnroll) {
        float4 b_value[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const std::uint32_t kk = k0 + u * kRowsPerStep;
            b_value[u] = (kk < p.k && col_ok)
                             ? __ldcs(reinterpret_cast<const float4*>(p.b + static_cast<std::int64_t>(kk) * p.b_row_stride + col))
                             : make_float4(0.0F, 0.0F, 0.0F, 0.0F);
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const std::uint32_t kk = k0 + u * kRowsPerStep;
            if (kk >= p.k) { break; }
#pragma unroll
            for (int i = 0; i < kRows; ++i) {
                if (i < static_cast<int>(p.m)) {
                    const float a_value =
                        __ldg(p.a + static_cast<std::int64_t>(i) * p.a_row_stride + static_cast<std::int64_t>(kk) * p.a_col_stride);
                    acc[i].x = fmaf(a_value, b_value[u].x, acc[i].x);
                    acc[i].y = fmaf(a_value, b_value[u].y, acc[i].y);
                    acc[i].z = fmaf(a_value, b_value[u].z, acc[i].z);
                    acc[i].w = fmaf(a_value, b_value[u].w, acc[i].w);
                }
            }
        }
    }

    // Fold the 4 row groups of the warp, then the 8 warps, in a fixed order.
#pragma unroll
    for (int i = 0; i < kRows; ++i) {
#pragma unroll
        for (int offset = 8; offset <= 16; offset <<= 1) {
            acc[i].x += __shfl_xor_sync(0xFFFFFFFFU, acc[i].x, offset);
            acc[i].y += __shfl_xor_sync(0xFFFFFFFFU, acc[i].y, offset);
            acc[i].z += __shfl_xor_sync(0xFFFFFFFFU, acc[i].z, offset);
            acc[i].w += __shfl_xor_sync(0xFFFFFFFFU, acc[i].w, offset);
        }
        if (row_group == 0) { across_warps[warp][i][quad] = acc[i]; }
    }
    __syncthreads();
    // kRows * 8 quads to finish; one thread each.
    for (int item = threadIdx.x; item < kRows * 8; item += kWarps * 32) {
        const int i = item >> 3;
        const int q = item & 7;
        const std::uint32_t out_col = blockIdx.x * kStripColumns + q * 4;
        if (i >= static_cast<int>(p.m) || out_col >= p.n) { continue; }
        float4 sum = across_warps[0][i][q];
#pragma unroll
        for (int w = 1; w < kWarps; ++w) {
            const float4 next = across_warps[w][i][q];
            sum.x += next.x;
            sum.y += next.y;
            sum.z += next.z;
            sum.w += next.w;
        }
        const float parts[4] = {sum.x, sum.y, sum.z, sum.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float value = p.alpha * parts[j];
            if (p.c != nullptr) {
                value += p.beta * p.c[static_cast<std::int64_t>(i) * p.c_row_stride +
                                      static_cast<std::int64_t>(out_col + j) * p.c_col_stride];
            }
            p.d[static_cast<std::int64_t>(i) * p.d_row_stride + static_cast<std::int64_t>(out_col + j) * p.d_col_stride] = value;
        }
    }
}

}  // namespace

const char* supportsSkinny(const FtcudaGemmDesc& desc) {
    if (desc.m == 0 || desc.m > 32) { return "more than 32 rows (or none) in A"; }
    if (desc.n == 0 || desc.k == 0) { return "the problem is empty"; }
    if (desc.n >= (1ULL << 31) || desc.k >= (1ULL << 31)) { return "an extent does not fit 31 bits"; }
    if (desc.n % 4 != 0) { return "n is not a multiple of 4"; }
    if (desc.b_col_stride != 1 || desc.b_row_stride % 4 != 0 || desc.b_row_stride < static_cast<std::int64_t>(desc.n)) {
        return "B is not row-major with a 16-byte row pitch";
    }
    if (reinterpret_cast<std::uintptr_t>(desc.b) % 16 != 0) { return "B is not 16-byte aligned"; }
    return nullptr;
}

int configureSkinny(LaunchState& state, char*, std::size_t) {
    const FtcudaGemmDesc& desc = state.desc;
    state.variant              = kVariantGeneric;
    state.grid_x               = static_cast<std::uint32_t>(ceilDiv(desc.n, kStripColumns));
    state.grid_y               = 1;
    state.grid_z               = 1;
    state.block                = kWarps * 32;
    state.smem_bytes           = 0;
    state.splits               = 1;
    state.workspace_bytes      = 0;
    state.row_tile             = desc.m <= 1 ? 1 : desc.m <= 4 ? 4 : desc.m <= 8 ? 8 : desc.m <= 16 ? 16 : 32;
    return 0;
}

cudaError_t launchSkinny(const LaunchState& state, cudaStream_t stream) {
    const FtcudaGemmDesc& desc = state.desc;
    SkinnyParams p{};
    p.a            = desc.a;
    p.b            = desc.b;
    p.c            = desc.c;
    p.d            = desc.d;
    p.a_row_stride = desc.a_row_stride;
    p.a_col_stride = desc.a_col_stride;
    p.b_row_stride = desc.b_row_stride;
    p.c_row_stride = desc.c_row_stride;
    p.c_col_stride = desc.c_col_stride;
    p.d_row_stride = desc.d_row_stride;
    p.d_col_stride = desc.d_col_stride;
    p.m            = static_cast<std::uint32_t>(desc.m);
    p.n            = static_cast<std::uint32_t>(desc.n);
    p.k            = static_cast<std::uint32_t>(desc.k);
    p.alpha        = desc.alpha;
    p.beta         = desc.beta;
    switch (state.row_tile) {
        case 1: skinnyGemm<1><<<state.grid_x, state.block, 0, stream>>>(p); break;
        case 4: skinnyGemm<4><<<state.grid_x, state.block, 0, stream>>>(p); break;
        case 8: skinnyGemm<8><<<state.grid_x, state.block, 0, stream>>>(p); break;
        case 16: skinnyGemm<16><<<state.grid_x, state.block, 0, stream>>>(p); break;
        default: skinnyGemm<32><<<state.grid_x, state.block, 0, stream>>>(p); break;
    }
    countLaunches(1);
    return cudaGetLastError();
}

}  // namespace ftcuda
