// Exact-FP32 GEMM for very few rows of A (m <= 32): D = alpha * A * B + beta * C
// where the whole cost is reading B once. HBM-bound; algorithmic traffic
// 4 * (k * n + m * k + m * n [+ m * n]) bytes, of which k * n dominates.
//
// Work split. A strip of 128 columns of B belongs to one thread-block CLUSTER
// of up to 8 CTAs; the CTAs of a cluster take consecutive ranges of K, and the
// eight warps of a CTA take interleaved groups of four K rows inside the range.
// One warp instruction loads one K row of the strip: 32 lanes x 128 bits = 512
// contiguous bytes, and a warp keeps two to four groups (8-16 such loads) in
// flight. The rows of A are staged in shared memory 256 K rows at a time, so the
// four values A[i][k..k+3] a group needs for row i are one 128-bit shared load
// with the same address for the whole warp (a broadcast).
//
// Reduction, all in a fixed order (results are deterministic): the warps of a
// CTA add their partial sums one after the other into a shared-memory tile;
// after a cluster-wide barrier the first CTA of the cluster reads the other
// CTAs' tiles through distributed shared memory, adds them in rank order,
// applies alpha / beta and writes D. No workspace, no atomics.
//
// Sums are FP32 FFMA; the order over K differs from a sequential loop only by
// this fixed partition.
#include <cooperative_groups.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "gemm_kernels.hpp"

namespace ftcuda {
namespace {

namespace cg = cooperative_groups;

constexpr int kStripColumns = 128;
constexpr int kWarps        = 8;
constexpr int kGroupRows    = 4;   // K rows per group (one 128-bit load of A covers them)
constexpr int kChunkRows    = 256; // K rows of A staged in shared memory at a time
constexpr int kMaxCluster   = 8;

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
    std::uint32_t groups_per_cta;  // groups of four K rows per CTA of a cluster
    std::uint32_t rows_per_z;      // rows of A per blockIdx.z slab
    float alpha, beta;
};

// Streaming 128-bit load, zero when `valid` is false. Volatile, so that all
// loads of an iteration are issued, in program order, before the first use.
__device__ __forceinline__ float4 loadStreaming(const float* address, bool valid) {
    float4 value;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "mov.f32 %0, 0f00000000;\n\t"
        "mov.f32 %1, 0f00000000;\n\t"
        "mov.f32 %2, 0f00000000;\n\t"
        "mov.f32 %3, 0f00000000;\n\t"
        "@p ld.global.cs.v4.f32 {%0, %1, %2, %3}, [%4];\n\t"
        "}"
        : "=f"(value.x), "=f"(value.y), "=f"(value.z), "=f"(value.w)
        : "l"(address), "r"(static_cast<int>(valid)));
    return value;
}

template<int kRows>
__global__ void __launch_bounds__(kWarps * 32) skinnyGemm(const SkinnyParams p) {
    // Groups of B kept in flight per warp: more while the accumulators are few.
    constexpr int kAhead = kRows <= 8 ? 4 : 2;
    // The K range of a CTA is walked in chunks of kChunkRows rows; the chunk of
    // A that goes with it sits in shared memory, [row of A][k within chunk].
    // After the last chunk the same memory holds the CTA's partial sums,
    // [row of A][128 columns].
    __shared__ float4 shared_pool[kRows * kChunkRows / 4];
    float (*a_chunk)[kChunkRows] = reinterpret_cast<float (*)[kChunkRows]>(shared_pool);
    float4 (*tile)[32]           = reinterpret_cast<float4 (*)[32]>(shared_pool);
    static_assert(kChunkRows >= 128, "the partial-sum tile must fit the pool");

    cg::cluster_group cluster = cg::this_cluster();
    const unsigned rank       = cluster.block_rank();
    const unsigned ranks      = cluster.num_blocks();

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const std::uint32_t col = blockIdx.x * kStripColumns + lane * 4;
    const bool col_ok       = col < p.n;  // n % 4 == 0: a lane's four columns are all in or all out

    // blockIdx.z selects a slab of up to kRows rows of A (and of C and D).
    const std::uint32_t row0    = blockIdx.z * p.rows_per_z;
    const int slab_rows         = static_cast<int>(min(p.rows_per_z, p.m - row0));
    const float* const a_slab   = p.a + static_cast<std::int64_t>(row0) * p.a_row_stride;

    float4 acc[kRows];
#pragma unroll
    for (int i = 0; i < kRows; ++i) { acc[i] = make_float4(0.0F, 0.0F, 0.0F, 0.0F); }

    const std::uint32_t k_begin = rank * p.groups_per_cta * kGroupRows;
    const std::uint32_t k_end   = min(k_begin + p.groups_per_cta * kGroupRows, p.k);
    for (std::uint32_t chunk = k_begin; chunk < k_end; chunk += kChunkRows) {
        // Stage A[0..m)[chunk .. chunk + kChunkRows): zeros past the end of K.
        // Consecutive threads walk the unit-stride direction of A.
        __syncthreads();
        const bool k_fastest = p.a_col_stride == 1;
        for (int item = threadIdx.x; item < kRows * kChunkRows; item += kWarps * 32) {
            const int i  = k_fastest ? item / kChunkRows : item % kRows;
            const int kc = k_fastest ? item % kChunkRows : item / kRows;
            const std::uint32_t kk = chunk + kc;
            a_chunk[i][kc] = (i < slab_rows && kk < k_end)
                                 ? __ldg(a_slab + static_cast<std::int64_t>(i) * p.a_row_stride + static_cast<std::int64_t>(kk) * p.a_col_stride)
                                 : 0.0F;
        }
        __syncthreads();
        constexpr int kChunkGroups = kChunkRows / kGroupRows;
        for (int group = warp; group < kChunkGroups; group += kWarps * kAhead) {
            float4 b_value[kAhead][kGroupRows];
#pragma unroll
            for (int u = 0; u < kAhead; ++u) {
#pragma unroll
                for (int r = 0; r < kGroupRows; ++r) {
                    const std::uint32_t kk = chunk + (group + u * kWarps) * kGroupRows + r;
                    b_value[u][r] = loadStreaming(p.b + static_cast<std::int64_t>(kk) * p.b_row_stride + col,
                                                  group + u * kWarps < kChunkGroups && kk < k_end && col_ok);
                }
            }
#pragma unroll
            for (int u = 0; u < kAhead; ++u) {
                const int kc = (group + u * kWarps) * kGroupRows;
                if (group + u * kWarps >= kChunkGroups) { break; }
#pragma unroll
                for (int i = 0; i < kRows; ++i) {
                    // One 128-bit shared load, the same address for the whole warp.
                    const float4 four      = *reinterpret_cast<const float4*>(&a_chunk[i][kc]);
                    const float a_value[4] = {four.x, four.y, four.z, four.w};
#pragma unroll
                    for (int r = 0; r < kGroupRows; ++r) {
                        acc[i].x = fmaf(a_value[r], b_value[u][r].x, acc[i].x);
                        acc[i].y = fmaf(a_value[r], b_value[u][r].y, acc[i].y);
                        acc[i].z = fmaf(a_value[r], b_value[u][r].z, acc[i].z);
                        acc[i].w = fmaf(a_value[r], b_value[u][r].w, acc[i].w);
                    }
                }
            }
        }
    }
    __syncthreads();  // the pool changes its role

    // Warps fold into the shared tile one after the other.
    for (int turn = 0; turn < kWarps; ++turn) {
        if (warp == turn) {
#pragma unroll
            for (int i = 0; i < kRows; ++i) {
                if (turn == 0) {
                    tile[i][lane] = acc[i];
                } else {
                    float4 sum = tile[i][lane];
                    sum.x += acc[i].x;
                    sum.y += acc[i].y;
                    sum.z += acc[i].z;
                    sum.w += acc[i].w;
                    tile[i][lane] = sum;
                }
            }
        }
        __syncthreads();
    }
    cluster.sync();
    if (rank == 0) {
        for (int item = threadIdx.x; item < kRows * 32; item += kWarps * 32) {
            const int i                 = item >> 5;
            const int quad              = item & 31;
            const std::uint32_t out_col = blockIdx.x * kStripColumns + quad * 4;
            if (i >= slab_rows || out_col >= p.n) { continue; }
            const std::int64_t out_row = static_cast<std::int64_t>(row0) + i;
            float4 sum = tile[i][quad];
            for (unsigned other = 1; other < ranks; ++other) {
                const float4* remote = cluster.map_shared_rank(&tile[0][0], other);
                const float4 next    = remote[i * 32 + quad];
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
                    value += p.beta * p.c[out_row * p.c_row_stride + static_cast<std::int64_t>(out_col + j) * p.c_col_stride];
                }
                p.d[out_row * p.d_row_stride + static_cast<std::int64_t>(out_col + j) * p.d_col_stride] = value;
            }
        }
    }
    // Nobody's shared memory may go away while the first CTA still reads it.
    cluster.sync();
}

template<int kRows>
cudaError_t launchRows(const LaunchState& state, const SkinnyParams& p, cudaStream_t stream) {
    cudaLaunchConfig_t config{};
    config.gridDim          = dim3(state.grid_x, state.grid_y, state.grid_z);
    config.blockDim         = dim3(state.block, 1, 1);
    config.dynamicSmemBytes = 0;
    config.stream           = stream;
    cudaLaunchAttribute attribute{};
    attribute.id               = cudaLaunchAttributeClusterDimension;
    attribute.val.clusterDim.x = 1;
    attribute.val.clusterDim.y = state.grid_y;  // all K slices of a strip form one cluster
    attribute.val.clusterDim.z = 1;
    config.attrs               = &attribute;
    config.numAttrs            = 1;
    return cudaLaunchKernelEx(&config, skinnyGemm<kRows>, p);
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

int configureSkinny(LaunchState& state, char* message, std::size_t capacity) {
    const FtcudaGemmDesc& desc = state.desc;
    int sms                    = 0;
    if (!deviceSmCount(desc.device, &sms, message, capacity)) { return 1; }
    state.variant         = kVariantGeneric;
    state.grid_x          = static_cast<std::uint32_t>(ceilDiv(desc.n, kStripColumns));
    state.block           = kWarps * 32;
    state.smem_bytes      = 0;
    state.splits          = 1;
    state.workspace_bytes = 0;
    // Up to eight rows of A per CTA; more rows become slabs along blockIdx.z. The
    // slabs of a strip run side by side and read the same rows of B, which
    // therefore come from HBM once and from L2 for the other slabs. Eight rows
    // keep the accumulators small enough for sixteen loads in flight per warp.
    state.row_tile = desc.m <= 1 ? 1 : desc.m <= 2 ? 2 : desc.m <= 4 ? 4 : 8;
    state.grid_z   = static_cast<std::uint32_t>(ceilDiv(desc.m, state.row_tile));
    // CTAs per cluster (= K slices per strip): enough to put two CTAs on every
    // SM, as long as each CTA keeps at least two groups of K rows per warp.
    const std::uint64_t groups = ceilDiv(desc.k, kGroupRows);
    std::uint32_t cluster      = 1;
    while (cluster < kMaxCluster && static_cast<std::uint64_t>(state.grid_x) * state.grid_z * cluster < 2ULL * sms &&
           groups / (cluster * 2) >= 2ULL * kWarps) {
        cluster *= 2;
    }
    state.grid_y      = cluster;
    state.k_per_split = static_cast<std::uint32_t>(ceilDiv(groups, cluster));  // groups per CTA
    return 0;
}

cudaError_t launchSkinny(const LaunchState& state, cudaStream_t stream) {
    const FtcudaGemmDesc& desc = state.desc;
    SkinnyParams p{};
    p.a              = desc.a;
    p.b              = desc.b;
    p.c              = desc.c;
    p.d              = desc.d;
    p.a_row_stride   = desc.a_row_stride;
    p.a_col_stride   = desc.a_col_stride;
    p.b_row_stride   = desc.b_row_stride;
    p.c_row_stride   = desc.c_row_stride;
    p.c_col_stride   = desc.c_col_stride;
    p.d_row_stride   = desc.d_row_stride;
    p.d_col_stride   = desc.d_col_stride;
    p.m              = static_cast<std::uint32_t>(desc.m);
    p.n              = static_cast<std::uint32_t>(desc.n);
    p.k              = static_cast<std::uint32_t>(desc.k);
    p.groups_per_cta = state.k_per_split;
    p.rows_per_z     = state.row_tile;
    p.alpha          = desc.alpha;
    p.beta           = desc.beta;
    cudaError_t error = cudaSuccess;
    switch (state.row_tile) {
        case 1: error = launchRows<1>(state, p, stream); break;
        case 2: error = launchRows<2>(state, p, stream); break;
        case 4: error = launchRows<4>(state, p, stream); break;
        default: error = launchRows<8>(state, p, stream); break;
    }
    countLaunches(1);
    return error;
}

}  // namespace ftcuda
