// Pieces shared by the 3xTF32 tensor-core kernels:
// kernel parameters, the walk over output tiles, the TF32 split and the
// epilogue's row-segment writer.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace ftcuda {
namespace tf32x3 {

constexpr int kTileN = 192;
constexpr int kTileK = 32;

// K blocks (of 32) accumulated inside the tensor core between two drains, by default: floor(sqrt(K) / 12.5)
// clamped to [1, 16] (see chunkKBlocks in gemm_tf32x3.cu for the measurements behind it).
inline std::uint32_t drainInterval(std::uint64_t k) {
    std::uint32_t blocks = 1;
    while (blocks < 16 && static_cast<std::uint64_t>(blocks + 1) * (blocks + 1) * 156 <= k) { ++blocks; }  // 12.5^2 = 156.25
    return blocks;
}

struct GroupEntry;

struct TensorParams {
    const float* c;
    float* d;
    std::int64_t c_row_stride, c_col_stride;
    std::int64_t d_row_stride, d_col_stride;
    std::uint32_t m, n, k;
    std::uint32_t tiles_m, tiles_n;
    std::uint32_t splits, k_per_split;
    std::uint32_t chunk_k_blocks;
    std::uint32_t band_m_tiles;  // M tiles walked together, so that concurrent CTAs share B panels in L2
    std::uint32_t a_m_contiguous;  // A was given contiguous along M (a transposed view): raw tile is [k][m]
    std::uint32_t b_k_contiguous;  // B was given contiguous along K (a transposed view): raw tile is [n][k], swizzled
    float alpha, beta;
    float* partials;  // non-null: raw sums to partials[split][m][n]
    // Scatter mode (scatter_rows != 0): alpha * sum is ADDED, element by element,
    // into the buffer of the row's owner -- dense [scatter_rows][n] matrices that
    // may live on other GPUs (peer-mapped) -- instead of being written to d.
    float* scatter[8];
    std::uint32_t scatter_rows;
    // Above 1: the K slices of a tile are the CTAs of a thread-block cluster (blockIdx.x = tile *
    // cluster_ranks + slice, one work item per CTA) and meet through distributed shared memory.
    std::uint32_t cluster_ranks;
    int* status;
    // Grouped launches: the per-group table and, per work item, the index of its group.
    const GroupEntry* groups;
    const std::uint32_t* item_group;
};

// Grouped launches (one persistent launch over the output tiles of many independent GEMMs): one
// entry per group in device memory, followed by the list that names the group of every work item.
// The entry holds what differs from group to group -- the two TMA descriptors, the output views and
// the extents --; alpha, beta and the operands' layout class are those of the launch.
struct alignas(128) GroupEntry {
    CUtensorMap map_a;
    CUtensorMap map_b;
    const float* c;
    float* d;
    std::int64_t c_row_stride, c_col_stride;
    std::int64_t d_row_stride, d_col_stride;
    std::uint32_t m, n, k;
    std::uint32_t chunk_k_blocks;
    std::uint32_t first_item;  // index of the group's first work item in the launch's list
    std::uint32_t tiles_m, tiles_n;
    std::uint32_t band_m_tiles;
};
static_assert(sizeof(GroupEntry) % 128 == 0, "entries are laid out back to back at 128-byte boundaries");

struct WorkItem {
    std::uint32_t tile_m, tile_n;  // element offsets
    std::uint32_t split;
    std::uint32_t k_begin, k_blocks;
};

// `tile_rows`: rows of A per work item.
template<bool kClustered = false>
__device__ __forceinline__ WorkItem decodeItem(const TensorParams& p, std::uint32_t item, std::uint32_t tile_rows) {
    const std::uint32_t tiles = p.tiles_m * p.tiles_n;
    WorkItem w;
    constexpr bool clustered  = kClustered;
    w.split                   = clustered ? item % p.cluster_ranks : item / tiles;
    const std::uint32_t tile  = clustered ? item / p.cluster_ranks : item - w.split * tiles;
    const std::uint32_t band  = tile / (p.band_m_tiles * p.tiles_n);
    const std::uint32_t first = band * p.band_m_tiles;
    const std::uint32_t rows  = min(p.band_m_tiles, p.tiles_m - first);
    const std::uint32_t rest  = tile - band * p.band_m_tiles * p.tiles_n;
    w.tile_m                  = (first + rest % rows) * tile_rows;
    w.tile_n                  = (rest / rows) * kTileN;
    w.k_begin                 = w.split * p.k_per_split;
    const std::uint32_t k_end = min(p.k, w.k_begin + p.k_per_split);
    w.k_blocks                = (k_end - w.k_begin + kTileK - 1) / kTileK;
    return w;
}

// One work item as a role of the kernel needs it: where the tile is, how deep K is, how often the
// accumulator is drained, and (grouped launches) the group's table entry.
struct ItemView {
    WorkItem w;
    std::uint32_t chunk_k_blocks;
    const GroupEntry* group;  // null for an ordinary launch
};

template<bool kClustered, bool kGrouped>
__device__ __forceinline__ ItemView fetchItem(const TensorParams& p, std::uint32_t item, std::uint32_t tile_rows) {
    ItemView view;
    if constexpr (kGrouped) {
        const GroupEntry* group   = p.groups + p.item_group[item];
        const std::uint32_t tile  = item - group->first_item;
        const std::uint32_t band  = tile / (group->band_m_tiles * group->tiles_n);
        const std::uint32_t first = band * group->band_m_tiles;
        const std::uint32_t rows  = min(group->band_m_tiles, group->tiles_m - first);
        const std::uint32_t rest  = tile - band * group->band_m_tiles * group->tiles_n;
        view.w.tile_m             = (first + rest % rows) * tile_rows;
        view.w.tile_n             = (rest / rows) * kTileN;
        view.w.split              = 0;
        view.w.k_begin            = 0;
        view.w.k_blocks           = (group->k + kTileK - 1) / kTileK;
        view.chunk_k_blocks       = group->chunk_k_blocks;
        view.group                = group;
    } else {
        view.w              = decodeItem<kClustered>(p, item, tile_rows);
        view.chunk_k_blocks = p.chunk_k_blocks;
        view.group          = nullptr;
    }
    return view;
}

// Rounds to TF32 (10 explicit mantissa bits), to nearest with ties away from zero -- what
// cvt.rna.tf32.f32 computes -- with integer instructions at full rate: the conversion unit has a
// fraction of the ALU's throughput and the converter warps are on the kernel's critical path. Adding
// half a TF32 ulp to the sign-magnitude bit pattern and clearing the low 13 bits rounds the
// magnitude. The sum is capped at the largest finite pattern of the value's sign first: a finite
// value within half a TF32 ulp of FLT_MAX would otherwise round up to infinity, and infinities and
// NaNs come out as that largest finite TF32 magnitude too, which is what splitTf32 wants.
__device__ __forceinline__ std::uint32_t tf32RoundSaturated(float value) {
    const std::uint32_t bits  = __float_as_uint(value);
    const std::uint32_t limit = (bits & 0x80000000U) | 0x7F7FFFFFU;
    return min(bits + 0x1000U, limit) & 0xFFFFE000U;
}

// value = hi + lo: hi is value rounded to TF32 (always finite), lo the FP32 remainder value - hi,
// which is exact for every finite value, FLT_MAX included. lo is handed to the tensor core as it is:
// kind::tf32 reads the upper 19 bits of a 32-bit operand and ignores the rest, so the remainder is
// truncated to TF32 by the hardware (what is cut off is below 2^-21 |value|) and no instruction is
// spent on rounding it. For value = +-inf: hi = +-(largest TF32), lo = +-inf; for a NaN: lo = NaN.
// The three products a_lo b_hi + a_hi b_lo + a_hi b_hi then give what IEEE FP32 arithmetic gives
// for a b -- +-inf, or NaN for inf * 0, inf - inf and NaN operands -- instead of a NaN made inside
// the split (inf - inf) or a NaN lost in it.
__device__ __forceinline__ void splitTf32(float value, std::uint32_t& hi, std::uint32_t& lo) {
    hi = tf32RoundSaturated(value);
    lo = __float_as_uint(value - __uint_as_float(hi));
}

// Element-wise tail of writeRowSegment for outputs that cannot take 128-bit stores.
static __device__ __noinline__ void writeRowSegmentSlow(float* out, std::int64_t out_row_stride, std::int64_t out_col_stride,
                                                 const float* c, std::int64_t c_row_stride, std::int64_t c_col_stride,
                                                 float scale, float beta, std::uint32_t row, std::uint32_t col,
                                                 std::uint32_t n, const float* sum) {
    for (std::uint32_t j = 0; j < 16 && col + j < n; ++j) {
        float value = scale * sum[j];
        if (c != nullptr) {
            value += beta * c[static_cast<std::int64_t>(row) * c_row_stride + static_cast<std::int64_t>(col + j) * c_col_stride];
        }
        out[static_cast<std::int64_t>(row) * out_row_stride + static_cast<std::int64_t>(col + j) * out_col_stride] = value;
    }
}

// Scatter mode: adds scale * sum[j] to target[j] for the (up to 16) columns left in the row. K slices of
// this GPU and of other GPUs all add into the owner's rows; the order of the additions is not fixed. The
// atomics have system scope: device-scope atomics of different GPUs are not atomic with one another.
static __device__ __noinline__ void addRowSegment(float* target, float scale, std::uint32_t columns_left, const float* sum) {
    for (std::uint32_t j = 0; j < 16 && j < columns_left; ++j) { atomicAdd_system(target + j, scale * sum[j]); }
}

// Writes one row segment of 16 consecutive columns held by one thread.
__device__ __forceinline__ void writeRowSegment(const TensorParams& p, const WorkItem& w, std::uint32_t row,
                                                std::uint32_t col, const float (&sum)[16], bool vector_ok) {
    if (row >= p.m || col >= p.n) { return; }
    if (p.scatter_rows != 0) {
        // Out of line, through a local copy: the common path keeps its registers.
        const std::uint32_t owner = row / p.scatter_rows;
        float copy[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) { copy[j] = sum[j]; }
        addRowSegment(p.scatter[owner] + static_cast<std::uint64_t>(row - owner * p.scatter_rows) * p.n + col, p.alpha,
                      p.n - col, copy);
        return;
    }
    const bool partial = p.partials != nullptr;
    float* out         = partial ? p.partials + static_cast<std::uint64_t>(w.split) * p.m * p.n : p.d;
    const std::int64_t out_row_stride = partial ? p.n : p.d_row_stride;
    const std::int64_t out_col_stride = partial ? 1 : p.d_col_stride;
    const bool with_c                 = !partial && p.c != nullptr;
    const float scale                 = partial ? 1.0F : p.alpha;
    if (vector_ok) {
        float* out_row     = out + static_cast<std::int64_t>(row) * out_row_stride + col;
        const float* c_row = with_c ? p.c + static_cast<std::int64_t>(row) * p.c_row_stride + col : nullptr;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            if (col + q * 4 >= p.n) { continue; }
            float4 value = make_float4(scale * sum[q * 4 + 0], scale * sum[q * 4 + 1], scale * sum[q * 4 + 2],
                                       scale * sum[q * 4 + 3]);
            if (with_c) {
                const float4 addend = *reinterpret_cast<const float4*>(c_row + q * 4);
                value.x += p.beta * addend.x;
                value.y += p.beta * addend.y;
                value.z += p.beta * addend.z;
                value.w += p.beta * addend.w;
            }
            *reinterpret_cast<float4*>(out_row + q * 4) = value;
        }
        return;
    }
    // Any strides, any alignment: handed to an out-of-line routine through a
    // local copy, so that the common path keeps `sum` in registers.
    float copy[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) { copy[j] = sum[j]; }
    writeRowSegmentSlow(out, out_row_stride, out_col_stride, with_c ? p.c : nullptr, p.c_row_stride, p.c_col_stride,
                        scale, p.beta, row, col, p.n, copy);
}

}  // namespace tf32x3
}  // namespace ftcuda
