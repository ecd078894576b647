// Exact-FP32 GEMM on the SIMT pipes: D = alpha * A * B + beta * C with every
// product and sum in IEEE FP32 (FFMA), sequential over K inside one thread --
// the arithmetic of the reference kernel (src/primitive/hygon/gemm/fp32_gemm.hip:18-31),
// re-tiled for B200.
//
// Two kernels:
//   * simtGemmTma: 128x128 output tile per CTA, 256 threads, 8x8 outputs per
//     thread. K is walked in blocks of 32. Operand tiles are fetched by TMA
//     into a 3-stage shared-memory ring guarded by mbarriers, so the copy of
//     blocks i+1 and i+2 overlaps the FFMA work on block i. The A tile is
//     stored with the 128-byte swizzle so that the 8 rows a thread owns are
//     read as bank-conflict-free 128-bit loads. Two CTAs are resident per SM
//     (96 KiB of shared memory each). The epilogue swaps half-rows between
//     the two half-warps with shuffles so that each store instruction of a
//     warp writes one full 512-byte row segment.
//   * simtGemmGeneric: 64x64 tile with predicated scalar loads; takes any
//     strides, any alignment, tiny shapes and K == 0. It is the path for
//     layouts TMA cannot describe.
//   * simtGemmSmall: 32x32 tile, one to four groups of 128 threads that take the K blocks in turn
//     (their sums are added in group order at the end), the next K block's operands
//     fetched into registers while the current one is multiplied. For outputs so
//     small that the larger tiles would leave most SMs idle (64^3 ... 256^3, the
//     128x64x96 default): sixteen times as many CTAs as the 128x128 tiling, each
//     with a short K loop whose global-memory latency is hidden. Any strides.
// All can restrict themselves to one K slice (blockIdx.z) and write the raw
// partial tile to a workspace, which the split-K reduction finishes.
#include <cuda_runtime.h>

#include <cstdint>

#include "gemm_kernels.hpp"
#include "ptx.cuh"

namespace ftcuda {
namespace {

constexpr int kTileM   = 128;
constexpr int kTileN   = 128;
constexpr int kTileK   = 32;
constexpr int kStages  = 3;
constexpr int kThreads = 256;
constexpr int kTileBytes  = kTileM * kTileK * 4;  // 16 KiB for either operand
constexpr int kStageBytes = 2 * kTileBytes;
// 1024 bytes of slack lets the kernel align the ring to the swizzle atom.
constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 64;

struct SimtParams {
    const float* c;
    float* d;
    std::int64_t c_row_stride, c_col_stride;
    std::int64_t d_row_stride, d_col_stride;
    std::uint32_t m, n, k;
    std::uint32_t k_per_split;  // K elements per blockIdx.z slice
    float alpha, beta;
    float* partials;            // non-null: write raw sums to partials[z][m][n]
    int* status;
};

// Output stage shared by both kernels' slow path: one element, any strides.
__device__ __forceinline__ void storeElement(const SimtParams& p, std::uint32_t row, std::uint32_t col, float sum) {
    if (row >= p.m || col >= p.n) { return; }
    if (p.partials != nullptr) {
        p.partials[(static_cast<std::uint64_t>(blockIdx.z) * p.m + row) * p.n + col] = sum;
        return;
    }
    float value = p.alpha * sum;
    if (p.c != nullptr) {
        value += p.beta * p.c[static_cast<std::int64_t>(row) * p.c_row_stride + static_cast<std::int64_t>(col) * p.c_col_stride];
    }
    p.d[static_cast<std::int64_t>(row) * p.d_row_stride + static_cast<std::int64_t>(col) * p.d_col_stride] = value;
}

// kAContiguousK: the A tile is [128 rows][32 k] with 128-byte rows, swizzled;
// otherwise it is [32 k][128 rows], linear (A was given contiguous along M).
template<bool kAContiguousK, bool kBContiguousK>
__global__ void __launch_bounds__(kThreads, 2)
simtGemmTma(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const SimtParams p) {
    extern __shared__ unsigned char smem_raw[];
    // Ring of stages at a 1024-byte boundary, barriers behind it.
    const std::uint32_t ring_offset = (1024 - (smemAddress(smem_raw) & 1023)) & 1023;
    unsigned char* ring             = smem_raw + ring_offset;
    std::uint64_t* full             = reinterpret_cast<std::uint64_t*>(ring + kStages * kStageBytes);
    __shared__ int abort_flag;

    const int tid  = threadIdx.x;
    const int tx   = tid & 15;
    const int ty   = tid >> 4;
    const int lane = tid & 31;

    const std::uint32_t tile_m = blockIdx.y * kTileM;
    const std::uint32_t tile_n = blockIdx.x * kTileN;
    const std::uint32_t k_begin = blockIdx.z * p.k_per_split;
    const std::uint32_t k_end   = min(p.k, k_begin + p.k_per_split);
    const int k_blocks          = static_cast<int>((k_end - k_begin + kTileK - 1) / kTileK);

    if (tid == 0) {
        abort_flag = 0;
        for (int s = 0; s < kStages; ++s) { mbarrierInit(&full[s], 1); }
        fenceBarrierInit();
        prefetchTensorMap(&map_a);
        prefetchTensorMap(&map_b);
    }
    __syncthreads();

    // One thread feeds the ring. Out-of-range parts of a box (M, N and K
    // tails) arrive as zeros, which contribute nothing to the sums.
    auto issue = [&](int block) {
        const int s                = block % kStages;
        unsigned char* stage       = ring + s * kStageBytes;
        const std::int32_t k_coord = static_cast<std::int32_t>(k_begin + block * kTileK);
        mbarrierArriveExpectTx(&full[s], kStageBytes);
        if (kAContiguousK) {
            tmaLoad2d(stage, &map_a, &full[s], k_coord, static_cast<std::int32_t>(tile_m));
        } else {
            tmaLoad2d(stage, &map_a, &full[s], static_cast<std::int32_t>(tile_m), k_coord);
        }
        if (kBContiguousK) {
            tmaLoad2d(stage + kTileBytes, &map_b, &full[s], k_coord, static_cast<std::int32_t>(tile_n));
        } else {
            tmaLoad2d(stage + kTileBytes, &map_b, &full[s], static_cast<std::int32_t>(tile_n), k_coord);
        }
    };
    if (tid == 0) {
        for (int block = 0; block < kStages - 1 && block < k_blocks; ++block) { issue(block); }
    }

    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
#pragma unroll
        for (int j = 0; j < 8; ++j) { acc[i][j] = 0.0F; }
    }

    bool healthy = true;
    for (int block = 0; block < k_blocks; ++block) {
        const int s = block % kStages;
        // Refill the stage that block-1 used (all threads passed the barrier at
        // the end of that iteration, so nobody reads it any more).
        if (tid == 0 && block + kStages - 1 < k_blocks) { issue(block + kStages - 1); }
        if (!mbarrierWait(&full[s], (block / kStages) & 1, &abort_flag)) {
            abort_flag = 1;
            healthy    = false;
        }
        // A thread whose wait ran out has raised the CTA's flag; it multiplies what the stage holds all
        // the same and every thread reads the flag behind the barrier that ends the block, where the
        // tile is abandoned by all of them together: one block-wide barrier per K block.
        const unsigned char* a_tile = ring + s * kStageBytes;
        const unsigned char* b_tile = a_tile + kTileBytes;
#pragma unroll
        for (int k4 = 0; k4 < kTileK / 4; ++k4) {
            float a_frag[8][4];
            if (kAContiguousK) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int row      = ty * 8 + i;
                    const float4 value = *reinterpret_cast<const float4*>(a_tile + row * 128 + ((k4 ^ (row & 7)) << 4));
                    a_frag[i][0] = value.x;
                    a_frag[i][1] = value.y;
                    a_frag[i][2] = value.z;
                    a_frag[i][3] = value.w;
                }
            } else {
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) {
                    const float4* row = reinterpret_cast<const float4*>(a_tile + (k4 * 4 + kk) * (kTileM * 4) + ty * 32);
                    const float4 lo   = row[0];
                    const float4 hi   = row[1];
                    a_frag[0][kk] = lo.x;
                    a_frag[1][kk] = lo.y;
                    a_frag[2][kk] = lo.z;
                    a_frag[3][kk] = lo.w;
                    a_frag[4][kk] = hi.x;
                    a_frag[5][kk] = hi.y;
                    a_frag[6][kk] = hi.z;
                    a_frag[7][kk] = hi.w;
                }
            }
            if (kBContiguousK) {
                // B tile is [128 n][32 k], rows of 128 bytes with the 128-byte swizzle.
                // A thread owns columns j * 16 + tx: the 8 lanes of a quarter-warp read
                // 8 consecutive rows, i.e. 8 different 16-byte chunk positions.
                float b_frag[8][4];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int column   = j * 16 + tx;
                    const float4 value = *reinterpret_cast<const float4*>(b_tile + column * 128 + ((k4 ^ (column & 7)) << 4));
                    b_frag[j][0] = value.x;
                    b_frag[j][1] = value.y;
                    b_frag[j][2] = value.z;
                    b_frag[j][3] = value.w;
                }
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        // Columns forwards in even rows, backwards in odd ones (see the other branch).
#pragma unroll
                        for (int step = 0; step < 8; ++step) {
                            const int j = (i & 1) ? 7 - step : step;
                            acc[i][j] = fmaf(a_frag[i][kk], b_frag[j][kk], acc[i][j]);
                        }
                    }
                }
            } else {
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) {
                    const unsigned char* b_row = b_tile + (k4 * 4 + kk) * (kTileN * 4);
                    const float4 b0            = *reinterpret_cast<const float4*>(b_row + tx * 16);
                    const float4 b1            = *reinterpret_cast<const float4*>(b_row + 256 + tx * 16);
                    const float b_frag[8]      = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        // The columns are walked forwards in even rows and backwards in odd ones: every FFMA
                        // then shares an operand with the one before it (A within a row, B at the turn), which
                        // the compiler keeps in this order -- 54.8 against 52.8 TFLOP/s on 4096^3; columns on
                        // the outside lose (49.2).
#pragma unroll
                        for (int step = 0; step < 8; ++step) {
                            const int j = (i & 1) ? 7 - step : step;
                            acc[i][j] = fmaf(a_frag[i][kk], b_frag[j], acc[i][j]);
                        }
                    }
                }
            }
        }
        // This thread's reads of the stage (generic proxy) before its refill by TMA (async proxy).
        fenceProxyAsync();
        __syncthreads();
        if (*static_cast<volatile int*>(&abort_flag) != 0) {
            healthy = false;
            break;
        }
    }
    if (!healthy) {
        // Give up on the tile: report, then let the copies that are still in
        // flight land (bounded) before the CTA's shared memory is released.
        if (tid == 0) {
            if (p.status != nullptr) { *p.status = 1; }
            int never = 0;
            for (int s = 0; s < kStages; ++s) {
                mbarrierWait(&full[s], 0, &never);
                mbarrierWait(&full[s], 1, &never);
            }
        }
        return;
    }

    if (kBContiguousK) {
        // Columns j * 16 + tx: for one (i, j) the 16 lanes of a half-warp write 16
        // consecutive columns of one row.
#pragma unroll
        for (int i = 0; i < 8; ++i) {
#pragma unroll
            for (int j = 0; j < 8; ++j) { storeElement(p, tile_m + ty * 8 + i, tile_n + j * 16 + tx, acc[i][j]); }
        }
        return;
    }

    // Epilogue. Lanes 0-15 of a warp own rows ty_even*8+i, lanes 16-31 rows
    // ty_odd*8+i, each as two 4-column groups (tx*4.. and 64+tx*4..). One
    // shuffle round trades half-rows so that, per store instruction, the 32
    // lanes cover 128 consecutive columns of ONE row.
    const bool upper          = lane >= 16;
    const std::uint32_t col   = tile_n + (upper ? 64 : 0) + tx * 4;
    const std::uint32_t row_a = tile_m + (ty & ~1) * 8;  // row block of the even half-warp
    float* out                = p.partials != nullptr
                                    ? p.partials + static_cast<std::uint64_t>(blockIdx.z) * p.m * p.n
                                    : p.d;
    const std::int64_t out_row_stride = p.partials != nullptr ? p.n : p.d_row_stride;
    const std::int64_t out_col_stride = p.partials != nullptr ? 1 : p.d_col_stride;
    const bool scale                  = p.partials == nullptr;
    const bool with_c                 = scale && p.c != nullptr;
    const bool vector_ok =
        out_col_stride == 1 && (out_row_stride & 3) == 0 && (reinterpret_cast<std::uintptr_t>(out) & 15) == 0 &&
        (p.n & 3) == 0 &&
        (!with_c || (p.c_col_stride == 1 && (p.c_row_stride & 3) == 0 && (reinterpret_cast<std::uintptr_t>(p.c) & 15) == 0));
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float4 first  = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
        const float4 second = make_float4(acc[i][4], acc[i][5], acc[i][6], acc[i][7]);
        const float4 send   = upper ? first : second;
        float4 recv;
        recv.x = __shfl_xor_sync(0xFFFFFFFFU, send.x, 16);
        recv.y = __shfl_xor_sync(0xFFFFFFFFU, send.y, 16);
        recv.z = __shfl_xor_sync(0xFFFFFFFFU, send.z, 16);
        recv.w = __shfl_xor_sync(0xFFFFFFFFU, send.w, 16);
        const float4 part[2]       = {upper ? recv : first, upper ? second : recv};
        const std::uint32_t row[2] = {row_a + i, row_a + 8 + i};
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            if (row[h] >= p.m) { continue; }
            if (vector_ok) {
                if (col >= p.n) { continue; }
                float4 value = part[h];
                if (scale) {
                    value.x *= p.alpha;
                    value.y *= p.alpha;
                    value.z *= p.alpha;
                    value.w *= p.alpha;
                }
                if (with_c) {
                    const float4 addend =
                        *reinterpret_cast<const float4*>(p.c + static_cast<std::int64_t>(row[h]) * p.c_row_stride + col);
                    value.x += p.beta * addend.x;
                    value.y += p.beta * addend.y;
                    value.z += p.beta * addend.z;
                    value.w += p.beta * addend.w;
                }
                *reinterpret_cast<float4*>(out + static_cast<std::int64_t>(row[h]) * out_row_stride + col) = value;
            } else {
                storeElement(p, row[h], col + 0, part[h].x);
                storeElement(p, row[h], col + 1, part[h].y);
                storeElement(p, row[h], col + 2, part[h].z);
                storeElement(p, row[h], col + 3, part[h].w);
            }
        }
    }
}

// ---- generic path ----

constexpr int kGenericTile = 64;
constexpr int kGenericK    = 16;

struct GenericParams {
    const float* a;
    const float* b;
    std::int64_t a_row_stride, a_col_stride;
    std::int64_t b_row_stride, b_col_stride;
    SimtParams out;
};

__global__ void __launch_bounds__(256) simtGemmGeneric(const GenericParams g) {
    __shared__ float a_tile[kGenericK][kGenericTile + 4];
    __shared__ float b_tile[kGenericK][kGenericTile + 4];
    const SimtParams& p = g.out;
    const int tid       = threadIdx.x;
    const int tx        = tid & 15;
    const int ty        = tid >> 4;
    const std::uint32_t tile_m  = blockIdx.y * kGenericTile;
    const std::uint32_t tile_n  = blockIdx.x * kGenericTile;
    const std::uint32_t k_begin = blockIdx.z * p.k_per_split;
    const std::uint32_t k_end   = min(p.k, k_begin + p.k_per_split);

    float acc[4][4] = {};
    for (std::uint32_t k0 = k_begin; k0 < k_end; k0 += kGenericK) {
        // 64 x 16 elements per operand, 4 per thread; consecutive threads walk
        // the K index of A and the N index of B.
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int index         = tid + e * 256;
            const int a_k           = index & 15;
            const int a_m           = index >> 4;
            const std::uint32_t row = tile_m + a_m;
            const std::uint32_t kk  = k0 + a_k;
            a_tile[a_k][a_m] = (row < p.m && kk < k_end)
                                   ? g.a[static_cast<std::int64_t>(row) * g.a_row_stride + static_cast<std::int64_t>(kk) * g.a_col_stride]
                                   : 0.0F;
            const int b_n            = index & 63;
            const int b_k            = index >> 6;
            const std::uint32_t col  = tile_n + b_n;
            const std::uint32_t kk_b = k0 + b_k;
            b_tile[b_k][b_n] = (col < p.n && kk_b < k_end)
                                   ? g.b[static_cast<std::int64_t>(kk_b) * g.b_row_stride + static_cast<std::int64_t>(col) * g.b_col_stride]
                                   : 0.0F;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kGenericK; ++kk) {
            float a_frag[4];
            float b_frag[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                a_frag[i] = a_tile[kk][ty * 4 + i];
                b_frag[i] = b_tile[kk][tx * 4 + i];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
#pragma unroll
                for (int j = 0; j < 4; ++j) { acc[i][j] = fmaf(a_frag[i], b_frag[j], acc[i][j]); }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int j = 0; j < 4; ++j) { storeElement(p, tile_m + ty * 4 + i, tile_n + tx * 4 + j, acc[i][j]); }
    }
}

// ---- small outputs: 32 x 32 tiles, 2 x 4 outputs per thread ----
// A tile is one CTA of kGroups groups of 128 threads. With one such CTA per SM a group of four warps has
// a scheduler each to itself and the K loop is a chain of latencies (fetch, park, 32 steps of three
// shared loads and eight FFMAs), so the groups take the K blocks in turn -- group g the blocks g,
// g + kGroups, ... -- each with its own pair of tiles and its own barrier, and their sums are added in
// group order at the end: the loop of a thread is kGroups times shorter.
constexpr int kSmallTile         = 32;
constexpr int kSmallK            = 32;
constexpr int kSmallGroupThreads = 128;
// Measured (device time back to back): 256^3 10.3 -> 8.3 us, 200 x 1000 x 130 30.7 -> 22.6, 256 x 512 x 256 16.4 -> 14.4 with four
// groups; with a K of 64 or 128 the extra threads and the final addition cost what the shorter loop saves
// (128 x 64 x 96: 4.6 -> 5.7 us with two groups), so those keep one group.
__host__ __device__ constexpr int smallGroups(std::uint64_t k) { return k >= 8 * kSmallK ? 4 : 1; }

__device__ __forceinline__ void groupBarrier(int group) {
    asm volatile("bar.sync %0, %1;" ::"r"(group + 1), "n"(kSmallGroupThreads) : "memory");
}

template<int kGroups>
__global__ void __launch_bounds__(kSmallGroupThreads* kGroups) simtGemmSmall(const GenericParams g) {
    // Per group: [k][m] and [k][n], rows of A padded so that its transposing stores do not collide.
    __shared__ float a_tiles[kGroups][kSmallK][kSmallTile + 1];
    __shared__ __align__(16) float b_tiles[kGroups][kSmallK][kSmallTile];
    const SimtParams& p = g.out;
    const int group     = threadIdx.x / kSmallGroupThreads;
    const int tid       = threadIdx.x % kSmallGroupThreads;
    const int tx        = tid & 7;    // 8 column groups of 4
    const int ty        = tid >> 3;   // 16 row groups of 2
    float (*a_tile)[kSmallTile + 1] = a_tiles[group];
    float (*b_tile)[kSmallTile]     = b_tiles[group];
    const std::uint32_t tile_m  = blockIdx.y * kSmallTile;
    const std::uint32_t tile_n  = blockIdx.x * kSmallTile;
    const std::uint32_t k_begin = blockIdx.z * p.k_per_split;
    const std::uint32_t k_end   = min(p.k, k_begin + p.k_per_split);

    // Per K block a thread fetches 8 elements of A and 8 of B. A: consecutive threads walk K within
    // a row when rows are contiguous along K, M otherwise (so that the loads of a warp coalesce for
    // either layout); B: consecutive threads walk N, or K when B is contiguous along K.
    const bool a_along_k = g.a_col_stride == 1;
    const bool b_along_n = g.b_col_stride == 1;
    float a_next[8];
    float b_next[8];
    auto fetch = [&](std::uint32_t k0) {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const int index         = tid + e * kSmallGroupThreads;  // 0 .. 1023
            const int a_k           = a_along_k ? (index & 31) : (index >> 5);
            const int a_m           = a_along_k ? (index >> 5) : (index & 31);
            const std::uint32_t row = tile_m + a_m;
            const std::uint32_t kk  = k0 + a_k;
            a_next[e] = (row < p.m && kk < k_end)
                            ? g.a[static_cast<std::int64_t>(row) * g.a_row_stride + static_cast<std::int64_t>(kk) * g.a_col_stride]
                            : 0.0F;
            const int b_n            = b_along_n ? (index & 31) : (index >> 5);
            const int b_k            = b_along_n ? (index >> 5) : (index & 31);
            const std::uint32_t col  = tile_n + b_n;
            const std::uint32_t kk_b = k0 + b_k;
            b_next[e] = (col < p.n && kk_b < k_end)
                            ? g.b[static_cast<std::int64_t>(kk_b) * g.b_row_stride + static_cast<std::int64_t>(col) * g.b_col_stride]
                            : 0.0F;
        }
    };
    auto park = [&]() {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const int index = tid + e * kSmallGroupThreads;
            a_tile[a_along_k ? (index & 31) : (index >> 5)][a_along_k ? (index >> 5) : (index & 31)] = a_next[e];
            b_tile[b_along_n ? (index >> 5) : (index & 31)][b_along_n ? (index & 31) : (index >> 5)] = b_next[e];
        }
    };

    float acc[2][4] = {};
    constexpr std::uint32_t kStride = kSmallK * kGroups;
    const std::uint32_t k_first     = k_begin + group * kSmallK;
    if (k_first < k_end) { fetch(k_first); }
    for (std::uint32_t k0 = k_first; k0 < k_end; k0 += kStride) {
        park();
        groupBarrier(group);
        if (k0 + kStride < k_end) { fetch(k0 + kStride); }  // in flight while this block is multiplied
#pragma unroll
        for (int kk = 0; kk < kSmallK; ++kk) {
            const float a0     = a_tile[kk][ty * 2];
            const float a1     = a_tile[kk][ty * 2 + 1];
            const float4 b_row = *reinterpret_cast<const float4*>(&b_tile[kk][tx * 4]);
            acc[0][0] = fmaf(a0, b_row.x, acc[0][0]);
            acc[0][1] = fmaf(a0, b_row.y, acc[0][1]);
            acc[0][2] = fmaf(a0, b_row.z, acc[0][2]);
            acc[0][3] = fmaf(a0, b_row.w, acc[0][3]);
            acc[1][0] = fmaf(a1, b_row.x, acc[1][0]);
            acc[1][1] = fmaf(a1, b_row.y, acc[1][1]);
            acc[1][2] = fmaf(a1, b_row.z, acc[1][2]);
            acc[1][3] = fmaf(a1, b_row.w, acc[1][3]);
        }
        groupBarrier(group);
    }
    if constexpr (kGroups > 1) {
        // The groups' sums meet in the first group, added in group order (the result does not depend on
        // which group finishes first). Every group parks into its own B tile, idle by now.
        float* parked = &b_tiles[group][0][0];
        if (group > 0) {
#pragma unroll
            for (int i = 0; i < 8; ++i) { parked[i * kSmallGroupThreads + tid] = acc[i >> 2][i & 3]; }
        }
        __syncthreads();
        if (group > 0) { return; }
#pragma unroll
        for (int other = 1; other < kGroups; ++other) {
#pragma unroll
            for (int i = 0; i < 8; ++i) { acc[i >> 2][i & 3] += b_tiles[other][0][i * kSmallGroupThreads + tid]; }
        }
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
#pragma unroll
        for (int j = 0; j < 4; ++j) { storeElement(p, tile_m + ty * 2 + i, tile_n + tx * 4 + j, acc[i][j]); }
    }
}

SimtParams makeOutputParams(const LaunchState& state, void* workspace) {
    const FtcudaGemmDesc& desc = state.desc;
    SimtParams p{};
    p.c            = desc.c;
    p.d            = desc.d;
    p.c_row_stride = desc.c_row_stride;
    p.c_col_stride = desc.c_col_stride;
    p.d_row_stride = desc.d_row_stride;
    p.d_col_stride = desc.d_col_stride;
    p.m            = static_cast<std::uint32_t>(desc.m);
    p.n            = static_cast<std::uint32_t>(desc.n);
    p.k            = static_cast<std::uint32_t>(desc.k);
    p.k_per_split  = state.k_per_split;
    p.alpha        = desc.alpha;
    p.beta         = desc.beta;
    p.partials     = state.splits > 1 ? static_cast<float*>(workspace) : nullptr;
    p.status       = state.device_status;
    return p;
}

}  // namespace

const char* supportsSimt(const FtcudaGemmDesc& desc, bool split_k) {
    if (desc.m >= (1ULL << 31) || desc.n >= (1ULL << 31) || desc.k >= (1ULL << 31)) {
        return "an extent does not fit 31 bits";
    }
    if (ceilDiv(desc.m, kGenericTile) > 65535) { return "more than 65535 row tiles"; }
    if (split_k) {
        if (desc.m * desc.n == 0) { return "the output is empty"; }
        if (desc.k < 2 * 256) { return "K is too short to split"; }
    }
    return nullptr;
}

int configureSimt(LaunchState& state, bool split_k, char* message, std::size_t capacity) {
    const FtcudaGemmDesc& desc = state.desc;
    int sms                    = 0;
    if (!deviceSmCount(desc.device, &sms, message, capacity)) { return 1; }
    if (!deviceStatusWord(desc.device, &state.device_status, &state.host_status, message, capacity)) { return 1; }

    // TMA path: both operands describable and at least one full-size tile of
    // work; otherwise the generic kernel.
    const bool b_n   = tmaEligible(desc.b, desc.b_col_stride, desc.b_row_stride, desc.n, desc.k);
    const bool b_k   = !b_n && tmaEligible(desc.b, desc.b_row_stride, desc.b_col_stride, desc.k, desc.n);
    const bool b_ok  = b_n || b_k;
    const bool a_k   = tmaEligible(desc.a, desc.a_col_stride, desc.a_row_stride, desc.k, desc.m);
    const bool a_m   = tmaEligible(desc.a, desc.a_row_stride, desc.a_col_stride, desc.m, desc.k);
    const bool large = desc.m >= 96 && desc.n >= 96 && desc.k >= 32;
    state.variant    = kVariantGeneric;
    if (b_ok && large && (a_k || a_m)) { state.variant = (a_k ? kVariantTmaAk : kVariantTmaAm) | (b_k ? kVariantFlagBk : 0); }
    // Small outputs: the tiling above would occupy a handful of SMs with long serial K loops (one CTA
    // for 128^3). 32 x 32 tiles put sixteen times as many CTAs to work; used while they still fit one
    // wave with room to spare and the whole-K loop of a tile stays short. (Split-K launches keep the
    // larger tiles: they are chosen for long K.)
    const std::uint64_t small_tiles = ceilDiv(desc.m, kSmallTile) * ceilDiv(desc.n, kSmallTile);
    const std::uint64_t tiles_now   = state.variant == kVariantGeneric ? ceilDiv(desc.m, kGenericTile) * ceilDiv(desc.n, kGenericTile)
                                                                       : ceilDiv(desc.m, kTileM) * ceilDiv(desc.n, kTileN);
    if (!split_k && desc.k > 0 && desc.k <= 1024 && tiles_now * 4 <= static_cast<std::uint64_t>(sms) &&
        small_tiles <= 2ULL * static_cast<std::uint64_t>(sms)) {
        state.variant = kVariantSmall;
    }

    const bool small           = state.variant == kVariantSmall;
    const std::uint32_t tile_m = small ? kSmallTile : state.variant == kVariantGeneric ? kGenericTile : kTileM;
    const std::uint32_t tile_n = small ? kSmallTile : state.variant == kVariantGeneric ? kGenericTile : kTileN;
    const std::uint32_t tile_k = small ? kSmallK : state.variant == kVariantGeneric ? kGenericK : kTileK;
    state.grid_x               = static_cast<std::uint32_t>(ceilDiv(desc.n, tile_n));
    state.grid_y               = static_cast<std::uint32_t>(ceilDiv(desc.m, tile_m));
    state.block                = small ? kSmallGroupThreads * smallGroups(desc.k) : kThreads;
    state.smem_bytes           = (state.variant == kVariantGeneric || small) ? 0 : kSmemBytes;

    state.splits      = 1;
    state.k_per_split = static_cast<std::uint32_t>(ceilDiv(desc.k == 0 ? 1 : desc.k, tile_k) * tile_k);
    if (split_k) {
        // Enough K slices to give every SM two CTAs, each slice at least 256 deep.
        const std::uint64_t tiles = static_cast<std::uint64_t>(state.grid_x) * state.grid_y;
        std::uint64_t splits      = ceilDiv(2ULL * sms, tiles);
        const std::uint64_t most  = desc.k / 256;
        if (splits > most) { splits = most; }
        if (splits > 64) { splits = 64; }
        if (splits < 2) { splits = 2; }
        state.k_per_split = static_cast<std::uint32_t>(ceilDiv(ceilDiv(desc.k, splits), tile_k) * tile_k);
        state.splits      = static_cast<std::uint32_t>(ceilDiv(desc.k, state.k_per_split));
    }
    state.grid_z          = state.splits;
    state.workspace_bytes = state.splits > 1 ? static_cast<std::uint64_t>(state.splits) * desc.m * desc.n * sizeof(float) : 0;

    if (state.variant != kVariantGeneric && state.variant != kVariantSmall) {
        const std::uint64_t a_pitch =
            static_cast<std::uint64_t>((state.variant & kVariantMaskA) == kVariantTmaAk ? desc.a_row_stride : desc.a_col_stride) * sizeof(float);
        const bool a_encoded =
            (state.variant & kVariantMaskA) == kVariantTmaAk
                ? encodeTensorMap2d(&state.map_a, desc.a, desc.k, desc.m, a_pitch, kTileK, kTileM, true, message, capacity)
                : encodeTensorMap2d(&state.map_a, desc.a, desc.m, desc.k, a_pitch, kTileM, kTileK, false, message, capacity);
        if (!a_encoded) { return 1; }
        const bool b_encoded =
            b_k ? encodeTensorMap2d(&state.map_b, desc.b, desc.k, desc.n, static_cast<std::uint64_t>(desc.b_col_stride) * sizeof(float),
                                    kTileK, kTileN, kSwizzle128, message, capacity)
                : encodeTensorMap2d(&state.map_b, desc.b, desc.n, desc.k, static_cast<std::uint64_t>(desc.b_row_stride) * sizeof(float),
                                    kTileN, kTileK, kSwizzleNone, message, capacity);
        if (!b_encoded) { return 1; }
        // Opting in to 97 KiB of dynamic shared memory is a per-device setting.
        cudaError_t error = cudaSuccess;
        const void* kernels[4] = {reinterpret_cast<const void*>(simtGemmTma<true, false>), reinterpret_cast<const void*>(simtGemmTma<false, false>),
                                  reinterpret_cast<const void*>(simtGemmTma<true, true>), reinterpret_cast<const void*>(simtGemmTma<false, true>)};
        for (const void* kernel : kernels) {
            if (error == cudaSuccess) { error = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes); }
        }
        if (error != cudaSuccess) {
            return fail(message, capacity, 1, "cudaFuncSetAttribute failed: %s", cudaGetErrorString(error));
        }
    }
    return 0;
}

void planSimtGenericSplitK(LaunchState& state, std::uint32_t splits) {
    const FtcudaGemmDesc& desc = state.desc;
    state.variant              = kVariantGeneric;
    state.grid_x               = static_cast<std::uint32_t>(ceilDiv(desc.n, kGenericTile));
    state.grid_y               = static_cast<std::uint32_t>(ceilDiv(desc.m, kGenericTile));
    state.block                = kThreads;
    state.smem_bytes           = 0;
    state.k_per_split = static_cast<std::uint32_t>(ceilDiv(ceilDiv(desc.k, splits), kGenericK) * kGenericK);
    state.splits      = static_cast<std::uint32_t>(ceilDiv(desc.k, state.k_per_split));
    state.grid_z      = state.splits;
    state.workspace_bytes = static_cast<std::uint64_t>(state.splits) * desc.m * desc.n * sizeof(float);
}

cudaError_t launchSimt(const LaunchState& state, void* workspace, cudaStream_t stream) {
    const SimtParams out = makeOutputParams(state, workspace);
    const dim3 grid(state.grid_x, state.grid_y, state.grid_z);
    if (state.variant == kVariantGeneric || state.variant == kVariantSmall) {
        GenericParams g{};
        g.a            = state.desc.a;
        g.b            = state.desc.b;
        g.a_row_stride = state.desc.a_row_stride;
        g.a_col_stride = state.desc.a_col_stride;
        g.b_row_stride = state.desc.b_row_stride;
        g.b_col_stride = state.desc.b_col_stride;
        g.out          = out;
        if (state.variant == kVariantSmall) {
            switch (state.block / kSmallGroupThreads) {
                case 4: simtGemmSmall<4><<<grid, state.block, 0, stream>>>(g); break;
                case 2: simtGemmSmall<2><<<grid, state.block, 0, stream>>>(g); break;
                default: simtGemmSmall<1><<<grid, state.block, 0, stream>>>(g); break;
            }
        } else {
            simtGemmGeneric<<<grid, state.block, 0, stream>>>(g);
        }
    } else {
        const bool a_k = (state.variant & kVariantMaskA) == kVariantTmaAk;
        const bool b_k = (state.variant & kVariantFlagBk) != 0;
        if (a_k && !b_k) {
            simtGemmTma<true, false><<<grid, state.block, state.smem_bytes, stream>>>(state.map_a, state.map_b, out);
        } else if (!a_k && !b_k) {
            simtGemmTma<false, false><<<grid, state.block, state.smem_bytes, stream>>>(state.map_a, state.map_b, out);
        } else if (a_k) {
            simtGemmTma<true, true><<<grid, state.block, state.smem_bytes, stream>>>(state.map_a, state.map_b, out);
        } else {
            simtGemmTma<false, true><<<grid, state.block, state.smem_bytes, stream>>>(state.map_a, state.map_b, out);
        }
    }
    cudaError_t error = cudaGetLastError();
    std::uint64_t launches = 1;
    if (error == cudaSuccess && state.splits > 1) {
        error = launchSplitKReduce(state.desc, static_cast<const float*>(workspace), state.splits, stream);
        ++launches;
    }
    countLaunches(launches);
    return error;
}

}  // namespace ftcuda
