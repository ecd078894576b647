// Exact-FP32 GEMM for very few rows of A (m <= 32): D = alpha * A * B + beta * C
// where the whole cost is reading B once. HBM-bound up to about 16 rows (beyond
// that the FP32 pipe catches up); algorithmic traffic
// 4 * (k * n + m * k + m * n [+ m * n]) bytes, of which k * n dominates.
//
// Work split. A strip of 128 columns of B belongs to one thread-block CLUSTER
// of up to 8 CTAs; the CTAs of a cluster take consecutive ranges of K (whole
// boxes of 32 rows). Inside a CTA the range streams through a ring of
// shared-memory slots filled by TMA, one 32 x 128 box (16 KiB) per copy, so
// that 64-144 KiB per CTA are in flight without holding registers. Warp 0
// issues the copies; all eight warps consume: each takes four rows of every
// box, one 128-bit shared load per row (32 lanes x 16 bytes = the 512-byte row,
// conflict free), and releases the slot as soon as the values are in registers.
// The rows of A that go with the range are staged in shared memory 128 K values
// at a time by asynchronous copies, one stage ahead, so the four values
// A[i][k..k+3] a warp needs for row i are one 128-bit shared load with the same
// address for the whole warp (a broadcast). All rows of A (templates for 1, 2,
// 4, 8, 16, 24, 32) are accumulated by the same CTA, so B leaves HBM once.
//
// Reduction, all in a fixed order (results are deterministic): the warps of a
// CTA park their sums in shared memory and each element is summed in warp
// order; each CTA of the cluster owns a share of the strip's columns and
// receives the other CTAs' sums for them through distributed shared memory;
// after one cluster barrier the owner adds them in rank order, applies
// alpha / beta and writes D. No workspace, no atomics.
//
// Every wait on an mbarrier is bounded; a wait that runs out sets the CTA's
// abort flag, the CTA skips its remaining work, still meets the cluster
// barriers and reports through the status word (D is then undefined).
//
// Sums are FP32 FFMA; the order over K differs from a sequential loop only by
// this fixed partition.
#include <cooperative_groups.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "gemm_kernels.hpp"
#include "ptx.cuh"

namespace ftcuda {
namespace {

namespace cg = cooperative_groups;

constexpr int kStripColumns = 128;
constexpr int kWarps        = 8;
constexpr int kThreads      = kWarps * 32;
constexpr int kBoxRows      = 32;                 // K rows per TMA box: four per consumer warp
constexpr int kBoxBytes     = kBoxRows * kStripColumns * 4;
constexpr int kMaxCluster   = 8;
static_assert(kBoxRows == kWarps * 4, "a consumer warp takes four rows of a box");

// Per row count: up to 16 rows of A two CTAs share an SM (five boxes in flight
// each); 24 and 32 rows need most of the register file, one CTA per SM with ten
// boxes in flight.
__host__ __device__ constexpr int slots(int rows) { return rows <= 16 ? 5 : 10; }
constexpr int kStageRows = 128;  // K values of each row of A per stage (four boxes); two stages in shared memory
__host__ __device__ constexpr int ctasPerSm(int rows) { return rows <= 16 ? 2 : 1; }
// Shared memory: ring | two A stages | received partial sums | barriers.
__host__ __device__ constexpr int ringBytes(int rows) { return slots(rows) * kBoxBytes; }
__host__ __device__ constexpr int stageBytes(int rows) { return 2 * rows * kStageRows * 4; }
__host__ __device__ constexpr int receiveBytes(int rows) { return rows * kStripColumns * 4; }
constexpr std::uint32_t smemBytes(int rows) {
    return 127 + ringBytes(rows) + stageBytes(rows) + receiveBytes(rows) + 2 * slots(rows) * 8;
}

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
    std::uint32_t rows_per_cta;    // K rows per CTA of a cluster, a multiple of the box
    std::uint32_t rows_per_z;      // rows of A per blockIdx.z slab
    float alpha, beta;
    int* status;  // mapped host word, set when a wait ran out
};

// The cluster barrier in its two halves; every thread of every CTA executes both.
__device__ __forceinline__ void clusterArrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void clusterWait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

// Asynchronous copies global -> shared that hold no registers while in flight;
// `bytes` (0 ... size) are read, the rest of the destination is zero-filled.
__device__ __forceinline__ void copyAsync4(void* destination, const float* source, std::uint32_t bytes) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(smemAddress(destination)), "l"(source), "r"(bytes) : "memory");
}
__device__ __forceinline__ void copyAsync16(void* destination, const float* source, std::uint32_t bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smemAddress(destination)), "l"(source), "r"(bytes) : "memory");
}
__device__ __forceinline__ void copyAsyncCommit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void copyAsyncWaitAll() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ float4 add4(float4 x, float4 y) { return make_float4(x.x + y.x, x.y + y.y, x.z + y.z, x.w + y.w); }

template<int kRows>
__global__ void __launch_bounds__(kThreads, ctasPerSm(kRows))
skinnyGemm(const __grid_constant__ CUtensorMap map_b, const SkinnyParams p) {
    constexpr int kSlots = slots(kRows);
    static_assert(kStageRows % kBoxRows == 0, "stages hold whole boxes");
    static_assert(kWarps * kRows * kStripColumns * 4 <= ringBytes(kRows), "the per-warp partial sums reuse the ring");

    extern __shared__ unsigned char smem_raw[];
    const std::uint32_t align_offset = (128 - (smemAddress(smem_raw) & 127)) & 127;
    unsigned char* ring              = smem_raw + align_offset;
    // [stage parity][row of A][k within the stage]
    float (*a_stage)[kRows][kStageRows] = reinterpret_cast<float (*)[kRows][kStageRows]>(ring + ringBytes(kRows));
    // [rank of the sender][row][quad within the receiver's share of the strip]
    float4* received                 = reinterpret_cast<float4*>(ring + ringBytes(kRows) + stageBytes(kRows));
    std::uint64_t* full  = reinterpret_cast<std::uint64_t*>(ring + ringBytes(kRows) + stageBytes(kRows) + receiveBytes(kRows));
    std::uint64_t* empty = full + kSlots;
    // After the K loop the ring holds every warp's partial sums: [warp][row][quad].
    float4 (*part)[kRows][32] = reinterpret_cast<float4 (*)[kRows][32]>(ring);
    __shared__ int abort_flag;
    __shared__ int never_abort;

    cg::cluster_group cluster = cg::this_cluster();
    const unsigned rank       = cluster.block_rank();
    const unsigned ranks      = cluster.num_blocks();  // 1, 2, 4 or 8

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const std::uint32_t strip_col = blockIdx.x * kStripColumns;

    // blockIdx.z selects a slab of up to kRows rows of A (and of C and D).
    const std::uint32_t row0  = blockIdx.z * p.rows_per_z;
    const int slab_rows       = static_cast<int>(min(p.rows_per_z, p.m - row0));
    const float* const a_slab = p.a + static_cast<std::int64_t>(row0) * p.a_row_stride;

    // K range of this CTA: whole boxes of 32 rows.
    const std::uint32_t k_begin = min(rank * p.rows_per_cta, p.k);
    const std::uint32_t k_end   = min(k_begin + p.rows_per_cta, p.k);
    const std::uint32_t boxes   = (k_end - k_begin + kBoxRows - 1) / kBoxRows;

    if (threadIdx.x == 0) {
        abort_flag  = 0;
        never_abort = 0;
        for (int s = 0; s < kSlots; ++s) {
            mbarrierInit(&full[s], 1);
            mbarrierInit(&empty[s], kWarps);
        }
        fenceBarrierInit();
        prefetchTensorMap(&map_b);
    }
    // The set-up above overlaps the tail of the kernel before this one in the stream; nothing below
    // touches global memory before that kernel has completed.
    gridDependencyWait();
    gridDependencyLaunchDependents();
    __syncthreads();
    // First half of a cluster barrier whose only purpose is "every CTA of the
    // cluster runs": its second half sits in front of the first remote store.
    clusterArrive();

    float4 acc[kRows];
#pragma unroll
    for (int i = 0; i < kRows; ++i) { acc[i] = make_float4(0.0F, 0.0F, 0.0F, 0.0F); }

    // Warp 0 doubles as the producer. Before the loop it fills every slot; inside
    // the loop, once it has taken box b into registers, it waits until all warps
    // have released box b-1 (they release right after their loads, so this is
    // short) and refills that slot with box b-1+kSlots.
    std::uint32_t issued = 0;  // boxes handed to TMA (tracked by warp 0)
    auto issue_box = [&](std::uint32_t box) {
        const std::uint32_t s = box % kSlots;
        mbarrierArriveExpectTx(&full[s], kBoxBytes);
        tmaLoad2d(ring + s * kBoxBytes, &map_b, &full[s], static_cast<std::int32_t>(strip_col),
                  static_cast<std::int32_t>(k_begin + box * kBoxRows));
    };
    if (warp == 0) {
        issued = min(boxes, static_cast<std::uint32_t>(kSlots));
        if (lane == 0) {
            for (std::uint32_t box = 0; box < issued; ++box) { issue_box(box); }
        }
        __syncwarp();
    }
    {
        // The rows of A for this CTA's K range are staged kStageRows at a time with
        // asynchronous copies, one stage ahead of the boxes being multiplied.
        const bool vector_copies = p.a_col_stride == 1 && (p.a_row_stride & 3) == 0 &&
                                   (reinterpret_cast<std::uintptr_t>(a_slab) & 15) == 0;
        auto stage_in = [&](std::uint32_t stage_begin, int parity) {
            if (vector_copies) {
                // Four consecutive K values per copy; k_begin is a multiple of 32, so they are 16-byte aligned.
                for (int item = threadIdx.x; item < kRows * (kStageRows / 4); item += kThreads) {
                    const int i            = item / (kStageRows / 4);
                    const int kc           = (item % (kStageRows / 4)) * 4;
                    const std::uint32_t kk = stage_begin + kc;
                    const bool valid       = i < slab_rows && kk < k_end;
                    const std::uint32_t bytes = valid ? min(k_end - kk, 4U) * 4U : 0U;
                    copyAsync16(&a_stage[parity][i][kc], valid ? a_slab + static_cast<std::int64_t>(i) * p.a_row_stride + kk : p.a, bytes);
                }
            } else {
                // Any strides: one element per copy, consecutive threads along the unit-stride direction of A.
                const bool k_fastest = p.a_col_stride == 1;
                for (int item = threadIdx.x; item < kRows * kStageRows; item += kThreads) {
                    const int i            = k_fastest ? item / kStageRows : item % kRows;
                    const int kc           = k_fastest ? item % kStageRows : item / kRows;
                    const std::uint32_t kk = stage_begin + kc;
                    const bool valid       = i < slab_rows && kk < k_end;
                    copyAsync4(&a_stage[parity][i][kc],
                               valid ? a_slab + static_cast<std::int64_t>(i) * p.a_row_stride + static_cast<std::int64_t>(kk) * p.a_col_stride : p.a,
                               valid ? 4U : 0U);
                }
            }
            copyAsyncCommit();
        };
        bool ok = true;
        if (k_begin < k_end) { stage_in(k_begin, 0); }
        int parity = 0;
        for (std::uint32_t stage_begin = k_begin; stage_begin < k_end; stage_begin += kStageRows, parity ^= 1) {
            // This thread's copies of the stage have landed; after the barrier so have
            // everybody's, and every warp is done with the other stage.
            copyAsyncWaitAll();
            __syncthreads();
            if (stage_begin + kStageRows < k_end) { stage_in(stage_begin + kStageRows, parity ^ 1); }
            const std::uint32_t first_box = (stage_begin - k_begin) / kBoxRows;
            const std::uint32_t last_box  = min(first_box + kStageRows / kBoxRows, boxes);
            for (std::uint32_t box = first_box; box < last_box && ok; ++box) {
                const std::uint32_t s = box % kSlots;
                ok = __all_sync(0xFFFFFFFFU, mbarrierWait(&full[s], (box / kSlots) & 1, &abort_flag));
                if (!ok) {
                    abort_flag = 1;
                    break;
                }
                // Warp w owns rows 4w..4w+3 of the box: one 128-bit load per row,
                // 32 lanes x 16 bytes = the 512-byte row.
                const unsigned char* rows = ring + s * kBoxBytes + (warp * 4) * (kStripColumns * 4) + lane * 16;
                const int kc              = static_cast<int>(box - first_box) * kBoxRows + warp * 4;
                float4 b_value[4];
#pragma unroll
                for (int r = 0; r < 4; ++r) { b_value[r] = *reinterpret_cast<const float4*>(rows + r * (kStripColumns * 4)); }
                // The box is in registers now. The proxy fence orders these generic-proxy reads before
                // the TMA write that refills the slot.
                fenceProxyAsync();
                __syncwarp();
                if (lane == 0) { mbarrierArrive(&empty[s]); }
                if (warp == 0 && box >= 1 && issued < boxes) {
                    const std::uint32_t freed = box - 1;  // its slot takes box freed + kSlots == issued
                    if (!__all_sync(0xFFFFFFFFU, mbarrierWait(&empty[freed % kSlots], (freed / kSlots) & 1, &abort_flag))) {
                        abort_flag = 1;
                        ok         = false;
                        break;
                    }
                    if (lane == 0) { issue_box(issued); }
                    ++issued;
                    __syncwarp();
                }
#pragma unroll
                for (int i = 0; i < kRows; ++i) {
                    const float4 four      = *reinterpret_cast<const float4*>(&a_stage[parity][i][kc]);
                    const float a_value[4] = {four.x, four.y, four.z, four.w};
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        acc[i].x = fmaf(a_value[r], b_value[r].x, acc[i].x);
                        acc[i].y = fmaf(a_value[r], b_value[r].y, acc[i].y);
                        acc[i].z = fmaf(a_value[r], b_value[r].z, acc[i].z);
                        acc[i].w = fmaf(a_value[r], b_value[r].w, acc[i].w);
                    }
                }
            }
        }
    }
    __syncthreads();  // every box is consumed: the ring changes its role
    const bool failed = abort_flag != 0;
    if (failed) {
        // Copies still in flight must land before this CTA's shared memory goes away.
        if (warp == 0 && lane == 0) {
            for (std::uint32_t box = issued > kSlots ? issued - kSlots : 0; box < issued; ++box) {
                mbarrierWait(&full[box % kSlots], (box / kSlots) & 1, &never_abort);
            }
        }
        if (threadIdx.x == 0 && p.status != nullptr) { *p.status = 3; }
    }

    // ---- reduction, in a fixed order throughout.
    // (1) Every consumer warp parks its sums; then each (row, quad) is summed over
    //     the warps in warp order.
    // (2) The strip's 32 quads of columns are shared out among the CTAs of the
    //     cluster; every CTA sends each of its sums to the owner's `received`
    //     array (a remote shared-memory store), in the slot of the sender's rank.
    // (3) After the cluster barrier the owner adds the ranks' contributions in
    //     rank order, applies alpha and beta and writes D. Nobody touches remote
    //     shared memory after the barrier, so CTAs may leave independently.
    if (!failed) {
#pragma unroll
        for (int i = 0; i < kRows; ++i) { part[warp][i][lane] = acc[i]; }
    }
    __syncthreads();
    clusterWait();  // second half of the start-up barrier: long complete by now
    const unsigned quads_per_rank = 32 / ranks;
    if (!failed) {
        for (int item = threadIdx.x; item < kRows * 32; item += kThreads) {
            const int i    = item >> 5;
            const int quad = item & 31;
            float4 sum     = part[0][i][quad];
#pragma unroll
            for (int w = 1; w < kWarps; ++w) { sum = add4(sum, part[w][i][quad]); }
            const unsigned owner = quad / quads_per_rank;
            float4* remote       = cluster.map_shared_rank(received, owner);
            remote[(rank * kRows + i) * quads_per_rank + quad % quads_per_rank] = sum;
        }
    }
    clusterArrive();
    clusterWait();
    if (abort_flag == 0) {
        for (int item = threadIdx.x; item < kRows * static_cast<int>(quads_per_rank); item += kThreads) {
            const int i                 = item / quads_per_rank;
            const unsigned local_quad   = item % quads_per_rank;
            const std::uint32_t out_col = strip_col + (rank * quads_per_rank + local_quad) * 4;
            if (i >= slab_rows || out_col >= p.n) { continue; }
            float4 contribution[kMaxCluster];
#pragma unroll
            for (unsigned r = 0; r < kMaxCluster; ++r) {
                contribution[r] = r < ranks ? received[(r * kRows + i) * quads_per_rank + local_quad] : make_float4(0.0F, 0.0F, 0.0F, 0.0F);
            }
            float4 sum = contribution[0];
#pragma unroll
            for (unsigned r = 1; r < kMaxCluster; ++r) {
                if (r < ranks) { sum = add4(sum, contribution[r]); }
            }
            const std::int64_t out_row = static_cast<std::int64_t>(row0) + i;
            const float parts[4]       = {sum.x, sum.y, sum.z, sum.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (out_col + j >= p.n) { continue; }
                float value = p.alpha * parts[j];
                if (p.c != nullptr) {
                    value += p.beta * p.c[out_row * p.c_row_stride + static_cast<std::int64_t>(out_col + j) * p.c_col_stride];
                }
                p.d[out_row * p.d_row_stride + static_cast<std::int64_t>(out_col + j) * p.d_col_stride] = value;
            }
        }
    }
}

// ---------------------------------------------------------------------------
// The same problem with B given contiguous along K (dims (k, n), strides
// (1, pitch): the transposed view of an n x k weight matrix W, as in x @ W^T).
// Every output column is then the dot product of a row of A with a row of W.
// A strip is 32 rows of W; a box is 32 rows x 128 K values (16 KiB, rows of 512
// bytes). Warp w takes rows 4w..4w+3 of every box, a lane takes four K values of
// each (one conflict-free 128-bit shared load per row), multiplies them with
// the matching four values of every row of A (128-bit shared loads at
// consecutive addresses) and keeps rows x 4 scalar sums. At the end the 32
// lanes' sums are added by a butterfly of shuffles, the CTAs of the cluster (K
// slices) send theirs to the first CTA through distributed shared memory, and
// that CTA adds them in rank order and writes D. Ring, producer, A stages (one
// box = one stage of 128 K values) and bounded waits as above.
constexpr int kBtStripRows = 32;   // rows of W (= output columns) per strip
constexpr int kBtBoxK      = 128;  // K values per box
static_assert(kBtStripRows * kBtBoxK * 4 == kBoxBytes, "both box shapes have the same size");
static_assert(kBtBoxK == kStageRows, "one box per A stage");
__host__ __device__ constexpr int receiveBytesBt(int rows) { return kMaxCluster * rows * kBtStripRows * 4; }
constexpr std::uint32_t smemBytesBt(int rows) {
    return 127 + ringBytes(rows) + stageBytes(rows) + receiveBytesBt(rows) + 2 * slots(rows) * 8;
}

template<int kRows>
__global__ void __launch_bounds__(kThreads, ctasPerSm(kRows))
skinnyGemmBt(const __grid_constant__ CUtensorMap map_b, const SkinnyParams p) {
    constexpr int kSlots = slots(kRows);
    extern __shared__ unsigned char smem_raw[];
    const std::uint32_t align_offset = (128 - (smemAddress(smem_raw) & 127)) & 127;
    unsigned char* ring              = smem_raw + align_offset;
    // [stage parity][row of A][k within the box]
    float (*a_stage)[kRows][kBtBoxK] = reinterpret_cast<float (*)[kRows][kBtBoxK]>(ring + ringBytes(kRows));
    // first CTA only: [rank of the sender][row of A][row of W within the strip]
    float* received      = reinterpret_cast<float*>(ring + ringBytes(kRows) + stageBytes(kRows));
    std::uint64_t* full  = reinterpret_cast<std::uint64_t*>(ring + ringBytes(kRows) + stageBytes(kRows) + receiveBytesBt(kRows));
    std::uint64_t* empty = full + kSlots;
    __shared__ int abort_flag;
    __shared__ int never_abort;

    cg::cluster_group cluster = cg::this_cluster();
    const unsigned rank       = cluster.block_rank();
    const unsigned ranks      = cluster.num_blocks();

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const std::uint32_t strip_row = blockIdx.x * kBtStripRows;  // first row of W = first output column

    const int slab_rows = static_cast<int>(min(static_cast<std::uint32_t>(kRows), p.m));

    const std::uint32_t k_begin = min(rank * p.rows_per_cta, p.k);
    const std::uint32_t k_end   = min(k_begin + p.rows_per_cta, p.k);
    const std::uint32_t boxes   = (k_end - k_begin + kBtBoxK - 1) / kBtBoxK;

    if (threadIdx.x == 0) {
        abort_flag  = 0;
        never_abort = 0;
        for (int s = 0; s < kSlots; ++s) {
            mbarrierInit(&full[s], 1);
            mbarrierInit(&empty[s], kWarps);
        }
        fenceBarrierInit();
        prefetchTensorMap(&map_b);
    }
    // The set-up above overlaps the tail of the kernel before this one in the stream; nothing below
    // touches global memory before that kernel has completed.
    gridDependencyWait();
    gridDependencyLaunchDependents();
    __syncthreads();
    clusterArrive();  // "every CTA of the cluster runs", second half before the first remote store

    float acc[kRows][4];
#pragma unroll
    for (int i = 0; i < kRows; ++i) {
#pragma unroll
        for (int r = 0; r < 4; ++r) { acc[i][r] = 0.0F; }
    }

    std::uint32_t issued = 0;
    auto issue_box = [&](std::uint32_t box) {
        const std::uint32_t s = box % kSlots;
        mbarrierArriveExpectTx(&full[s], kBoxBytes);
        tmaLoad2d(ring + s * kBoxBytes, &map_b, &full[s], static_cast<std::int32_t>(k_begin + box * kBtBoxK),
                  static_cast<std::int32_t>(strip_row));
    };
    if (warp == 0) {
        issued = min(boxes, static_cast<std::uint32_t>(kSlots));
        if (lane == 0) {
            for (std::uint32_t box = 0; box < issued; ++box) { issue_box(box); }
        }
        __syncwarp();
    }
    const bool vector_copies = p.a_col_stride == 1 && (p.a_row_stride & 3) == 0 && (reinterpret_cast<std::uintptr_t>(p.a) & 15) == 0;
    auto stage_in = [&](std::uint32_t stage_begin, int parity) {
        if (vector_copies) {
            for (int item = threadIdx.x; item < kRows * (kBtBoxK / 4); item += kThreads) {
                const int i            = item / (kBtBoxK / 4);
                const int kc           = (item % (kBtBoxK / 4)) * 4;
                const std::uint32_t kk = stage_begin + kc;
                const bool valid       = i < slab_rows && kk < k_end;
                const std::uint32_t bytes = valid ? min(k_end - kk, 4U) * 4U : 0U;
                copyAsync16(&a_stage[parity][i][kc], valid ? p.a + static_cast<std::int64_t>(i) * p.a_row_stride + kk : p.a, bytes);
            }
        } else {
            const bool k_fastest = p.a_col_stride == 1;
            for (int item = threadIdx.x; item < kRows * kBtBoxK; item += kThreads) {
                const int i            = k_fastest ? item / kBtBoxK : item % kRows;
                const int kc           = k_fastest ? item % kBtBoxK : item / kRows;
                const std::uint32_t kk = stage_begin + kc;
                const bool valid       = i < slab_rows && kk < k_end;
                copyAsync4(&a_stage[parity][i][kc],
                           valid ? p.a + static_cast<std::int64_t>(i) * p.a_row_stride + static_cast<std::int64_t>(kk) * p.a_col_stride : p.a,
                           valid ? 4U : 0U);
            }
        }
        copyAsyncCommit();
    };
    bool ok = true;
    if (boxes > 0) { stage_in(k_begin, 0); }
    for (std::uint32_t box = 0; box < boxes; ++box) {
        const int parity = static_cast<int>(box & 1);
        copyAsyncWaitAll();
        __syncthreads();  // this box's values of A are in place; everybody is done with the other stage
        if (box + 1 < boxes) { stage_in(k_begin + (box + 1) * kBtBoxK, parity ^ 1); }
        if (!ok) { continue; }
        const std::uint32_t s = box % kSlots;
        ok = __all_sync(0xFFFFFFFFU, mbarrierWait(&full[s], (box / kSlots) & 1, &abort_flag));
        if (!ok) {
            abort_flag = 1;
            continue;
        }
        const unsigned char* rows = ring + s * kBoxBytes + (warp * 4) * (kBtBoxK * 4) + lane * 16;
        float4 b_value[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) { b_value[r] = *reinterpret_cast<const float4*>(rows + r * (kBtBoxK * 4)); }
        fenceProxyAsync();  // reads of the slot before its refill by TMA
        __syncwarp();
        if (lane == 0) { mbarrierArrive(&empty[s]); }
        if (warp == 0 && box >= 1 && issued < boxes) {
            const std::uint32_t freed = box - 1;
            if (!__all_sync(0xFFFFFFFFU, mbarrierWait(&empty[freed % kSlots], (freed / kSlots) & 1, &abort_flag))) {
                abort_flag = 1;
                ok         = false;
                continue;
            }
            if (lane == 0) { issue_box(issued); }
            ++issued;
            __syncwarp();
        }
#pragma unroll
        for (int i = 0; i < kRows; ++i) {
            const float4 a_value = *reinterpret_cast<const float4*>(&a_stage[parity][i][lane * 4]);
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                float sum = acc[i][r];
                sum       = fmaf(a_value.x, b_value[r].x, sum);
                sum       = fmaf(a_value.y, b_value[r].y, sum);
                sum       = fmaf(a_value.z, b_value[r].z, sum);
                sum       = fmaf(a_value.w, b_value[r].w, sum);
                acc[i][r] = sum;
            }
        }
    }
    __syncthreads();
    const bool failed = abort_flag != 0;
    if (failed) {
        if (warp == 0 && lane == 0) {
            for (std::uint32_t box = issued > kSlots ? issued - kSlots : 0; box < issued; ++box) {
                mbarrierWait(&full[box % kSlots], (box / kSlots) & 1, &never_abort);
            }
        }
        if (threadIdx.x == 0 && p.status != nullptr) { *p.status = 3; }
    }

    // Lanes hold sums over disjoint K values: butterfly over the warp, then value
    // number v (of rows x 4) is sent by lane v % 32 to the first CTA.
    clusterWait();
    float* remote = cluster.map_shared_rank(received, 0);
#pragma unroll
    for (int i = 0; i < kRows; ++i) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            float sum = acc[i][r];
#pragma unroll
            for (int offset = 16; offset >= 1; offset >>= 1) { sum += __shfl_xor_sync(0xFFFFFFFFU, sum, offset); }
            if (!failed && lane == ((i * 4 + r) & 31)) { remote[(rank * kRows + i) * kBtStripRows + warp * 4 + r] = sum; }
        }
    }
    clusterArrive();
    clusterWait();
    if (rank == 0 && abort_flag == 0) {
        for (int item = threadIdx.x; item < kRows * kBtStripRows; item += kThreads) {
            const int i                 = item / kBtStripRows;
            const int column            = item % kBtStripRows;
            const std::uint32_t out_col = strip_row + column;
            if (i >= slab_rows || out_col >= p.n) { continue; }
            float sum = received[i * kBtStripRows + column];
            for (unsigned r = 1; r < ranks; ++r) { sum += received[(r * kRows + i) * kBtStripRows + column]; }
            float value = p.alpha * sum;
            if (p.c != nullptr) { value += p.beta * p.c[static_cast<std::int64_t>(i) * p.c_row_stride + static_cast<std::int64_t>(out_col) * p.c_col_stride]; }
            p.d[static_cast<std::int64_t>(i) * p.d_row_stride + static_cast<std::int64_t>(out_col) * p.d_col_stride] = value;
        }
    }
}

template<int kRows>
cudaError_t allowSharedMemory() {
    return cudaFuncSetAttribute(skinnyGemm<kRows>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smemBytes(kRows)));
}

template<int kRows>
cudaError_t allowSharedMemoryBt() {
    return cudaFuncSetAttribute(skinnyGemmBt<kRows>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smemBytesBt(kRows)));
}

template<int kRows>
cudaError_t launchRows(const LaunchState& state, const SkinnyParams& p, cudaStream_t stream) {
    cudaLaunchConfig_t config{};
    config.gridDim          = dim3(state.grid_x, state.grid_y, state.grid_z);
    config.blockDim         = dim3(state.block, 1, 1);
    config.dynamicSmemBytes = state.smem_bytes;
    config.stream           = stream;
    cudaLaunchAttribute attributes[2] = {};
    attributes[0].id               = cudaLaunchAttributeClusterDimension;
    attributes[0].val.clusterDim.x = 1;
    attributes[0].val.clusterDim.y = state.grid_y;  // all K slices of a strip form one cluster
    attributes[0].val.clusterDim.z = 1;
    // The kernels wait for their predecessor in the stream by themselves (gridDependencyWait), so
    // their CTAs could start while that predecessor drains. Measured back to back at k = n = 4096:
    // a gain for the B-along-K form (22.8 -> 20.9 us at 8 rows), a loss for the row-major form
    // (14.6 -> 16.7 us at 1 row, 18.7 -> 23.0 us at 8), so only the former asks for it.
    attributes[1].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs                                             = attributes;
    if ((state.variant & kVariantFlagBk) != 0) {
        config.numAttrs = 2;
        return cudaLaunchKernelEx(&config, skinnyGemmBt<kRows>, state.map_b, p);
    }
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, skinnyGemm<kRows>, state.map_b, p);
}

}  // namespace

const char* supportsSkinny(const FtcudaGemmDesc& desc) {
    if (desc.m == 0 || desc.m > 32) { return "more than 32 rows (or none) in A"; }
    if (desc.n == 0 || desc.k == 0) { return "the problem is empty"; }
    if (desc.n >= (1ULL << 31) || desc.k >= (1ULL << 31)) { return "an extent does not fit 31 bits"; }
    if (!tmaEligible(desc.b, desc.b_col_stride, desc.b_row_stride, desc.n, desc.k) &&
        !tmaEligible(desc.b, desc.b_row_stride, desc.b_col_stride, desc.k, desc.n)) {
        return "B is neither row-major nor a transposed row-major view with a 16-byte aligned base and pitch";
    }
    return nullptr;
}

int configureSkinny(LaunchState& state, char* message, std::size_t capacity) {
    const FtcudaGemmDesc& desc = state.desc;
    int sms                    = 0;
    if (!deviceSmCount(desc.device, &sms, message, capacity)) { return 1; }
    if (!deviceStatusWord(desc.device, &state.device_status, &state.host_status, message, capacity)) { return 1; }
    const bool b_k_contiguous = !tmaEligible(desc.b, desc.b_col_stride, desc.b_row_stride, desc.n, desc.k);
    state.variant         = b_k_contiguous ? kVariantFlagBk : kVariantGeneric;
    const std::uint32_t strip = b_k_contiguous ? kBtStripRows : kStripColumns;  // output columns per strip
    const std::uint32_t box_k = b_k_contiguous ? kBtBoxK : kBoxRows;            // K values per box
    state.grid_x          = static_cast<std::uint32_t>(ceilDiv(desc.n, strip));
    state.block           = kThreads;
    state.splits          = 1;
    state.workspace_bytes = 0;
    // All rows of A (at most 32) stay in one CTA's registers, so B is read once.
    state.row_tile   = desc.m <= 1 ? 1 : desc.m <= 2 ? 2 : desc.m <= 4 ? 4 : desc.m <= 8 ? 8 : desc.m <= 16 ? 16 : desc.m <= 24 ? 24 : 32;
    state.grid_z     = 1;
    const int rows   = static_cast<int>(state.row_tile);
    state.smem_bytes = b_k_contiguous ? smemBytesBt(rows) : smemBytes(rows);
    // CTAs per cluster (= K slices per strip): as many as still fit the GPU in one
    // wave, as long as each CTA keeps at least four boxes.
    const std::uint64_t resident = static_cast<std::uint64_t>(sms) * ctasPerSm(rows);
    const std::uint64_t boxes    = ceilDiv(desc.k, box_k);
    std::uint32_t cluster        = 1;
    while (cluster < kMaxCluster && static_cast<std::uint64_t>(state.grid_x) * cluster * 2 <= resident && boxes / (cluster * 2) >= 4) {
        cluster *= 2;
    }
    state.grid_y      = cluster;
    state.k_per_split = static_cast<std::uint32_t>(ceilDiv(boxes, cluster)) * box_k;  // K values per CTA
    const bool encoded =
        b_k_contiguous ? encodeTensorMap2d(&state.map_b, desc.b, desc.k, desc.n, static_cast<std::uint64_t>(desc.b_col_stride) * sizeof(float),
                                           kBtBoxK, kBtStripRows, kSwizzleNone, message, capacity)
                       : encodeTensorMap2d(&state.map_b, desc.b, desc.n, desc.k, static_cast<std::uint64_t>(desc.b_row_stride) * sizeof(float),
                                           kStripColumns, kBoxRows, kSwizzleNone, message, capacity);
    if (!encoded) { return 1; }
    // More than 48 KiB of dynamic shared memory is a per-device opt-in.
    cudaError_t error = cudaSuccess;
    switch (state.row_tile) {
        case 1: error = b_k_contiguous ? allowSharedMemoryBt<1>() : allowSharedMemory<1>(); break;
        case 2: error = b_k_contiguous ? allowSharedMemoryBt<2>() : allowSharedMemory<2>(); break;
        case 4: error = b_k_contiguous ? allowSharedMemoryBt<4>() : allowSharedMemory<4>(); break;
        case 8: error = b_k_contiguous ? allowSharedMemoryBt<8>() : allowSharedMemory<8>(); break;
        case 16: error = b_k_contiguous ? allowSharedMemoryBt<16>() : allowSharedMemory<16>(); break;
        case 24: error = b_k_contiguous ? allowSharedMemoryBt<24>() : allowSharedMemory<24>(); break;
        default: error = b_k_contiguous ? allowSharedMemoryBt<32>() : allowSharedMemory<32>(); break;
    }
    if (error != cudaSuccess) { return fail(message, capacity, 1, "cudaFuncSetAttribute failed: %s", cudaGetErrorString(error)); }
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
    p.rows_per_cta   = state.k_per_split;
    p.rows_per_z     = state.row_tile;
    p.alpha          = desc.alpha;
    p.beta           = desc.beta;
    p.status         = state.device_status;
    cudaError_t error = cudaSuccess;
    switch (state.row_tile) {
        case 1: error = launchRows<1>(state, p, stream); break;
        case 2: error = launchRows<2>(state, p, stream); break;
        case 4: error = launchRows<4>(state, p, stream); break;
        case 8: error = launchRows<8>(state, p, stream); break;
        case 16: error = launchRows<16>(state, p, stream); break;
        case 24: error = launchRows<24>(state, p, stream); break;
        default: error = launchRows<32>(state, p, stream); break;
    }
    countLaunches(1);
    return error;
}

}  // namespace ftcuda
