// 3xTF32 FP32 GEMM for few rows of A (m <= 64) on the tensor cores, with the
// operands' roles swapped: D^T = B^T * A^T.
//
// With few rows the cost of the GEMM is reading B once. The exact few-rows
// kernel (gemm_skinny.cu) does that at HBM rate up to about 16 rows, after
// which its FP32 pipe limits it; the large-tile tensor kernel (gemm_tf32x3.cu)
// would spend a whole 128-row tile of MMA and conversion work on them. Here B
// is the operand that fills the tensor core's 128-row dimension: a CTA owns a
// strip of 128 COLUMNS of B (and D), the MMA's M operand is that strip's
// 32(k) x 128(n) tile -- an MN-major operand when B is row-major (no transpose,
// see gemm_tf32x3.cu), a K-major one when B is handed over contiguous along K
// (x @ W^T) --, its N operand the m_pad x 32 tile of A (K-major), and the
// accumulator D^T has 128 lanes = columns of D and a few tensor-memory columns
// per row of D. Per K block the tensor core has a sixth or less of the large
// kernel's work; what remains is streaming and splitting B, 16 KiB per K block.
//
// Split precision as in gemm_tf32x3.cu: both operands are split into TF32 hi and
// lo parts by converter warps (element by element, same offsets: the raw tiles
// already have the layouts the MMA reads). A_hi and A_lo lie one after the
// other in a converted stage, so a K step takes TWO MMAs, not three:
// B_hi x [A_hi ; A_lo] (N = 2 m_pad) and B_lo x A_hi, into three disjoint column
// blocks of the chunk accumulator. Accumulation chains are bounded by draining
// the accumulator every few K blocks into a running sum in the drain warps'
// REGISTERS (a thread owns one column of D for all rows); there are two chunk
// accumulators, so the MMAs never wait for a drain.
//
// The kernel is bound by latencies, not by HBM or the tensor pipe: per K block
// the single MMA-issuing thread spends about 70 cycles per MMA plus its barrier
// waits. Hence two MMAs per K step, counters instead of divisions in the
// issuer's loop, a scheduler nearly to itself for the issuer's warp, and
// converters that have all their loads in flight at once.
//
// K is split over the CTAs of a thread-block cluster (up to 8, blockIdx.y), as in
// gemm_skinny.cu: every CTA owns a share of the strip's columns, receives the
// other CTAs' sums for them through distributed shared memory, adds them in
// rank order, applies alpha / beta and writes D. No workspace, no atomics,
// deterministic.
//
// 16 warps: 0 TMA producer, 1 MMA issuer (and tensor-memory owner); 2, 3, 4, 6,
// 7, 8, 10, 11 converters (an eighth of the B tile and of the A tile each);
// 12-15 drain / epilogue (warp % 4 = tensor-memory lane quadrant); 5 and 9 idle.
// All waits are bounded (ptx.cuh).
#include <cooperative_groups.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "gemm_kernels.hpp"
#include "ptx.cuh"
#include "tf32x3_common.cuh"

namespace ftcuda {
namespace {

namespace cg = cooperative_groups;
using tf32x3::splitTf32;

constexpr int kStripColumns = 128;  // columns of B and D per CTA = M of the MMA
constexpr int kBlockK       = 32;
constexpr int kMaxRows      = 64;   // rows of A (N of the MMA) at most
constexpr int kMaxStages    = 3;
constexpr int kChunkBuffers = 2;
constexpr int kMaxCluster   = 8;

constexpr int kBoxBytes  = 32 * 32 * 4;         // one 32(k) x 32(n) box of B
constexpr int kBoxes     = kStripColumns / 32;  // 4
constexpr int kRawBBytes = kBoxes * kBoxBytes;  // 16 KiB
// Shared memory per padded row count: raw slots (B tile + A tile) | stages (B_hi, B_lo, A_hi, A_lo) |
// received sums [sender][row][column share] | barriers. Four raw slots cover the TMA latency (about
// 2 us under load, four K-block periods); the converted stages take what is left of the 227 KiB:
// three, or two for the 64-row form, whose stages are 48 KiB. The 16-row form has room for six raw
// slots, worth 3 % (two slots instead of four cost 25 %).
__host__ __device__ constexpr int aBytes(int rows) { return rows * kBlockK * 4; }
__host__ __device__ constexpr int rawSlots(int rows) { return rows <= 16 ? 6 : 4; }
__host__ __device__ constexpr int stages(int rows) { return rows <= 32 ? 3 : 2; }
__host__ __device__ constexpr int rawSlotBytes(int rows) { return kRawBBytes + aBytes(rows); }
__host__ __device__ constexpr int stageBytes(int rows) { return 2 * kRawBBytes + 2 * aBytes(rows); }
__host__ __device__ constexpr int stageOffset(int rows) { return rawSlots(rows) * rawSlotBytes(rows); }
__host__ __device__ constexpr int receiveOffset(int rows) { return stageOffset(rows) + stages(rows) * stageBytes(rows); }
__host__ __device__ constexpr int receiveBytes(int rows) { return rows * kStripColumns * 4; }
__host__ __device__ constexpr int barrierOffset(int rows) { return receiveOffset(rows) + receiveBytes(rows); }
__host__ __device__ constexpr int smemBytes(int rows) { return barrierOffset(rows) + 256 + 1024; }
static_assert(smemBytes(16) <= 232448 && smemBytes(32) <= 232448 && smemBytes(64) <= 232448, "shared memory budget");
constexpr int kMaxRawSlots = 6;

constexpr int kThreads        = 512;
constexpr int kProducerWarp   = 0;
constexpr int kMmaWarp        = 1;
// The MMA issuer is one thread whose instruction latencies add up to the K-block period, so it gets
// its scheduler (warps 1, 5, 9, 13) nearly to itself: warps 5 and 9 only take part in the block-wide
// steps, and the drain warps sleep between polls.
constexpr int kConverterWarps = 8;   // warps 2, 3, 4, 6, 7, 8, 10, 11
constexpr int kFirstEpilogue  = 12;  // warps 12..15
__device__ __forceinline__ bool isConverter(int warp) { return warp >= 2 && warp < kFirstEpilogue && (warp & 3) != 1; }
__device__ __forceinline__ int converterIndex(int warp) { return warp - 2 - (warp > 5 ? 1 : 0) - (warp > 9 ? 1 : 0); }

// mbarrierWait for warps that are not on the critical path: sleeps between polls instead of
// competing with the MMA issuer for issue slots.
__device__ __forceinline__ bool mbarrierWaitRelaxed(std::uint64_t* barrier, std::uint32_t parity, const volatile int* abort_flag) {
    if (mbarrierTryWait(barrier, parity)) { return true; }
    const unsigned long long start = globalTimerNs();
    std::uint32_t spins            = 0;
    while (true) {
        __nanosleep(64);
        if (mbarrierTryWait(barrier, parity)) { return true; }
        if ((++spins & 0x3F) == 0) {
            if (*abort_flag != 0) { return false; }
            if (globalTimerNs() - start > kWaitBudgetNs) { return false; }
        }
    }
}
// A chunk accumulator: B_hi A_hi | B_hi A_lo | B_lo A_hi, each kRowsPad columns. The two MMAs of a
// K step write disjoint columns, so every accumulation chain is a plain same-shape chain.
constexpr int kChunkColumns   = 256;
constexpr int kTmemColumns    = 512;  // two chunk accumulators

constexpr std::uint32_t kUmaAMnMajor = 1u << 15;  // instruction-descriptor bit: the A operand is MN-major

struct RowsParams {
    const float* c;
    float* d;
    std::int64_t c_row_stride, c_col_stride;
    std::int64_t d_row_stride, d_col_stride;
    std::uint32_t m, n, k;
    std::uint32_t k_blocks_per_cta;
    std::uint32_t chunk_k_blocks;
    std::uint32_t b_k_contiguous;  // B given contiguous along K: its strip tile is a K-major operand [128 n][32 k]
    float alpha, beta;
    int* status;
};

struct Barriers {
    std::uint64_t raw_full[kMaxRawSlots];
    std::uint64_t raw_empty[kMaxRawSlots];
    std::uint64_t mma_done[kMaxStages];
    std::uint64_t conv_done[kMaxStages];
    std::uint64_t acc_full[kChunkBuffers];
    std::uint64_t acc_empty[kChunkBuffers];
    std::uint64_t flush;
    std::uint32_t tmem_base;
    int abort_flag;
};

__device__ __forceinline__ void clusterArrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void clusterWait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

// A converter warp's share of a raw tile, kBytes from `raw`, already split into TF32 hi and lo parts:
// lane L holds bytes [512 i + 16 L, +16) of pass i. All loads are issued before the first value is
// used: a converter's time per K block is latency, not arithmetic.
template<int kBytes>
struct SplitShare {
    static constexpr int kPasses = (kBytes + 511) / 512;
    uint4 hi[kPasses];
    uint4 lo[kPasses];

    __device__ __forceinline__ static bool holds(int pass, int lane) { return kBytes % 512 == 0 || pass * 512 + lane * 16 < kBytes; }

    __device__ __forceinline__ void load(const unsigned char* raw, int lane) {
        float4 value[kPasses];
#pragma unroll
        for (int i = 0; i < kPasses; ++i) {
            if (holds(i, lane)) { value[i] = *reinterpret_cast<const float4*>(raw + i * 512 + lane * 16); }
        }
#pragma unroll
        for (int i = 0; i < kPasses; ++i) {
            if (holds(i, lane)) {
                splitTf32(value[i].x, hi[i].x, lo[i].x);
                splitTf32(value[i].y, hi[i].y, lo[i].y);
                splitTf32(value[i].z, hi[i].z, lo[i].z);
                splitTf32(value[i].w, hi[i].w, lo[i].w);
            }
        }
    }

    // The parts to the same offsets of the two converted tiles.
    __device__ __forceinline__ void store(unsigned char* hi_out, unsigned char* lo_out, int lane) const {
#pragma unroll
        for (int i = 0; i < kPasses; ++i) {
            if (holds(i, lane)) {
                *reinterpret_cast<uint4*>(hi_out + i * 512 + lane * 16) = hi[i];
                *reinterpret_cast<uint4*>(lo_out + i * 512 + lane * 16) = lo[i];
            }
        }
    }
};

// kRowsPad: rows of A rounded up to 16, 32 or 64 = N of the MMA = columns of the accumulator.
template<int kRowsPad>
__global__ void __launch_bounds__(kThreads, 1)
tensorGemm3xTf32Rows(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const RowsParams p) {
    constexpr int kRawSlots     = rawSlots(kRowsPad);
    constexpr int kStages       = stages(kRowsPad);
    constexpr int kRawSlotBytes = rawSlotBytes(kRowsPad);
    constexpr int kRawABytes    = aBytes(kRowsPad);
    constexpr int kStageBytes   = stageBytes(kRowsPad);
    constexpr int kStageOffset  = stageOffset(kRowsPad);
    extern __shared__ unsigned char smem_raw[];
    const std::uint32_t align_offset = (1024 - (smemAddress(smem_raw) & 1023)) & 1023;
    unsigned char* smem              = smem_raw + align_offset;
    float* received                  = reinterpret_cast<float*>(smem + receiveOffset(kRowsPad));
    Barriers* bars                   = reinterpret_cast<Barriers*>(smem + barrierOffset(kRowsPad));
    volatile int* abort_flag         = &bars->abort_flag;

    cg::cluster_group cluster = cg::this_cluster();
    const unsigned rank       = cluster.block_rank();
    const unsigned ranks      = cluster.num_blocks();  // 1, 2, 4 or 8

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const std::uint32_t strip_col = blockIdx.x * kStripColumns;

    const std::uint32_t total_k_blocks = (p.k + kBlockK - 1) / kBlockK;
    const std::uint32_t first_block    = min(rank * p.k_blocks_per_cta, total_k_blocks);
    const std::uint32_t k_blocks       = min(p.k_blocks_per_cta, total_k_blocks - first_block);
    const std::uint32_t num_chunks     = (k_blocks + p.chunk_k_blocks - 1) / p.chunk_k_blocks;

    if (threadIdx.x == 0) {
        for (int r = 0; r < kRawSlots; ++r) {
            mbarrierInit(&bars->raw_full[r], 1);
            mbarrierInit(&bars->raw_empty[r], kConverterWarps);
        }
        for (int s = 0; s < kStages; ++s) {
            mbarrierInit(&bars->mma_done[s], 1);
            mbarrierInit(&bars->conv_done[s], kConverterWarps);
        }
        for (int c = 0; c < kChunkBuffers; ++c) {
            mbarrierInit(&bars->acc_full[c], 1);
            mbarrierInit(&bars->acc_empty[c], 4);
        }
        mbarrierInit(&bars->flush, 1);
        bars->abort_flag = 0;
        fenceBarrierInit();
        prefetchTensorMap(&map_a);
        prefetchTensorMap(&map_b);
    }
    if (warp == kMmaWarp) { tmemAllocate(&bars->tmem_base, kTmemColumns); }
    // Everything above overlaps the tail of the kernel before this one in the stream; nothing below
    // touches global memory before that kernel has completed.
    gridDependencyWait();
    gridDependencyLaunchDependents();
    tcgen05FenceBeforeSync();
    __syncthreads();
    tcgen05FenceAfterSync();
    const std::uint32_t tmem_base = bars->tmem_base;
    // First half of a cluster barrier ("every CTA of the cluster runs"); its second
    // half sits in front of the first remote store.
    clusterArrive();

    // This thread's column of D for all rows, summed over the chunks (drain warps only).
    float running[kRowsPad];
#pragma unroll
    for (int i = 0; i < kRowsPad; ++i) { running[i] = 0.0F; }

    if (warp == kProducerWarp) {
        // ------------------------------------------------------------ producer
        bool ok = true;
        for (std::uint32_t kb = 0; kb < k_blocks && ok; ++kb) {
            const std::uint32_t r      = kb % kRawSlots;
            unsigned char* slot        = smem + r * kRawSlotBytes;
            const std::int32_t k_coord = static_cast<std::int32_t>((first_block + kb) * kBlockK);
            ok = __all_sync(0xFFFFFFFFU, mbarrierWait(&bars->raw_empty[r], ((kb / kRawSlots) & 1) ^ 1, abort_flag));
            if (!ok) { break; }
            if (lane == 0) {
                mbarrierArriveExpectTx(&bars->raw_full[r], kRawSlotBytes);
                if (p.b_k_contiguous != 0) {
                    tmaLoad2d(slot, &map_b, &bars->raw_full[r], k_coord, static_cast<std::int32_t>(strip_col));
                } else {
                    for (int q = 0; q < kBoxes; ++q) {
                        tmaLoad2d(slot + q * kBoxBytes, &map_b, &bars->raw_full[r], static_cast<std::int32_t>(strip_col + q * 32), k_coord);
                    }
                }
                tmaLoad2d(slot + kRawBBytes, &map_a, &bars->raw_full[r], k_coord, 0);
            }
            __syncwarp();
        }
        if (!ok) { *abort_flag = 1; }
    } else if (warp == kMmaWarp) {
        // ------------------------------------------------------------ MMA issuer
        // M operand: the strip of B, MN-major (N of B contiguous); N operand: A, K-major.
        const bool b_k_major            = p.b_k_contiguous != 0;
        const std::uint32_t layout_flag = b_k_major ? 0U : kUmaAMnMajor;
        // A_hi and A_lo lie one after the other in a stage, so one MMA with N = 2 * kRowsPad multiplies B_hi with both.
        const std::uint32_t instruction_both = umaInstructionTf32(kStripColumns, 2 * kRowsPad) | layout_flag;
        const std::uint32_t instruction_one  = umaInstructionTf32(kStripColumns, kRowsPad) | layout_flag;
        std::uint32_t chunks                 = 0;
        std::uint32_t in_chunk               = 0;  // K blocks accumulated into the current chunk
        std::uint32_t s                      = 0;  // stage of this K block and the parity of its barriers
        std::uint32_t stage_parity           = 0;
        bool ok                              = true;
        for (std::uint32_t kb = 0; kb < k_blocks && ok; ++kb) {
            const bool chunk_start = in_chunk == 0;
            if (chunk_start) {
                ok = __all_sync(0xFFFFFFFFU, mbarrierWait(&bars->acc_empty[chunks % kChunkBuffers],
                                                          ((chunks / kChunkBuffers) & 1) ^ 1, abort_flag));
                if (!ok) { break; }
                ++chunks;
            }
            const std::uint32_t buffer = (chunks - 1) % kChunkBuffers;
            ok = __all_sync(0xFFFFFFFFU, mbarrierWait(&bars->conv_done[s], stage_parity, abort_flag));
            if (!ok) { break; }
            tcgen05FenceAfterSync();
            if (lane == 0) {
                const std::uint32_t stage = smemAddress(smem + kStageOffset + s * kStageBytes);
                const std::uint64_t b_hi  = b_k_major ? umaDescriptorK128(stage) : umaDescriptorMn128Base32(stage, kBoxBytes, 512);
                const std::uint64_t b_lo  = b_k_major ? umaDescriptorK128(stage + kRawBBytes)
                                                      : umaDescriptorMn128Base32(stage + kRawBBytes, kBoxBytes, 512);
                const std::uint64_t a_hi  = umaDescriptorK128(stage + 2 * kRawBBytes);
                const std::uint64_t a_lo  = umaDescriptorK128(stage + 2 * kRawBBytes + kRawABytes);
                const std::uint32_t d_tmem = tmem_base + buffer * kChunkColumns;
#pragma unroll
                for (int step = 0; step < kBlockK / 8; ++step) {
                    // 8 k further: two 512-byte atoms of the MN-major tile, 32 bytes of a K-major row.
                    const std::uint64_t mn_step = static_cast<std::uint64_t>(step) * (b_k_major ? 2 : 64);
                    const std::uint64_t k_step  = static_cast<std::uint64_t>(step) * 2;
                    const std::uint32_t fresh   = (chunk_start && step == 0) ? 0U : 1U;
                    umaTf32(d_tmem, b_hi + mn_step, a_hi + k_step, instruction_both, fresh);
                    umaTf32(d_tmem + 2 * kRowsPad, b_lo + mn_step, a_hi + k_step, instruction_one, fresh);
                }
                umaCommit(&bars->mma_done[s]);
                if (in_chunk + 1 == p.chunk_k_blocks || kb + 1 == k_blocks) { umaCommit(&bars->acc_full[buffer]); }
            }
            in_chunk = (in_chunk + 1 == p.chunk_k_blocks) ? 0 : in_chunk + 1;
            if (++s == kStages) {
                s = 0;
                stage_parity ^= 1;
            }
            __syncwarp();
        }
        if (!ok) {
            *abort_flag = 1;
            if (lane == 0) {
                umaCommit(&bars->flush);
                int never = 0;
                mbarrierWait(&bars->flush, 0, &never);
            }
            __syncwarp();
        }
    } else if (isConverter(warp)) {
        // ------------------------------------------------------------ converters
        // Every converter warp takes an eighth of the B tile and an eighth of the A tile.
        constexpr int kBShare = kRawBBytes / kConverterWarps;
        constexpr int kAShare = kRawABytes / kConverterWarps;
        const int b_at        = converterIndex(warp) * kBShare;
        const int a_at        = converterIndex(warp) * kAShare;
        bool ok               = true;
        std::uint32_t s            = 0;
        std::uint32_t stage_parity = 0;
        for (std::uint32_t kb = 0; kb < k_blocks && ok; ++kb) {
            const std::uint32_t r     = kb % kRawSlots;
            const unsigned char* slot = smem + r * kRawSlotBytes;
            unsigned char* stage      = smem + kStageOffset + s * kStageBytes;
            ok = mbarrierWait(&bars->raw_full[r], (kb / kRawSlots) & 1, abort_flag);
            if (!ok) { break; }
            // Load and split in registers while the converted stage may still be busy. The raw slot is
            // handed back only below, behind the proxy fence: released right after the loads (even
            // behind a block-level fence) a refill by TMA was seen to overtake them now and then.
            SplitShare<kBShare> b_parts;
            SplitShare<kAShare> a_parts;
            b_parts.load(slot + b_at, lane);
            a_parts.load(slot + kRawBBytes + a_at, lane);
            ok = mbarrierWait(&bars->mma_done[s], stage_parity ^ 1, abort_flag);
            if (!ok) { break; }
            b_parts.store(stage + b_at, stage + kRawBBytes + b_at, lane);
            a_parts.store(stage + 2 * kRawBBytes + a_at, stage + 2 * kRawBBytes + kRawABytes + a_at, lane);
            fenceProxyAsync();
            __syncwarp();
            if (lane == 0) {
                mbarrierArrive(&bars->raw_empty[r]);
                mbarrierArrive(&bars->conv_done[s]);
            }
            if (++s == kStages) {
                s = 0;
                stage_parity ^= 1;
            }
        }
        if (!ok) { *abort_flag = 1; }
    } else if (warp >= kFirstEpilogue) {
        // ------------------------------------------------------------ drain
        const std::uint32_t lane_base = static_cast<std::uint32_t>(32 * (warp & 3));
        const std::uint32_t tmem_row  = tmem_base + (lane_base << 16);
        bool ok                       = true;
        for (std::uint32_t chunk = 0; chunk < num_chunks && ok; ++chunk) {
            const std::uint32_t buffer = chunk % kChunkBuffers;
            ok = mbarrierWaitRelaxed(&bars->acc_full[buffer], (chunk / kChunkBuffers) & 1, abort_flag);
            if (!ok) { break; }
            tcgen05FenceAfterSync();
#pragma unroll
            for (int piece = 0; piece < kRowsPad / 16; ++piece) {
                float sum[16];
                float hi_lo[16];
                float lo_hi[16];
                tmemLoad16(tmem_row + buffer * kChunkColumns + piece * 16, sum);
                tmemLoad16(tmem_row + buffer * kChunkColumns + kRowsPad + piece * 16, hi_lo);
                tmemLoad16(tmem_row + buffer * kChunkColumns + 2 * kRowsPad + piece * 16, lo_hi);
#pragma unroll
                for (int j = 0; j < 16; ++j) { running[piece * 16 + j] += sum[j] + (hi_lo[j] + lo_hi[j]); }
            }
            tcgen05FenceBeforeSync();
            __syncwarp();
            if (lane == 0) { mbarrierArrive(&bars->acc_empty[buffer]); }
        }
        if (!ok) { *abort_flag = 1; }
    }

    __syncthreads();
    const bool failed = *abort_flag != 0;
    if (failed && threadIdx.x == 0) {
        if (p.status != nullptr) { *p.status = 5; }
        int never = 0;
        for (int r = 0; r < kRawSlots; ++r) {
            mbarrierWait(&bars->raw_full[r], 0, &never);
            mbarrierWait(&bars->raw_full[r], 1, &never);
        }
    }

    // ---- reduction over the cluster's K slices, in rank order. The strip's 128
    // columns are shared out among the CTAs; a drain thread (one column, all rows)
    // sends its sums to the column's owner.
    clusterWait();
    const unsigned columns_per_rank = kStripColumns / ranks;
    if (warp >= kFirstEpilogue && !failed) {
        const unsigned column = 32 * (warp & 3) + lane;
        const unsigned owner  = column / columns_per_rank;
        float* remote         = cluster.map_shared_rank(received, owner);
#pragma unroll
        for (int i = 0; i < kRowsPad; ++i) {
            remote[(rank * kRowsPad + i) * columns_per_rank + column % columns_per_rank] = running[i];
        }
    }
    clusterArrive();
    clusterWait();
    if (*abort_flag == 0) {
        for (unsigned item = threadIdx.x; item < kRowsPad * columns_per_rank; item += kThreads) {
            const unsigned i            = item / columns_per_rank;
            const unsigned local        = item % columns_per_rank;
            const std::uint32_t out_col = strip_col + rank * columns_per_rank + local;
            if (i >= p.m || out_col >= p.n) { continue; }
            float sum = received[i * columns_per_rank + local];
            for (unsigned r = 1; r < ranks; ++r) { sum += received[(r * kRowsPad + i) * columns_per_rank + local]; }
            float value = p.alpha * sum;
            if (p.c != nullptr) {
                value += p.beta * p.c[static_cast<std::int64_t>(i) * p.c_row_stride + static_cast<std::int64_t>(out_col) * p.c_col_stride];
            }
            p.d[static_cast<std::int64_t>(i) * p.d_row_stride + static_cast<std::int64_t>(out_col) * p.d_col_stride] = value;
        }
    }
    __syncthreads();
    if (warp == kMmaWarp) {
        tcgen05FenceAfterSync();
        tmemFree(tmem_base, kTmemColumns);
    }
}

template<int kRowsPad>
cudaError_t launchRowsPad(const LaunchState& state, const RowsParams& p, cudaStream_t stream) {
    cudaLaunchConfig_t config{};
    config.gridDim          = dim3(state.grid_x, state.grid_y, 1);
    config.blockDim         = dim3(state.block, 1, 1);
    config.dynamicSmemBytes = state.smem_bytes;
    config.stream           = stream;
    cudaLaunchAttribute attributes[2] = {};
    attributes[0].id               = cudaLaunchAttributeClusterDimension;
    attributes[0].val.clusterDim.x = 1;
    attributes[0].val.clusterDim.y = state.grid_y;  // the K slices of a strip form one cluster
    attributes[0].val.clusterDim.z = 1;
    // The kernel waits for its predecessor in the stream by itself (gridDependencyWait), so its
    // CTAs may start while that predecessor drains.
    attributes[1].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs                                             = attributes;
    config.numAttrs                                          = 2;
    return cudaLaunchKernelEx(&config, tensorGemm3xTf32Rows<kRowsPad>, state.map_a, state.map_b, p);
}

std::uint32_t paddedRows(std::uint64_t m) { return m <= 16 ? 16 : m <= 32 ? 32 : 64; }

}  // namespace

const char* supportsTensorRows(const FtcudaGemmDesc& desc) {
    if (desc.m == 0 || desc.m > kMaxRows) { return "more than 64 rows (or none) in A"; }
    if (desc.n == 0) { return "the problem is empty"; }
    if (desc.n >= (1ULL << 31) || desc.k >= (1ULL << 31)) { return "an extent does not fit 31 bits"; }
    if (desc.k < 128) { return "K is too short for the split-precision kernel (under 128)"; }
    if (!tmaEligible(desc.a, desc.a_col_stride, desc.a_row_stride, desc.k, desc.m)) {
        return "A is not row-major with a 16-byte aligned base and row pitch";
    }
    if (!tmaEligible(desc.b, desc.b_col_stride, desc.b_row_stride, desc.n, desc.k) &&
        !tmaEligible(desc.b, desc.b_row_stride, desc.b_col_stride, desc.k, desc.n)) {
        return "B is neither row-major nor a transposed row-major view with a 16-byte aligned base and pitch";
    }
    return nullptr;
}

int configureTensorRows(LaunchState& state, char* message, std::size_t capacity) {
    const FtcudaGemmDesc& desc = state.desc;
    int sms                    = 0;
    if (!deviceSmCount(desc.device, &sms, message, capacity)) { return 1; }
    if (!deviceStatusWord(desc.device, &state.device_status, &state.host_status, message, capacity)) { return 1; }
    const bool b_n_contiguous = tmaEligible(desc.b, desc.b_col_stride, desc.b_row_stride, desc.n, desc.k);
    state.variant         = kVariantTmaAk | (b_n_contiguous ? 0 : kVariantFlagBk);
    state.grid_x          = static_cast<std::uint32_t>(ceilDiv(desc.n, kStripColumns));
    state.block           = kThreads;
    state.row_tile        = paddedRows(desc.m);
    state.smem_bytes      = static_cast<std::uint32_t>(smemBytes(static_cast<int>(state.row_tile)));
    state.splits          = 1;
    state.workspace_bytes = 0;
    state.chunk_k_blocks  = tf32x3::drainInterval(desc.k);
    // CTAs per cluster (= K slices per strip): as many as fit the GPU in one wave
    // (one CTA per SM), each keeping at least eight K blocks.
    const std::uint64_t k_blocks = ceilDiv(desc.k, kBlockK);
    std::uint32_t cluster        = 1;
    while (cluster < kMaxCluster && static_cast<std::uint64_t>(state.grid_x) * cluster * 2 <= static_cast<std::uint64_t>(sms) &&
           k_blocks / (cluster * 2) >= 8) {
        cluster *= 2;
    }
    state.grid_y      = cluster;
    state.grid_z      = 1;
    state.k_per_split = static_cast<std::uint32_t>(ceilDiv(k_blocks, cluster));  // K blocks per CTA
    const bool b_encoded =
        b_n_contiguous ? encodeTensorMap2d(&state.map_b, desc.b, desc.n, desc.k, static_cast<std::uint64_t>(desc.b_row_stride) * sizeof(float),
                                           32, kBlockK, kSwizzle128Atom32, message, capacity)
                       : encodeTensorMap2d(&state.map_b, desc.b, desc.k, desc.n, static_cast<std::uint64_t>(desc.b_col_stride) * sizeof(float),
                                           kBlockK, kStripColumns, kSwizzle128, message, capacity);
    if (!b_encoded) { return 1; }
    if (!encodeTensorMap2d(&state.map_a, desc.a, desc.k, desc.m, static_cast<std::uint64_t>(desc.a_row_stride) * sizeof(float), kBlockK,
                           state.row_tile, kSwizzle128, message, capacity)) {
        return 1;
    }
    cudaError_t error = cudaSuccess;
    switch (state.row_tile) {
        case 16: error = cudaFuncSetAttribute(tensorGemm3xTf32Rows<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, smemBytes(16)); break;
        case 32: error = cudaFuncSetAttribute(tensorGemm3xTf32Rows<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, smemBytes(32)); break;
        default: error = cudaFuncSetAttribute(tensorGemm3xTf32Rows<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smemBytes(64)); break;
    }
    if (error != cudaSuccess) { return fail(message, capacity, 1, "cudaFuncSetAttribute failed: %s", cudaGetErrorString(error)); }
    return 0;
}

cudaError_t launchTensorRows(const LaunchState& state, cudaStream_t stream) {
    const FtcudaGemmDesc& desc = state.desc;
    RowsParams p{};
    p.c                = desc.c;
    p.d                = desc.d;
    p.c_row_stride     = desc.c_row_stride;
    p.c_col_stride     = desc.c_col_stride;
    p.d_row_stride     = desc.d_row_stride;
    p.d_col_stride     = desc.d_col_stride;
    p.m                = static_cast<std::uint32_t>(desc.m);
    p.n                = static_cast<std::uint32_t>(desc.n);
    p.k                = static_cast<std::uint32_t>(desc.k);
    p.k_blocks_per_cta = state.k_per_split;
    p.chunk_k_blocks   = state.chunk_k_blocks;
    p.b_k_contiguous   = (state.variant & kVariantFlagBk) != 0 ? 1U : 0U;
    p.alpha            = desc.alpha;
    p.beta             = desc.beta;
    p.status           = state.device_status;
    cudaError_t error  = cudaSuccess;
    switch (state.row_tile) {
        case 16: error = launchRowsPad<16>(state, p, stream); break;
        case 32: error = launchRowsPad<32>(state, p, stream); break;
        default: error = launchRowsPad<64>(state, p, stream); break;
    }
    countLaunches(1);
    return error;
}

}  // namespace ftcuda
