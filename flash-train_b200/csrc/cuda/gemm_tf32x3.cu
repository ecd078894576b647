// FP32 GEMM on the 5th-generation tensor cores by 3xTF32 split precision:
//   a = a_hi + a_lo, b = b_hi + b_lo with every part a TF32 number, and
//   a*b ~= a_lo*b_hi + a_hi*b_lo + a_hi*b_hi,
// three tcgen05.mma.kind::tf32 products accumulated in FP32 in tensor memory.
// The dropped a_lo*b_lo term is below 2^-22 of |a*b|.
//
// One CTA per SM, persistent over 128 x 192 output tiles, K walked in blocks
// of 32. Twenty warps in five roles, connected only by mbarriers:
//
//   warp 0      TMA producer. Per K block it fetches the raw FP32 operands into
//               one slot of a 3-deep ring: the 128x32 A tile (rows of 128 bytes,
//               128-byte swizzle) and the 32x192 B tile as six 32(k) x 32(n)
//               swizzled boxes (or one 192(n) x 32(k) box when B is contiguous
//               along K). Three K blocks of raw data in flight cover the
//               L2 latency, independently of the stages below.
//   warps 4-7   A converters, one thread per row of A: they read their row from
//               the raw slot (for an A given contiguous along M -- a transposed
//               view -- the raw tile is [k][m] and a thread reads its column),
//               split it and store a_hi / a_lo into TENSOR MEMORY
//               (tcgen05.st), from where the MMA takes its A operand. A never
//               occupies MMA-side shared memory or its read bandwidth. Like the
//               B converters they load everything first and store afterwards.
//   warps 2,3,  B converters, 4 KiB of the B tile per warp. The raw tile already has
//   16-19       the layout the MMA reads: for a row-major B the six boxes (copied
//               with the 32-byte-base variant of the 128-byte swizzle) are the
//               swizzle atoms of an MN-major operand (N contiguous), for a B given
//               contiguous along K (a transposed view, one 32(k) x 192(n) box) it
//               is a K-major operand. Either way the split is element by element:
//               128-bit reads and writes at the same offset into B_hi / B_lo,
//               consecutive lanes at consecutive addresses.
//   warp 1      MMA issuer (one thread walks the whole loop): 4 K-steps x 3
//               products per K block, A from tensor memory, B by shared-memory
//               descriptor (MN-major or K-major, see above), into the
//               "chunk" accumulator (TMEM columns 0-191). A tcgen05.commit per
//               K block releases the stage (its B tiles and its A columns). An
//               MMA issue returns when the pipe has taken the instruction, so
//               whatever else this thread does between two K blocks is time the
//               tensor core idles: its loop carries counters and a table of
//               descriptors, no divisions, no warp votes.
//   warps 8-15  drain / epilogue. Every `chunk_k_blocks` K blocks the chunk
//               accumulator is added, in round-to-nearest FP32, to a running
//               sum kept in TMEM columns 192-383, and the chunk restarts from
//               zero (the interval grows with sqrt(K), see chunkKBlocks). This
//               bounds the length of any accumulation chain inside the tensor
//               core, whose internal FP32 additions truncate. A drain warp
//               reads its 32 lanes x 96 columns of the accumulator in one round
//               trip and hands the accumulator back at once; the running sum is
//               updated after that, while the next chunk is already being
//               multiplied. The 96 values live in registers: setmaxnreg moves
//               registers from the other roles (72 per thread) to the drain
//               warps (128). After the last
//               chunk the sum is scaled and written out -- or stored raw as a
//               split-K partial, or added into the rows' owners' buffers
//               (scatter launches) -- while the next tile's first chunk is
//               already being multiplied.
//
// Shared memory: 3 raw slots x 40 KiB + 2 stages x (B_hi 24 + B_lo 24 KiB) =
// 216 KiB. Tensor memory: chunk 192 + running 192 + 2 stages x (A_hi 32 +
// A_lo 32) columns = 512.
//
// Cluster form (template argument): when the tiles fill under half the SMs and K
// is worth cutting, the grid is tiles x ranks CTAs, the `ranks` (2, 3, 4 or 6) K
// slices of a tile forming a thread-block cluster, one work item per CTA. A CTA
// keeps its slice's sums in the running-sum columns; after a cluster barrier
// the twelve 16-column pieces of the tile are dealt out to the CTAs, every CTA
// stores the pieces of the others into their shared memory (the raw slots, idle
// by then) through distributed shared memory, and after a second cluster
// barrier the owner of a piece adds the slices in rank order, scales and writes
// D. One launch, no workspace, the same bits on every run.
//
// Every wait is bounded (ptx.cuh). A wait that gives up raises the CTA's abort
// flag; all roles then stop, outstanding copies and MMAs are given time to
// land, tensor memory is freed and the device status word is set to nonzero,
// which the host reports at the next launch.
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdlib>
#include <cstring>

#include "gemm_kernels.hpp"
#include <cooperative_groups.h>

#include "ptx.cuh"
#include "tf32x3_common.cuh"

namespace ftcuda {
namespace {

using namespace tf32x3;

constexpr int kTileM  = 128;
constexpr int kStages   = 2;  // converted (hi/lo) stages
constexpr int kRawSlots = 3;  // raw K blocks in flight

constexpr int kRawABytes    = kTileM * kTileK * 4;        // 16 KiB
constexpr int kBoxBytes     = 32 * 32 * 4;                // one 32(k) x 32(n) box of B
constexpr int kBoxes        = kTileN / 32;                // 6
constexpr int kRawSlotBytes = kRawABytes + kBoxes * kBoxBytes;  // 40 KiB
constexpr int kBTileBytes   = kTileN * kTileK * 4;        // 24 KiB, K-major
constexpr int kBHiOffset    = 0;
constexpr int kBLoOffset    = kBTileBytes;
constexpr int kStageBytes   = 2 * kBTileBytes;
constexpr int kStageOffset  = kRawSlots * kRawSlotBytes;
constexpr int kBarrierOffset = kStageOffset + kStages * kStageBytes;
constexpr int kSmemBytes     = kBarrierOffset + 256 + 1024;  // + barriers + alignment slack

constexpr int kThreads         = 640;  // 20 warps
constexpr int kRegsLight       = 72;   // producer, issuer, converters (warpgroups 0, 1, 4)
constexpr int kRegsDrain       = 128;  // drain / epilogue (warpgroups 2, 3)
static_assert(kStages == 2, "the issuer's descriptor table is indexed by s == 0");
static_assert(384 * kRegsLight + 256 * kRegsDrain <= 96 * kThreads, "the CTA's register pool is what it was launched with");
constexpr int kProducerWarp    = 0;
constexpr int kMmaWarp         = 1;
constexpr int kFirstAConverter = 4;   // warps 4..7 convert A (warp % 4 = tensor-memory lane quadrant)
constexpr int kFirstEpilogue   = 8;   // warps 8..15
constexpr int kFirstLateB      = 16;  // warps 2, 3 and 16..19 convert B, one box each
constexpr int kConverterWarps  = 4 + kBoxes;
constexpr int kTmemColumns     = 512;
constexpr int kRunningColumn   = kTileN;       // running sum: columns 192..383
constexpr int kAColumn         = 2 * kTileN;   // A operands: 64 columns per stage from 384
constexpr int kHalfColumns     = kTileN / 2;   // columns per epilogue warp
constexpr int kPieces          = kHalfColumns / 16;


struct Barriers {
    std::uint64_t raw_full[kRawSlots];
    std::uint64_t raw_empty[kRawSlots];
    std::uint64_t mma_done[kStages];
    std::uint64_t conv_done[kStages];
    std::uint64_t acc_full;
    std::uint64_t acc_empty;
    std::uint64_t flush;
    std::uint32_t tmem_base;
    int abort_flag;
};

// kClustered: the cluster form (K slices of a tile as a thread-block cluster) is its own
// instantiation, so that the plain form compiles exactly as it did without it.
// kGrouped: one persistent launch over the tiles of many independent GEMMs (ftcuda_grouped_gemm_*);
// the descriptors and output views of a work item come from its group's table entry.
template<bool kClustered, bool kGrouped = false>
__global__ void __launch_bounds__(kThreads, 1)
tensorGemm3xTf32(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const TensorParams p, const std::uint32_t num_items) {
    extern __shared__ unsigned char smem_raw[];
    const std::uint32_t align_offset = (1024 - (smemAddress(smem_raw) & 1023)) & 1023;
    unsigned char* smem              = smem_raw + align_offset;
    Barriers* bars                   = reinterpret_cast<Barriers*>(smem + kBarrierOffset);
    volatile int* abort_flag         = &bars->abort_flag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int r = 0; r < kRawSlots; ++r) {
            mbarrierInit(&bars->raw_full[r], 1);
            mbarrierInit(&bars->raw_empty[r], kConverterWarps);
        }
        for (int s = 0; s < kStages; ++s) {
            mbarrierInit(&bars->mma_done[s], 1);
            mbarrierInit(&bars->conv_done[s], kConverterWarps);
        }
        mbarrierInit(&bars->acc_full, 1);
        mbarrierInit(&bars->acc_empty, 8);
        mbarrierInit(&bars->flush, 1);
        bars->abort_flag = 0;
        fenceBarrierInit();
        prefetchTensorMap(&map_a);
        prefetchTensorMap(&map_b);
    }
    if (warp == kMmaWarp) { tmemAllocate(&bars->tmem_base, kTmemColumns); }
    // The kernel after this one in the stream (the split-K reduction, launched with programmatic
    // stream serialization) may place its CTAs as SMs come free; it waits for this grid's
    // completion by itself before it reads the partial sums.
    gridDependencyLaunchDependents();
    tcgen05FenceBeforeSync();
    __syncthreads();
    tcgen05FenceAfterSync();
    const std::uint32_t tmem_base = bars->tmem_base;
    // The cluster form is launched with programmatic stream serialization: its CTAs may have done
    // the set-up above while the kernel before it in the stream was still running, and wait here,
    // before the first access to global memory, for that kernel to complete. (Returns at once for
    // an ordinary launch.)
    if constexpr (kClustered) { gridDependencyWait(); }

    // Every role walks the same list of work items and K blocks; `it` counts K
    // blocks over all items and selects the raw slot (it % 3) and the stage
    // (it % 2). The producer and MMA warps keep all 32 lanes in their loops (so
    // that the warp is converged at the block-wide barrier at the end); lane 0
    // alone issues copies, MMAs and commits.
    // The drain warps keep 96 accumulator values at a time in registers; they take the registers the
    // other roles do not need (setmaxnreg acts on warpgroups: 0 and 1 producer / issuer / converters,
    // 2 and 3 drain, 4 converters).
    if (warp >= kFirstEpilogue && warp < kFirstLateB) {
        registersGrow<kRegsDrain>();
        // ------------------------------------------------------------ drain / epilogue
        const int e                   = warp - kFirstEpilogue;  // 0..7
        const std::uint32_t lane_base = static_cast<std::uint32_t>(32 * (e & 3));
        const std::uint32_t col_half  = static_cast<std::uint32_t>(kHalfColumns * (e >> 2));
        const std::uint32_t tmem_row  = tmem_base + (lane_base << 16);
        std::uint32_t chunks          = 0;
        bool ok                       = true;
        for (std::uint32_t item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
            const ItemView view            = fetchItem<kClustered, kGrouped>(p, item, kTileM);
            const WorkItem& w              = view.w;
            // The output of this item: the launch's, or (grouped launches) its group's.
            TensorParams out = p;
            if constexpr (kGrouped) {
                out.c            = view.group->c;
                out.d            = view.group->d;
                out.c_row_stride = view.group->c_row_stride;
                out.c_col_stride = view.group->c_col_stride;
                out.d_row_stride = view.group->d_row_stride;
                out.d_col_stride = view.group->d_col_stride;
                out.m            = view.group->m;
                out.n            = view.group->n;
            }
            const std::uint32_t num_chunks = (w.k_blocks + view.chunk_k_blocks - 1) / view.chunk_k_blocks;
            const std::uint32_t row        = w.tile_m + lane_base + lane;
            const bool partial             = out.partials != nullptr;
            const float* out_base = partial ? out.partials + static_cast<std::uint64_t>(w.split) * out.m * out.n : out.d;
            const bool vector_ok =
                (out.n & 3) == 0 && (reinterpret_cast<std::uintptr_t>(out_base) & 15) == 0 &&
                (partial || (out.d_col_stride == 1 && (out.d_row_stride & 3) == 0)) &&
                (partial || out.c == nullptr ||
                 (out.c_col_stride == 1 && (out.c_row_stride & 3) == 0 && (reinterpret_cast<std::uintptr_t>(out.c) & 15) == 0));
            for (std::uint32_t chunk = 0; chunk < num_chunks && ok; ++chunk, ++chunks) {
                ok = mbarrierWait(&bars->acc_full, chunks & 1, abort_flag);
                if (!ok) { break; }
                tcgen05FenceAfterSync();
                const bool first = chunk == 0;
                const bool last  = chunk + 1 == num_chunks;
                // The chunk accumulator goes to registers in one round trip and is handed back to the
                // MMA issuer at once; the running sum is folded in afterwards, piece by piece (16
                // columns), while the tensor core is already filling the accumulator again: either
                // the result is written out (last chunk) or the new running sum stored.
                float chunk_sum[kHalfColumns];
                tmemLoad96(tmem_row + col_half, chunk_sum);
                tcgen05FenceBeforeSync();
                __syncwarp();
                if (lane == 0) { mbarrierArrive(&bars->acc_empty); }
#pragma unroll
                for (int piece = 0; piece < kPieces; ++piece) {
                    float sum[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) { sum[j] = chunk_sum[piece * 16 + j]; }
                    if (!first) {
                        float running[16];
                        tmemLoad16(tmem_row + kRunningColumn + col_half + piece * 16, running);
#pragma unroll
                        for (int j = 0; j < 16; ++j) { sum[j] += running[j]; }
                    }
                    if (last && !kClustered) {
                        writeRowSegment(out, w, row, w.tile_n + col_half + piece * 16, sum, vector_ok);
                    } else {
                        tmemStore16NoWait(tmem_row + kRunningColumn + col_half + piece * 16, sum);
                    }
                }
                tmemStoreWait();
            }
        }
        if (!ok) { *abort_flag = 1; }
    } else {
        registersShrink<kRegsLight>();
        if (warp == kProducerWarp) {
            // ------------------------------------------------------------ producer
            std::uint32_t it = 0;
            bool ok          = true;
            for (std::uint32_t item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
                const ItemView view   = fetchItem<kClustered, kGrouped>(p, item, kTileM);
                const WorkItem& w     = view.w;
                const void* const at_a = kGrouped ? static_cast<const void*>(&view.group->map_a) : static_cast<const void*>(&map_a);
                const void* const at_b = kGrouped ? static_cast<const void*>(&view.group->map_b) : static_cast<const void*>(&map_b);
                for (std::uint32_t kb = 0; kb < w.k_blocks && ok; ++kb, ++it) {
                    const std::uint32_t r      = it % kRawSlots;
                    const std::uint32_t use    = it / kRawSlots;
                    unsigned char* slot        = smem + r * kRawSlotBytes;
                    const std::int32_t k_coord = static_cast<std::int32_t>(w.k_begin + kb * kTileK);
                    ok = __all_sync(0xFFFFFFFFU, mbarrierWait(&bars->raw_empty[r], (use & 1) ^ 1, abort_flag));
                    if (!ok) { break; }
                    if (lane == 0) {
                        mbarrierArriveExpectTx(&bars->raw_full[r], kRawSlotBytes);
                        if (p.a_m_contiguous != 0) {
                            tmaLoad2d(slot, at_a, &bars->raw_full[r], static_cast<std::int32_t>(w.tile_m), k_coord);
                        } else {
                            tmaLoad2d(slot, at_a, &bars->raw_full[r], k_coord, static_cast<std::int32_t>(w.tile_m));
                        }
                        if (p.b_k_contiguous != 0) {
                            // One box: 192 rows (n) of 32 K values, already in the MMA's K-major layout.
                            tmaLoad2d(slot + kRawABytes, at_b, &bars->raw_full[r], k_coord, static_cast<std::int32_t>(w.tile_n));
                        } else {
                            for (int q = 0; q < kBoxes; ++q) {
                                tmaLoad2d(slot + kRawABytes + q * kBoxBytes, at_b, &bars->raw_full[r],
                                          static_cast<std::int32_t>(w.tile_n + q * 32), k_coord);
                            }
                        }
                    }
                    __syncwarp();
                }
            }
            if (!ok) { *abort_flag = 1; }
        } else if (warp == kMmaWarp) {
            // ------------------------------------------------------------ MMA issuer
            // Row-major B stays N-contiguous in shared memory (MN-major operand); a B
            // given contiguous along K is a K-major operand.
            const std::uint32_t kInstruction =
                umaInstructionTf32(kTileM, kTileN) | (p.b_k_contiguous != 0 ? 0U : kUmaBMnMajor);
            // The issuing thread's own time per K block is what the tensor core waits for, so its loop
            // carries counters instead of divisions and takes its operand descriptors from a table
            // made once (they depend on the stage alone).
            const bool k_major = p.b_k_contiguous != 0;
            // Eight k further: 32 bytes within a K-major row, two 512-byte atoms in an MN-major tile.
            const std::uint64_t k_step = k_major ? 2 : 64;
            std::uint64_t b_hi_of[kStages];
            std::uint64_t b_lo_of[kStages];
#pragma unroll
            for (int stage_index = 0; stage_index < kStages; ++stage_index) {
                const std::uint32_t stage = smemAddress(smem + kStageOffset + stage_index * kStageBytes);
                b_hi_of[stage_index] = k_major ? umaDescriptorK128(stage + kBHiOffset) : umaDescriptorMn128Base32(stage + kBHiOffset, kBoxBytes, 512);
                b_lo_of[stage_index] = k_major ? umaDescriptorK128(stage + kBLoOffset) : umaDescriptorMn128Base32(stage + kBLoOffset, kBoxBytes, 512);
            }
            std::uint32_t s            = 0;  // stage of this K block and the parity of its barrier
            std::uint32_t stage_parity = 0;
            std::uint32_t chunks       = 0;  // chunks started so far, over all items
            bool ok                    = true;
            // One thread walks the loop; the other lanes of the warp wait at the end.
            if (lane == 0) {
                for (std::uint32_t item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
                    const ItemView view = fetchItem<kClustered, kGrouped>(p, item, kTileM);
                    const WorkItem& w   = view.w;
                    std::uint32_t in_chunk = 0;  // K blocks accumulated into the current chunk
                    for (std::uint32_t kb = 0; kb < w.k_blocks && ok; ++kb) {
                        const bool chunk_start = in_chunk == 0;
                        if (chunk_start) {
                            // The drain warps must have emptied the chunk accumulator.
                            ok = mbarrierWait(&bars->acc_empty, (chunks & 1) ^ 1, abort_flag);
                            if (!ok) { break; }
                            ++chunks;
                        }
                        ok = mbarrierWait(&bars->conv_done[s], stage_parity, abort_flag);
                        if (!ok) { break; }
                        tcgen05FenceAfterSync();
                        const bool chunk_end = in_chunk + 1 == view.chunk_k_blocks || kb + 1 == w.k_blocks;
                        const std::uint64_t b_hi = s == 0 ? b_hi_of[0] : b_hi_of[kStages - 1];
                        const std::uint64_t b_lo = s == 0 ? b_lo_of[0] : b_lo_of[kStages - 1];
                        const std::uint32_t a_hi = tmem_base + kAColumn + s * 64;
                        const std::uint32_t a_lo = a_hi + 32;
#pragma unroll
                        for (int step = 0; step < kTileK / 8; ++step) {
                            // 8 TF32 elements further along K: 8 columns of tensor
                            // memory for A, `k_step` descriptor units (of 16 bytes) for B.
                            const std::uint64_t advance = static_cast<std::uint64_t>(step) * k_step;
                            const std::uint32_t fresh   = (chunk_start && step == 0) ? 0U : 1U;
                            umaTf32TmemA(tmem_base, a_lo + step * 8, b_hi + advance, kInstruction, fresh);
                            umaTf32TmemA(tmem_base, a_hi + step * 8, b_lo + advance, kInstruction, 1U);
                            umaTf32TmemA(tmem_base, a_hi + step * 8, b_hi + advance, kInstruction, 1U);
                        }
                        umaCommit(&bars->mma_done[s]);
                        if (chunk_end) { umaCommit(&bars->acc_full); }
                        in_chunk = chunk_end ? 0 : in_chunk + 1;
                        if (++s == kStages) {
                            s = 0;
                            stage_parity ^= 1;
                        }
                    }
                }
            }
            ok = __all_sync(0xFFFFFFFFU, ok);
            if (!ok) {
                *abort_flag = 1;
                // Let MMAs already issued finish before tensor memory is freed.
                if (lane == 0) {
                    umaCommit(&bars->flush);
                    int never = 0;
                    mbarrierWait(&bars->flush, 0, &never);
                }
                __syncwarp();
            }
        } else if (warp < kFirstEpilogue || warp >= kFirstLateB) {
            // ------------------------------------------------------------ converters
            const bool converts_a = warp >= kFirstAConverter && warp < kFirstEpilogue;
            const int box_index   = warp < kFirstAConverter ? warp - 2 : warp - kFirstLateB + 2;  // B box of a B converter
            const int a_row       = 32 * (warp & 3) + lane;   // row of A = TMEM lane (warp % 4 selects the lane quadrant)
            std::uint32_t it = 0;
            bool ok          = true;
            for (std::uint32_t item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
                const WorkItem w = fetchItem<kClustered, kGrouped>(p, item, kTileM).w;
                for (std::uint32_t kb = 0; kb < w.k_blocks && ok; ++kb, ++it) {
                    const std::uint32_t r      = it % kRawSlots;
                    const std::uint32_t s      = it % kStages;
                    const unsigned char* slot  = smem + r * kRawSlotBytes;
                    unsigned char* stage       = smem + kStageOffset + s * kStageBytes;
                    ok = mbarrierWait(&bars->raw_full[r], (it / kRawSlots) & 1, abort_flag);
                    if (!ok) { break; }
                    // The stage (B tiles and A columns) is free once the MMAs of its
                    // previous use have completed.
                    ok = mbarrierWait(&bars->mma_done[s], ((it / kStages) & 1) ^ 1, abort_flag);
                    if (!ok) { break; }
                    tcgen05FenceAfterSync();
                    // Both kinds of converter first bring ALL their raw values into registers and only
                    // then split and store: a store in between (shared memory, or the tensor-memory
                    // store with its memory clobber) would pin every later load behind it, and the
                    // conversion would be eight load-split-store round trips one after the other.
                    if (converts_a) {
                        // One row of A per thread: 8 chunks of 4 floats, un-swizzled by
                        // the row index, split, and stored to this stage's A columns.
                        const unsigned char* row   = slot + a_row * 128;
                        const std::uint32_t a_tmem = tmem_base + (static_cast<std::uint32_t>(32 * (warp & 3)) << 16) +
                                                     kAColumn + s * 64;
                        float values[kTileK];
                        if (p.a_m_contiguous != 0) {
                            // Raw tile is [32 k][128 m], linear: a column per thread,
                            // consecutive lanes read consecutive words.
                            const float* column = reinterpret_cast<const float*>(slot) + a_row;
#pragma unroll
                            for (int j = 0; j < kTileK; ++j) { values[j] = column[j * kTileM]; }
                        } else {
#pragma unroll
                            for (int chunk = 0; chunk < kTileK / 4; ++chunk) {
                                const float4 raw = *reinterpret_cast<const float4*>(row + ((chunk ^ (a_row & 7)) << 4));
                                values[chunk * 4 + 0] = raw.x;
                                values[chunk * 4 + 1] = raw.y;
                                values[chunk * 4 + 2] = raw.z;
                                values[chunk * 4 + 3] = raw.w;
                            }
                        }
#pragma unroll
                        for (int half = 0; half < 2; ++half) {
                            float hi[16];
                            float lo[16];
#pragma unroll
                            for (int j = 0; j < 16; ++j) {
                                std::uint32_t hi_bits, lo_bits;
                                splitTf32(values[half * 16 + j], hi_bits, lo_bits);
                                hi[j] = __uint_as_float(hi_bits);
                                lo[j] = __uint_as_float(lo_bits);
                            }
                            tmemStore16NoWait(a_tmem + half * 16, hi);
                            tmemStore16NoWait(a_tmem + 32 + half * 16, lo);
                        }
                        tmemStoreWait();
                    } else {
                        // B arrives in the layout the MMA reads it in -- six 32 (n) x 32 (k)
                        // boxes of an MN-major operand for a row-major B, 192 rows (n) of a
                        // K-major operand for a B contiguous along K, both with the
                        // 128-byte swizzle -- so it is split element by element, same offset
                        // in the raw tile and in B_hi / B_lo. A warp takes 4 KiB, 128 bits
                        // per lane and step, consecutive lanes at consecutive addresses.
                        const int offset          = box_index * kBoxBytes;
                        const unsigned char* rows = slot + kRawABytes + offset;
                        float4 raw[8];
#pragma unroll
                        for (int c = 0; c < 8; ++c) { raw[c] = *reinterpret_cast<const float4*>(rows + c * 512 + lane * 16); }
#pragma unroll
                        for (int c = 0; c < 8; ++c) {
                            const int at = c * 512 + lane * 16;
                            uint4 hi, lo;
                            splitTf32(raw[c].x, hi.x, lo.x);
                            splitTf32(raw[c].y, hi.y, lo.y);
                            splitTf32(raw[c].z, hi.z, lo.z);
                            splitTf32(raw[c].w, hi.w, lo.w);
                            *reinterpret_cast<uint4*>(stage + kBHiOffset + offset + at) = hi;
                            *reinterpret_cast<uint4*>(stage + kBLoOffset + offset + at) = lo;
                        }
                    }
                    // Publish: shared-memory writes to the async proxy, tensor-memory
                    // stores (already waited for) to the MMA issuer. The same proxy fence
                    // orders this warp's reads of the raw slot before its refill by TMA.
                    fenceProxyAsync();
                    tcgen05FenceBeforeSync();
                    __syncwarp();
                    if (lane == 0) {
                        mbarrierArrive(&bars->raw_empty[r]);
                        mbarrierArrive(&bars->conv_done[s]);
                    }
                }
            }
            if (!ok) { *abort_flag = 1; }
        }
    }

    __syncthreads();
    if (*abort_flag != 0) {
        if (threadIdx.x == 0) {
            if (p.status != nullptr) { *p.status = 2; }
            // Copies that were armed but never consumed may still be landing.
            int never = 0;
            for (int r = 0; r < kRawSlots; ++r) {
                mbarrierWait(&bars->raw_full[r], 0, &never);
                mbarrierWait(&bars->raw_full[r], 1, &never);
            }
        }
        __syncthreads();
    }
    if constexpr (kClustered) {
        // ---- the K slices of this tile meet. Each CTA's sums sit in its running-sum columns. The
        // twelve 16-column pieces of the tile are dealt out to the CTAs (piece q to rank q % ranks);
        // a CTA sends the pieces it does not own to their owners' shared memory -- the raw slots,
        // idle once every CTA of the cluster has left its main loop --, the owner adds the slices in
        // rank order, applies alpha / beta and writes D.
        namespace cg = cooperative_groups;
        cg::cluster_group cluster   = cg::this_cluster();
        const std::uint32_t ranks   = p.cluster_ranks;
        const std::uint32_t rank    = clusterCtaRank();
        const std::uint32_t slots   = (2 * kPieces) / ranks;  // pieces per owner
        // [sender][slot][quad of columns][row]: a warp's 32 rows of one quad are 512 consecutive bytes, so
        // a remote store instruction of a warp is one contiguous segment (row-major 64-byte records cost
        // 32 separate 16-byte transfers per instruction and made the exchange take 4.8 us).
        float4* receive             = reinterpret_cast<float4*>(smem);
        const bool healthy          = *abort_flag == 0;
        const int e                 = warp - kFirstEpilogue;
        const std::uint32_t in_tile = static_cast<std::uint32_t>(32 * (e & 3) + lane);
        const std::uint32_t half    = static_cast<std::uint32_t>(e >> 2);
        const std::uint32_t tmem_at = tmem_base + ((32U * static_cast<std::uint32_t>(e & 3)) << 16) + kRunningColumn + half * kHalfColumns;
        clusterBarrierArrive();
        clusterBarrierWait();
        if (warp >= kFirstEpilogue && warp < kFirstEpilogue + 8 && healthy) {
            tcgen05FenceAfterSync();
#pragma unroll
            for (int piece = 0; piece < kPieces; ++piece) {
                const std::uint32_t q     = half * kPieces + piece;
                const std::uint32_t owner = q % ranks;
                if (owner == rank) { continue; }
                float sum[16];
                tmemLoad16(tmem_at + piece * 16, sum);
                float4* remote = cluster.map_shared_rank(receive, owner) + ((rank * slots + q / ranks) * 4) * kTileM + in_tile;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    remote[j * kTileM] = make_float4(sum[4 * j], sum[4 * j + 1], sum[4 * j + 2], sum[4 * j + 3]);
                }
            }
        }
        clusterBarrierArrive();
        clusterBarrierWait();
        if (warp >= kFirstEpilogue && warp < kFirstEpilogue + 8 && healthy) {
            tcgen05FenceAfterSync();
            const WorkItem w        = decodeItem<kClustered>(p, blockIdx.x, kTileM);
            const std::uint32_t row = w.tile_m + in_tile;
            const bool vector_ok    = (p.n & 3) == 0 && (reinterpret_cast<std::uintptr_t>(p.d) & 15) == 0 && p.d_col_stride == 1 &&
                                   (p.d_row_stride & 3) == 0 &&
                                   (p.c == nullptr || (p.c_col_stride == 1 && (p.c_row_stride & 3) == 0 &&
                                                       (reinterpret_cast<std::uintptr_t>(p.c) & 15) == 0));
#pragma unroll
            for (int piece = 0; piece < kPieces; ++piece) {
                const std::uint32_t q = half * kPieces + piece;
                if (q % ranks != rank) { continue; }
                float own[16];
                float sum[16];
                tmemLoad16(tmem_at + piece * 16, own);
                for (std::uint32_t r = 0; r < ranks; ++r) {
                    const float4* part = receive + ((r * slots + q / ranks) * 4) * kTileM + in_tile;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        float4 v = r == rank ? make_float4(own[4 * j], own[4 * j + 1], own[4 * j + 2], own[4 * j + 3]) : part[j * kTileM];
                        if (r == 0) {
                            sum[4 * j] = v.x, sum[4 * j + 1] = v.y, sum[4 * j + 2] = v.z, sum[4 * j + 3] = v.w;
                        } else {
                            sum[4 * j] += v.x, sum[4 * j + 1] += v.y, sum[4 * j + 2] += v.z, sum[4 * j + 3] += v.w;
                        }
                    }
                }
                writeRowSegment(p, w, row, w.tile_n + half * kHalfColumns + piece * 16, sum, vector_ok);
            }
        }
        __syncthreads();
    }
    if (warp == kMmaWarp) {
        tcgen05FenceAfterSync();
        tmemFree(tmem_base, kTmemColumns);
    }
}

// Clusters of `ranks` CTAs of the cluster form that the current device holds at once (0 on failure).
int residentClusters(std::uint32_t ranks, std::uint32_t clusters_wanted) {
    if (cudaFuncSetAttribute(tensorGemm3xTf32<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess) {
        (void)cudaGetLastError();
        return 0;
    }
    cudaLaunchConfig_t config{};
    config.gridDim          = dim3(clusters_wanted * ranks, 1, 1);
    config.blockDim         = dim3(kThreads, 1, 1);
    config.dynamicSmemBytes = kSmemBytes;
    cudaLaunchAttribute attribute{};
    attribute.id               = cudaLaunchAttributeClusterDimension;
    attribute.val.clusterDim.x = ranks;
    attribute.val.clusterDim.y = 1;
    attribute.val.clusterDim.z = 1;
    config.attrs               = &attribute;
    config.numAttrs            = 1;
    int clusters               = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, tensorGemm3xTf32<true>, &config) != cudaSuccess) {
        (void)cudaGetLastError();
        return 0;
    }
    return clusters;
}

// FTCUDA_TF32_CLUSTER_SPLIT=0 keeps the single-launch family on one CTA per tile (read when a
// launch is configured).
bool clusterSplitEnabled() {
    const char* text = std::getenv("FTCUDA_TF32_CLUSTER_SPLIT");
    return text == nullptr || std::atoi(text) != 0;
}

// Number of K slices that fills the SMs in whole waves: the smallest count
// whose last wave is at least 90 % full, bounded by the slice length.
std::uint32_t chooseSplits(std::uint64_t tiles, std::uint64_t k, int sms) {
    const std::uint64_t most = k / 256 < 2 ? 2 : k / 256;  // slices of >= 256 (8 K blocks)
    std::uint32_t best       = 2;
    double best_fill         = 0.0;
    for (std::uint64_t s = 2; s <= most && s <= 128; ++s) {
        const std::uint64_t items = tiles * s;
        const std::uint64_t waves = ceilDiv(items, static_cast<std::uint64_t>(sms));
        const double fill         = static_cast<double>(items) / static_cast<double>(waves * sms);
        if (fill > best_fill + 1e-9) {
            best_fill = fill;
            best      = static_cast<std::uint32_t>(s);
        }
        if (fill >= 0.90 && waves >= 2) { return static_cast<std::uint32_t>(s); }
    }
    return best;
}

// K blocks accumulated inside the tensor core between two drains. The tensor
// core's FP32 accumulation truncates, so the error of an undrained chain grows
// with its length: measured on B200, the scaled error against float64,
// relative to that of an FP32 FFMA GEMM on the same inputs, is about
// 6 * L / sqrt(K) for a drain every L K blocks (L = 4: 1.08 at K = 512, 0.39 at
// K = 4096; L = 8: 0.82 at K = 4096, 0.18 at K = 65536; never: 12 at K = 4096,
// 47 at K = 65536). A drain stalls the MMAs for about 0.6 us, so L should be as
// long as accuracy allows: L = sqrt(K) / 12.5 aims at half the FFMA GEMM's
// error whatever K is -- 2 at K = 1000, 5 at K = 4096, 16 (the cap) from
// K = 40000 on. FTCUDA_TF32_CHUNK_K_BLOCKS overrides it (a knob for
// accuracy/throughput experiments; read when a launch is configured).
std::uint32_t chunkKBlocks(std::uint64_t k) {
    const char* text = std::getenv("FTCUDA_TF32_CHUNK_K_BLOCKS");
    if (text != nullptr) {
        const long value = std::strtol(text, nullptr, 10);
        if (value >= 1 && value <= (1L << 20)) { return static_cast<std::uint32_t>(value); }
    }
    return drainInterval(k);
}

// Output tiles are walked in bands of this many M tiles (all N tiles of a band
// before the next band): every band re-reads B once from HBM while its A
// panels (band x 128 rows x K) stay in L2. FTCUDA_TF32_BAND_M_TILES overrides (read when a launch is configured).
std::uint32_t bandMTiles() {
    const char* text = std::getenv("FTCUDA_TF32_BAND_M_TILES");
    if (text != nullptr) {
        const long value = std::strtol(text, nullptr, 10);
        if (value >= 1 && value <= 4096) { return static_cast<std::uint32_t>(value); }
    }
    return 16;
}

}  // namespace

const char* supportsTensor(const FtcudaGemmDesc& desc, bool split_k) {
    if (desc.m * desc.n == 0 || desc.k == 0) { return "the problem is empty"; }
    if (desc.m >= (1ULL << 31) || desc.n >= (1ULL << 31) || desc.k >= (1ULL << 31)) {
        return "an extent does not fit 31 bits";
    }
    // Even one K block is twelve truncating accumulations inside the tensor core;
    // against a sum of so few products that error shows (measured: up to 2.3x an
    // FFMA GEMM's at K = 32), so short K is left to the exact kernels.
    if (desc.k < 128) { return "K is too short for the split-precision kernel (under 128)"; }
    if (!tmaEligible(desc.a, desc.a_col_stride, desc.a_row_stride, desc.k, desc.m) &&
        !tmaEligible(desc.a, desc.a_row_stride, desc.a_col_stride, desc.m, desc.k)) {
        return "A is neither row-major nor a transposed row-major view with a 16-byte aligned base and pitch";
    }
    if (!tmaEligible(desc.b, desc.b_col_stride, desc.b_row_stride, desc.n, desc.k) &&
        !tmaEligible(desc.b, desc.b_row_stride, desc.b_col_stride, desc.k, desc.n)) {
        return "B is neither row-major nor a transposed row-major view with a 16-byte aligned base and pitch";
    }
    if (ceilDiv(desc.m, kTileM) * ceilDiv(desc.n, kTileN) >= (1ULL << 24)) { return "too many output tiles"; }
    if (split_k && desc.k < 512) { return "K is too short to split"; }
    return nullptr;
}

int configureTensor(LaunchState& state, bool split_k, char* message, std::size_t capacity) {
    const FtcudaGemmDesc& desc = state.desc;
    int sms                    = 0;
    if (!deviceSmCount(desc.device, &sms, message, capacity)) { return 1; }
    if (!deviceStatusWord(desc.device, &state.device_status, &state.host_status, message, capacity)) { return 1; }
    state.variant = tmaEligible(desc.a, desc.a_col_stride, desc.a_row_stride, desc.k, desc.m) ? kVariantTmaAk : kVariantTmaAm;
    state.band_m_tiles = bandMTiles();  // environment switches are read here, never on the launch path
    const bool b_n_contiguous = tmaEligible(desc.b, desc.b_col_stride, desc.b_row_stride, desc.n, desc.k);
    if (!b_n_contiguous) { state.variant |= kVariantFlagBk; }
    const std::uint64_t tiles  = ceilDiv(desc.m, kTileM) * ceilDiv(desc.n, kTileN);
    state.splits               = 1;
    state.k_per_split          = static_cast<std::uint32_t>(ceilDiv(desc.k, kTileK) * kTileK);
    if (split_k) {
        const std::uint32_t wanted = chooseSplits(tiles, desc.k, sms);
        state.k_per_split = static_cast<std::uint32_t>(ceilDiv(ceilDiv(desc.k, wanted), kTileK) * kTileK);
        state.splits      = static_cast<std::uint32_t>(ceilDiv(desc.k, state.k_per_split));
    }
    // Few tiles and a K worth cutting, in the single-launch family: the K slices of a tile become a
    // thread-block cluster that meets through distributed shared memory -- no workspace, no second
    // kernel. The twelve 16-column pieces of a tile are dealt out to the CTAs, hence 2, 3, 4 or 6.
    if (!split_k && clusterSplitEnabled() && tiles * 2 <= static_cast<std::uint64_t>(sms) && desc.k >= 512) {
        for (const std::uint32_t ranks : {6U, 4U, 3U, 2U}) {
            if (tiles * ranks > static_cast<std::uint64_t>(sms) || desc.k / ranks < 256) { continue; }
            const std::uint32_t per_slice = static_cast<std::uint32_t>(ceilDiv(ceilDiv(desc.k, ranks), kTileK) * kTileK);
            if (ceilDiv(desc.k, per_slice) != ranks) { continue; }  // every CTA of the cluster needs a slice
            // All clusters have to be resident together (a second wave would double the time): a
            // cluster lives inside one GPC, whose SM count need not be a multiple of the cluster size.
            if (static_cast<std::uint64_t>(residentClusters(ranks, static_cast<std::uint32_t>(tiles))) < tiles) { continue; }
            state.variant |= kVariantFlagCluster;
            state.splits      = ranks;
            state.k_per_split = per_slice;
            // Back-to-back launches: letting the next launch's CTAs set up on idle SMs while this one
            // runs saves 1.5 us of 30.7 at 1024^3 (96 CTAs) -- but with most SMs taken (132 CTAs at
            // 256 x 4096 x 4096) the early CTAs fragment the GPCs, the rest of their grid no longer fits
            // at once, and the launch takes 75 instead of 57 us. Hence only up to two thirds of the SMs.
            if (tiles * ranks * 3 <= static_cast<std::uint64_t>(sms) * 2) { state.variant |= kVariantFlagEarlyStart; }
            break;
        }
    }
    const bool clustered      = (state.variant & kVariantFlagCluster) != 0;
    const std::uint64_t items = tiles * state.splits;
    state.grid_x              = static_cast<std::uint32_t>(items < static_cast<std::uint64_t>(sms) ? items : sms);
    state.grid_y              = 1;
    state.grid_z              = 1;
    state.block               = kThreads;
    state.smem_bytes          = kSmemBytes;
    state.chunk_k_blocks      = chunkKBlocks(desc.k);
    state.workspace_bytes =
        state.splits > 1 && !clustered ? static_cast<std::uint64_t>(state.splits) * desc.m * desc.n * sizeof(float) : 0;
    const bool a_encoded =
        (state.variant & kVariantMaskA) == kVariantTmaAk
            ? encodeTensorMap2d(&state.map_a, desc.a, desc.k, desc.m,
                                static_cast<std::uint64_t>(desc.a_row_stride) * sizeof(float), kTileK, kTileM, true,
                                message, capacity)
            : encodeTensorMap2d(&state.map_a, desc.a, desc.m, desc.k,
                                static_cast<std::uint64_t>(desc.a_col_stride) * sizeof(float), kTileM, kTileK, false,
                                message, capacity);
    if (!a_encoded) { return 1; }
    // B row-major: six boxes of 32 (n) x 32 (k) per K block; B contiguous along K: one box of 32 (k) x 192 (n).
    const bool b_encoded =
        b_n_contiguous ? encodeTensorMap2d(&state.map_b, desc.b, desc.n, desc.k,
                                           static_cast<std::uint64_t>(desc.b_row_stride) * sizeof(float), 32, kTileK,
                                           kSwizzle128Atom32, message, capacity)
                       : encodeTensorMap2d(&state.map_b, desc.b, desc.k, desc.n,
                                           static_cast<std::uint64_t>(desc.b_col_stride) * sizeof(float), kTileK, kTileN,
                                           kSwizzle128, message, capacity);
    if (!b_encoded) { return 1; }
    // The plain form always: scatter launches use it even for a launch configured for the cluster form.
    cudaError_t error = cudaFuncSetAttribute(tensorGemm3xTf32<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (error == cudaSuccess && clustered) {
        error = cudaFuncSetAttribute(tensorGemm3xTf32<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    }
    if (error != cudaSuccess) {
        return fail(message, capacity, 1, "cudaFuncSetAttribute failed: %s", cudaGetErrorString(error));
    }
    return 0;
}

namespace {

TensorParams makeTensorParams(const LaunchState& state) {
    const FtcudaGemmDesc& desc = state.desc;
    TensorParams p{};
    p.c              = desc.c;
    p.d              = desc.d;
    p.c_row_stride   = desc.c_row_stride;
    p.c_col_stride   = desc.c_col_stride;
    p.d_row_stride   = desc.d_row_stride;
    p.d_col_stride   = desc.d_col_stride;
    p.m              = static_cast<std::uint32_t>(desc.m);
    p.n              = static_cast<std::uint32_t>(desc.n);
    p.k              = static_cast<std::uint32_t>(desc.k);
    p.tiles_m        = static_cast<std::uint32_t>(ceilDiv(desc.m, kTileM));
    p.tiles_n        = static_cast<std::uint32_t>(ceilDiv(desc.n, kTileN));
    p.splits         = state.splits;
    p.k_per_split    = state.k_per_split;
    p.chunk_k_blocks = state.chunk_k_blocks;
    p.band_m_tiles   = state.band_m_tiles;
    p.a_m_contiguous = (state.variant & kVariantMaskA) == kVariantTmaAm ? 1U : 0U;
    p.b_k_contiguous = (state.variant & kVariantFlagBk) != 0 ? 1U : 0U;
    p.alpha          = desc.alpha;
    p.beta           = desc.beta;
    p.status         = state.device_status;
    return p;
}

}  // namespace

cudaError_t launchTensor(const LaunchState& state, void* workspace, cudaStream_t stream) {
    const FtcudaGemmDesc& desc = state.desc;
    TensorParams p             = makeTensorParams(state);
    const bool clustered       = (state.variant & kVariantFlagCluster) != 0;
    p.partials                 = state.splits > 1 && !clustered ? static_cast<float*>(workspace) : nullptr;
    cudaError_t error          = cudaSuccess;
    if (clustered) {
        p.cluster_ranks = state.splits;
        cudaLaunchConfig_t config{};
        config.gridDim          = dim3(state.grid_x, 1, 1);  // tiles x slices, all resident at once
        config.blockDim         = dim3(state.block, 1, 1);
        config.dynamicSmemBytes = state.smem_bytes;
        config.stream           = stream;
        cudaLaunchAttribute attributes[2] = {};
        attributes[0].id               = cudaLaunchAttributeClusterDimension;
        attributes[0].val.clusterDim.x = state.splits;
        attributes[0].val.clusterDim.y = 1;
        attributes[0].val.clusterDim.z = 1;
        // Short launches (tens of microseconds) in a row, with SMs to spare: the next one's barrier and
        // tensor-memory set-up overlaps this one's tail; the kernel waits for its predecessor by itself.
        attributes[1].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
        attributes[1].val.programmaticStreamSerializationAllowed = 1;
        config.attrs                                             = attributes;
        config.numAttrs                                          = (state.variant & kVariantFlagEarlyStart) != 0 ? 2 : 1;
        error = cudaLaunchKernelEx(&config, tensorGemm3xTf32<true>, state.map_a, state.map_b, p, state.grid_x);
        countLaunches(1);
        return error;
    }
    const std::uint32_t items = p.tiles_m * p.tiles_n * p.splits;
    tensorGemm3xTf32<false><<<state.grid_x, state.block, state.smem_bytes, stream>>>(state.map_a, state.map_b, p, items);
    error = cudaGetLastError();
    std::uint64_t launches = 1;
    if (error == cudaSuccess && state.splits > 1) {
        error = launchSplitKReduce(desc, static_cast<const float*>(workspace), state.splits, stream);
        ++launches;
    }
    countLaunches(launches);
    return error;
}

// Without a workspace: one launch, every work item (output tile x K slice) adds
// alpha * its sums into the owner's rows. With a workspace and several K slices:
// the slices are written as partials, combined locally and added once per element.
cudaError_t launchTensorScatter(const LaunchState& state, void* workspace, float* const* owner_rows, std::uint32_t owners,
                                std::uint32_t rows_per_owner, cudaStream_t stream) {
    TensorParams p = makeTensorParams(state);
    p.c            = nullptr;
    p.beta         = 0.0F;
    // (The cluster form also has several K slices but no workspace: its slices add directly here.)
    const bool two_pass = workspace != nullptr && state.splits > 1 && state.workspace_bytes > 0;
    p.partials          = two_pass ? static_cast<float*>(workspace) : nullptr;
    if (!two_pass) {
        p.scatter_rows = rows_per_owner;
        for (std::uint32_t i = 0; i < owners && i < 8; ++i) { p.scatter[i] = owner_rows[i]; }
    }
    const std::uint32_t items = p.tiles_m * p.tiles_n * p.splits;
    tensorGemm3xTf32<false><<<state.grid_x, state.block, state.smem_bytes, stream>>>(state.map_a, state.map_b, p, items);
    cudaError_t error      = cudaGetLastError();
    std::uint64_t launches = 1;
    if (error == cudaSuccess && two_pass) {
        error = launchSplitKReduceScatter(state.desc, static_cast<const float*>(workspace), state.splits, owner_rows, owners,
                                          rows_per_owner, stream);
        ++launches;
    }
    countLaunches(launches);
    return error;
}

// ---------------------------------------------------------------- grouped launches
//
// One persistent launch over the 128 x 192 tiles of all groups: the work list names the group of
// every tile, the group's table entry carries its TMA descriptors, output views and extents. The
// table is made once, when the launch is configured, and copied into the caller's workspace in
// front of every launch (the workspace is the caller's between launches).

namespace {

constexpr std::uint64_t kTableAlignment = 128;

// Layout class of a group's operands, or a reason why the tensor-core kernel cannot take it.
const char* groupLayout(const FtcudaGemmDesc& desc, bool* a_m_contiguous, bool* b_k_contiguous) {
    const char* reason = supportsTensor(desc, false);
    if (reason != nullptr) { return reason; }
    *a_m_contiguous = !tmaEligible(desc.a, desc.a_col_stride, desc.a_row_stride, desc.k, desc.m);
    *b_k_contiguous = !tmaEligible(desc.b, desc.b_col_stride, desc.b_row_stride, desc.n, desc.k);
    return nullptr;
}

}  // namespace

const char* supportsTensorGrouped(const FtcudaGemmDesc* groups, std::uint32_t count) {
    bool any = false, first_a = false, first_b = false;
    std::uint64_t tiles = 0;
    for (std::uint32_t g = 0; g < count; ++g) {
        const FtcudaGemmDesc& desc = groups[g];
        if (desc.m * desc.n == 0) { continue; }  // an empty group has no tiles
        bool a_m = false, b_k = false;
        const char* reason = groupLayout(desc, &a_m, &b_k);
        if (reason != nullptr) { return reason; }
        if (any && (a_m != first_a || b_k != first_b)) { return "the groups do not share one operand layout (row-major or transposed view)"; }
        if (!any) { first_a = a_m, first_b = b_k, any = true; }
        tiles += ceilDiv(desc.m, kTileM) * ceilDiv(desc.n, kTileN);
        if (tiles >= (1ULL << 24)) { return "too many output tiles"; }
    }
    if (!any) { return "every group is empty"; }
    return nullptr;
}

int configureTensorGrouped(GroupedLaunchState& state, const FtcudaGemmDesc* groups, std::uint32_t count, char* message,
                           std::size_t capacity) {
    int sms = 0;
    if (!deviceSmCount(state.device, &sms, message, capacity)) { return 1; }
    if (!deviceStatusWord(state.device, &state.device_status, &state.host_status, message, capacity)) { return 1; }
    std::vector<GroupEntry> entries;
    std::vector<std::uint32_t> item_group;
    const std::uint32_t band = bandMTiles();
    for (std::uint32_t g = 0; g < count; ++g) {
        const FtcudaGemmDesc& desc = groups[g];
        if (desc.m * desc.n == 0) { continue; }
        bool a_m = false, b_k = false;
        if (const char* reason = groupLayout(desc, &a_m, &b_k)) { return fail(message, capacity, 1, "group %u: %s", g, reason); }
        state.a_m_contiguous = a_m ? 1U : 0U;
        state.b_k_contiguous = b_k ? 1U : 0U;
        GroupEntry entry{};
        const bool a_encoded =
            !a_m ? encodeTensorMap2d(&entry.map_a, desc.a, desc.k, desc.m, static_cast<std::uint64_t>(desc.a_row_stride) * sizeof(float),
                                     kTileK, kTileM, true, message, capacity)
                 : encodeTensorMap2d(&entry.map_a, desc.a, desc.m, desc.k, static_cast<std::uint64_t>(desc.a_col_stride) * sizeof(float),
                                     kTileM, kTileK, false, message, capacity);
        if (!a_encoded) { return 1; }
        const bool b_encoded =
            !b_k ? encodeTensorMap2d(&entry.map_b, desc.b, desc.n, desc.k, static_cast<std::uint64_t>(desc.b_row_stride) * sizeof(float), 32,
                                     kTileK, kSwizzle128Atom32, message, capacity)
                 : encodeTensorMap2d(&entry.map_b, desc.b, desc.k, desc.n, static_cast<std::uint64_t>(desc.b_col_stride) * sizeof(float),
                                     kTileK, kTileN, kSwizzle128, message, capacity);
        if (!b_encoded) { return 1; }
        entry.c              = desc.c;
        entry.d              = desc.d;
        entry.c_row_stride   = desc.c_row_stride;
        entry.c_col_stride   = desc.c_col_stride;
        entry.d_row_stride   = desc.d_row_stride;
        entry.d_col_stride   = desc.d_col_stride;
        entry.m              = static_cast<std::uint32_t>(desc.m);
        entry.n              = static_cast<std::uint32_t>(desc.n);
        entry.k              = static_cast<std::uint32_t>(desc.k);
        entry.chunk_k_blocks = chunkKBlocks(desc.k);
        entry.first_item     = static_cast<std::uint32_t>(item_group.size());
        entry.tiles_m        = static_cast<std::uint32_t>(ceilDiv(desc.m, kTileM));
        entry.tiles_n        = static_cast<std::uint32_t>(ceilDiv(desc.n, kTileN));
        entry.band_m_tiles   = band;
        item_group.insert(item_group.end(), static_cast<std::size_t>(entry.tiles_m) * entry.tiles_n,
                          static_cast<std::uint32_t>(entries.size()));
        entries.push_back(entry);
        state.alpha = desc.alpha;
        state.beta  = desc.beta;
    }
    state.entries = static_cast<std::uint32_t>(entries.size());
    state.items   = static_cast<std::uint32_t>(item_group.size());
    state.grid    = state.items < static_cast<std::uint32_t>(sms) ? state.items : static_cast<std::uint32_t>(sms);
    const std::size_t entry_bytes = entries.size() * sizeof(GroupEntry);
    state.table.assign(entry_bytes + item_group.size() * sizeof(std::uint32_t), 0);
    if (!state.table.empty()) {  // (vectors of size zero have no data pointer worth passing to memcpy)
        std::memcpy(state.table.data(), entries.data(), entry_bytes);
        std::memcpy(state.table.data() + entry_bytes, item_group.data(), item_group.size() * sizeof(std::uint32_t));
    }
    // Room to place the table at a 128-byte boundary whatever the workspace's own alignment is.
    state.workspace_bytes = state.table.size() + kTableAlignment;
    const cudaError_t error =
        cudaFuncSetAttribute(tensorGemm3xTf32<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (error != cudaSuccess) { return fail(message, capacity, 1, "cudaFuncSetAttribute failed: %s", cudaGetErrorString(error)); }
    return 0;
}

cudaError_t launchTensorGrouped(const GroupedLaunchState& state, void* workspace, cudaStream_t stream) {
    if (state.items == 0) { return cudaSuccess; }
    const std::uintptr_t aligned = (reinterpret_cast<std::uintptr_t>(workspace) + kTableAlignment - 1) & ~(kTableAlignment - 1);
    unsigned char* table         = reinterpret_cast<unsigned char*>(aligned);
    cudaError_t error = cudaMemcpyAsync(table, state.table.data(), state.table.size(), cudaMemcpyHostToDevice, stream);
    if (error != cudaSuccess) { return error; }
    TensorParams p{};
    p.splits         = 1;
    p.a_m_contiguous = state.a_m_contiguous;
    p.b_k_contiguous = state.b_k_contiguous;
    p.alpha          = state.alpha;
    p.beta           = state.beta;
    p.status         = state.device_status;
    p.groups         = reinterpret_cast<const GroupEntry*>(table);
    p.item_group     = reinterpret_cast<const std::uint32_t*>(table + static_cast<std::size_t>(state.entries) * sizeof(GroupEntry));
    // The descriptor arguments of the ordinary form are unused here: every item takes its group's.
    const CUtensorMap unused{};
    tensorGemm3xTf32<false, true><<<state.grid, kThreads, kSmemBytes, stream>>>(unused, unused, p, state.items);
    error = cudaGetLastError();
    countLaunches(1);
    return error;
}

}  // namespace ftcuda
