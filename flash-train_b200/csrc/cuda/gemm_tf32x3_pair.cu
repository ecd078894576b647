// 3xTF32 FP32 GEMM on CTA PAIRS: the tensor cores of two neighbouring SMs work
// on one 256 x 192 output tile (tcgen05 cta_group::2).
//
// Same scheme as the single-CTA kernel (gemm_tf32x3.cu): raw FP32 tiles arrive
// by TMA, converter warps split them into TF32 hi / lo parts (A into tensor
// memory, B into shared memory), three MMAs per K step accumulate in tensor
// memory, a running round-to-nearest sum absorbs the chunk accumulator every few
// K blocks. What the pair changes: each CTA holds its own 128 rows of A and of
// the accumulators, but only HALF of the B tile (96 of the 192 columns); the
// MMA, issued by one thread of the even CTA, reads both halves. Per SM this
// halves the B traffic through shared memory -- TMA writes, converter reads and
// writes, operand fetch -- which is what bounds the single-CTA kernel.
//
// Per CTA, 21 warps:
//   warp 0        TMA producer: its 128 x 32 tile of A and its 32 x 96 half of B
//                 into one of four raw slots (28 KiB each).
//   warp 1        tensor-memory allocation in both CTAs; in the even CTA also the
//                 MMA issuer.
//   warps 4-7     A converters for K values 0-15 of the K block, warps 16-19 for
//                 16-31 (warp % 4 = tensor-memory lane quadrant, a thread per row).
//   warps 2,3,20  B converters, one 32-column box (4 KiB) each.
//   warps 8-15    drain / epilogue of the CTA's own 128 rows.
//
// Barriers. raw_full / raw_empty are local. conv_done and acc_empty live in
// the EVEN CTA and collect arrivals from both CTAs (22 converter warps, 16
// epilogue warps); the odd CTA's warps arrive remotely. mma_done and acc_full
// are signalled in both CTAs at once by the MMA's commit. Start and end of the
// kernel are cluster-wide barriers: nobody touches the other CTA's barriers
// before they are initialised, and no CTA leaves (or frees tensor memory) while
// its partner may still be working on the shared tile.
//
// Every wait is bounded (ptx.cuh); a wait that gives up raises the CTA's abort
// flag, all roles stop, and the status word reports it. The partner CTA then
// runs into its own bounded waits.
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdlib>

#include "gemm_kernels.hpp"
#include "ptx.cuh"
#include "tf32x3_common.cuh"

namespace ftcuda {
namespace {

using namespace tf32x3;

constexpr int kCtaRows   = 128;           // rows of A (and D) per CTA
constexpr int kPairRows  = 2 * kCtaRows;  // rows per work item
constexpr int kHalfN     = kTileN / 2;    // 96 columns of B per CTA
constexpr int kStages    = 2;
constexpr int kRawSlots  = 4;

constexpr int kRawABytes     = kCtaRows * kTileK * 4;            // 16 KiB
constexpr int kBoxBytes      = 32 * 32 * 4;                      // one 32(k) x 32(n) box of B
constexpr int kBoxes         = kHalfN / 32;                      // 3
constexpr int kRawSlotBytes  = kRawABytes + kBoxes * kBoxBytes;  // 28 KiB
constexpr int kBTileBytes    = kHalfN * kTileK * 4;              // 12 KiB
constexpr int kBHiOffset     = 0;
constexpr int kBLoOffset     = kBTileBytes;
constexpr int kStageBytes    = 2 * kBTileBytes;
constexpr int kStageOffset   = kRawSlots * kRawSlotBytes;
constexpr int kBarrierOffset = kStageOffset + kStages * kStageBytes;
constexpr int kSmemBytes     = kBarrierOffset + 256 + 1024;

constexpr int kThreads          = 672;  // 21 warps
constexpr int kProducerWarp     = 0;
constexpr int kMmaWarp          = 1;
constexpr int kFirstAConverter  = 4;   // warps 4..7: K values 0-15
constexpr int kFirstEpilogue    = 8;   // warps 8..15
constexpr int kSecondAConverter = 16;  // warps 16..19: K values 16-31
constexpr int kLastBConverter   = 20;  // warps 2, 3 and 20 convert B
constexpr int kConverterWarps   = 8 + kBoxes;
constexpr int kTmemColumns      = 512;
constexpr int kRunningColumn    = kTileN;      // running sum: columns 192..383
constexpr int kAColumn          = 2 * kTileN;  // A operands: 64 columns per stage from 384
constexpr int kHalfColumns      = kTileN / 2;  // columns per epilogue warp
constexpr int kPieces           = kHalfColumns / 16;
constexpr std::uint16_t kBothCtas = 3;

struct Barriers {
    std::uint64_t raw_full[kRawSlots];
    std::uint64_t raw_empty[kRawSlots];
    std::uint64_t mma_done[kStages];
    std::uint64_t conv_done[kStages];  // used in the even CTA
    std::uint64_t acc_full;
    std::uint64_t acc_empty;           // used in the even CTA
    std::uint64_t flush;
    std::uint32_t tmem_base;
    int abort_flag;
};

__global__ void __launch_bounds__(kThreads, 1)
tensorGemm3xTf32Pair(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                     const TensorParams p, const std::uint32_t num_items) {
    extern __shared__ unsigned char smem_raw[];
    const std::uint32_t align_offset = (1024 - (smemAddress(smem_raw) & 1023)) & 1023;
    unsigned char* smem              = smem_raw + align_offset;
    Barriers* bars                   = reinterpret_cast<Barriers*>(smem + kBarrierOffset);
    volatile int* abort_flag         = &bars->abort_flag;

    const int warp                 = threadIdx.x >> 5;
    const int lane                 = threadIdx.x & 31;
    const std::uint32_t rank       = clusterCtaRank();  // 0: issues the MMAs
    const std::uint32_t pair       = blockIdx.x >> 1;
    const std::uint32_t num_pairs  = gridDim.x >> 1;
    const bool leader              = rank == 0;

    if (threadIdx.x == 0) {
        for (int r = 0; r < kRawSlots; ++r) {
            mbarrierInit(&bars->raw_full[r], 1);
            mbarrierInit(&bars->raw_empty[r], kConverterWarps);
        }
        for (int s = 0; s < kStages; ++s) {
            mbarrierInit(&bars->mma_done[s], 1);
            mbarrierInit(&bars->conv_done[s], 2 * kConverterWarps);
        }
        mbarrierInit(&bars->acc_full, 1);
        mbarrierInit(&bars->acc_empty, 16);
        mbarrierInit(&bars->flush, 1);
        bars->abort_flag = 0;
        fenceBarrierInit();
        prefetchTensorMap(&map_a);
        prefetchTensorMap(&map_b);
    }
    __syncthreads();
    // Both CTAs have initialised their barriers before either touches the other's.
    clusterBarrierArrive();
    clusterBarrierWait();
    if (warp == kMmaWarp) { tmemAllocatePair(&bars->tmem_base, kTmemColumns); }
    tcgen05FenceBeforeSync();
    __syncthreads();
    tcgen05FenceAfterSync();
    const std::uint32_t tmem_base = bars->tmem_base;

    // Every role of both CTAs walks the same list of work items and K blocks;
    // `it` counts K blocks over all items and selects the raw slot (it % 4) and
    // the stage (it % 2).
    if (warp == kProducerWarp) {
        // ------------------------------------------------------------ producer
        std::uint32_t it = 0;
        bool ok          = true;
        for (std::uint32_t item = pair; item < num_items && ok; item += num_pairs) {
            const WorkItem w           = decodeItem(p, item, kPairRows);
            const std::int32_t a_row   = static_cast<std::int32_t>(w.tile_m + rank * kCtaRows);
            const std::int32_t b_col   = static_cast<std::int32_t>(w.tile_n + rank * kHalfN);
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
                        tmaLoad2d(slot, &map_a, &bars->raw_full[r], a_row, k_coord);
                    } else {
                        tmaLoad2d(slot, &map_a, &bars->raw_full[r], k_coord, a_row);
                    }
                    if (p.b_k_contiguous != 0) {
                        tmaLoad2d(slot + kRawABytes, &map_b, &bars->raw_full[r], k_coord, b_col);
                    } else {
                        for (int q = 0; q < kBoxes; ++q) {
                            tmaLoad2d(slot + kRawABytes + q * kBoxBytes, &map_b, &bars->raw_full[r], b_col + q * 32, k_coord);
                        }
                    }
                }
                __syncwarp();
            }
        }
        if (!ok) { *abort_flag = 1; }
    } else if (warp == kMmaWarp) {
        // ------------------------------------------------------------ MMA issuer (even CTA only)
        if (leader) {
            const std::uint32_t kInstruction =
                umaInstructionTf32(kPairRows, kTileN) | (p.b_k_contiguous != 0 ? 0U : kUmaBMnMajor);
            std::uint32_t it     = 0;
            std::uint32_t chunks = 0;
            bool ok              = true;
            for (std::uint32_t item = pair; item < num_items && ok; item += num_pairs) {
                const WorkItem w = decodeItem(p, item, kPairRows);
                for (std::uint32_t kb = 0; kb < w.k_blocks && ok; ++kb, ++it) {
                    const bool chunk_start = kb % p.chunk_k_blocks == 0;
                    if (chunk_start) {
                        // The drain warps of both CTAs must have emptied the chunk accumulator.
                        ok = __all_sync(0xFFFFFFFFU, mbarrierWaitCluster(&bars->acc_empty, (chunks & 1) ^ 1, abort_flag));
                        if (!ok) { break; }
                        ++chunks;
                    }
                    const std::uint32_t s   = it % kStages;
                    const std::uint32_t use = it / kStages;
                    ok = __all_sync(0xFFFFFFFFU, mbarrierWaitCluster(&bars->conv_done[s], use & 1, abort_flag));
                    if (!ok) { break; }
                    tcgen05FenceAfterSync();
                    if (lane == 0) {
                        const std::uint32_t stage = smemAddress(smem + kStageOffset + s * kStageBytes);
                        const bool k_major        = p.b_k_contiguous != 0;
                        const std::uint64_t b_hi  = k_major ? umaDescriptorK128(stage + kBHiOffset)
                                                            : umaDescriptorMn128Base32(stage + kBHiOffset, kBoxBytes, 512);
                        const std::uint64_t b_lo  = k_major ? umaDescriptorK128(stage + kBLoOffset)
                                                            : umaDescriptorMn128Base32(stage + kBLoOffset, kBoxBytes, 512);
                        const std::uint64_t k_step = k_major ? 2 : 64;
                        const std::uint32_t a_hi   = tmem_base + kAColumn + s * 64;
                        const std::uint32_t a_lo   = a_hi + 32;
#pragma unroll
                        for (int step = 0; step < kTileK / 8; ++step) {
                            const std::uint64_t advance = static_cast<std::uint64_t>(step) * k_step;
                            const std::uint32_t fresh   = (chunk_start && step == 0) ? 0U : 1U;
                            umaTf32TmemAPair(tmem_base, a_lo + step * 8, b_hi + advance, kInstruction, fresh);
                            umaTf32TmemAPair(tmem_base, a_hi + step * 8, b_lo + advance, kInstruction, 1U);
                            umaTf32TmemAPair(tmem_base, a_hi + step * 8, b_hi + advance, kInstruction, 1U);
                        }
                        umaCommitPair(&bars->mma_done[s], kBothCtas);
                        const bool chunk_end = (kb + 1) % p.chunk_k_blocks == 0 || kb + 1 == w.k_blocks;
                        if (chunk_end) { umaCommitPair(&bars->acc_full, kBothCtas); }
                    }
                    __syncwarp();
                }
            }
            if (!ok) {
                *abort_flag = 1;
                // Let MMAs already issued finish before tensor memory is freed.
                if (lane == 0) {
                    umaCommitPair(&bars->flush, 1);
                    int never = 0;
                    mbarrierWait(&bars->flush, 0, &never);
                }
                __syncwarp();
            }
        }
    } else if (warp < kFirstEpilogue || warp >= kSecondAConverter) {
        // ------------------------------------------------------------ converters
        const bool converts_a = (warp >= kFirstAConverter && warp < kFirstEpilogue) ||
                                (warp >= kSecondAConverter && warp < kLastBConverter);
        const int k_half      = warp >= kSecondAConverter ? 1 : 0;  // A: which 16 K values of the K block
        const int box_index   = warp == kLastBConverter ? 2 : warp - 2;  // B: which 32-column box
        const int a_row       = 32 * (warp & 3) + lane;  // row of A = tensor-memory lane
        std::uint32_t it = 0;
        bool ok          = true;
        for (std::uint32_t item = pair; item < num_items && ok; item += num_pairs) {
            const WorkItem w = decodeItem(p, item, kPairRows);
            for (std::uint32_t kb = 0; kb < w.k_blocks && ok; ++kb, ++it) {
                const std::uint32_t r      = it % kRawSlots;
                const std::uint32_t s      = it % kStages;
                const unsigned char* slot  = smem + r * kRawSlotBytes;
                unsigned char* stage       = smem + kStageOffset + s * kStageBytes;
                ok = mbarrierWait(&bars->raw_full[r], (it / kRawSlots) & 1, abort_flag);
                if (!ok) { break; }
                // The stage (B tiles and A columns, in both CTAs) is free once the
                // MMAs of its previous use have completed.
                ok = mbarrierWait(&bars->mma_done[s], ((it / kStages) & 1) ^ 1, abort_flag);
                if (!ok) { break; }
                tcgen05FenceAfterSync();
                if (converts_a) {
                    // Half a row of A per thread: 4 chunks of 4 floats, un-swizzled by
                    // the row index, split, stored to this stage's A columns.
                    const unsigned char* row   = slot + a_row * 128;
                    const std::uint32_t a_tmem = tmem_base + (static_cast<std::uint32_t>(32 * (warp & 3)) << 16) +
                                                 kAColumn + s * 64 + k_half * 16;
                    float hi[16];
                    float lo[16];
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const int chunk = k_half * 4 + c;
                        float values[4];
                        if (p.a_m_contiguous != 0) {
                            // Raw tile is [32 k][128 m], linear: a column per thread.
                            const float* column = reinterpret_cast<const float*>(slot) + a_row;
#pragma unroll
                            for (int j = 0; j < 4; ++j) { values[j] = column[(chunk * 4 + j) * kCtaRows]; }
                        } else {
                            const float4 raw = *reinterpret_cast<const float4*>(row + ((chunk ^ (a_row & 7)) << 4));
                            values[0] = raw.x;
                            values[1] = raw.y;
                            values[2] = raw.z;
                            values[3] = raw.w;
                        }
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            std::uint32_t hi_bits, lo_bits;
                            splitTf32(values[j], hi_bits, lo_bits);
                            hi[c * 4 + j] = __uint_as_float(hi_bits);
                            lo[c * 4 + j] = __uint_as_float(lo_bits);
                        }
                    }
                    tmemStore16NoWait(a_tmem, hi);
                    tmemStore16NoWait(a_tmem + 32, lo);
                    tmemStoreWait();
                } else {
                    // B: split element by element, same offset in the raw tile and in
                    // B_hi / B_lo (see gemm_tf32x3.cu).
                    const int offset          = box_index * kBoxBytes;
                    const unsigned char* rows = slot + kRawABytes + offset;
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        const int at     = c * 512 + lane * 16;
                        const float4 raw = *reinterpret_cast<const float4*>(rows + at);
                        uint4 hi, lo;
                        splitTf32(raw.x, hi.x, lo.x);
                        splitTf32(raw.y, hi.y, lo.y);
                        splitTf32(raw.z, hi.z, lo.z);
                        splitTf32(raw.w, hi.w, lo.w);
                        *reinterpret_cast<uint4*>(stage + kBHiOffset + offset + at) = hi;
                        *reinterpret_cast<uint4*>(stage + kBLoOffset + offset + at) = lo;
                    }
                }
                // Publish: shared-memory writes to the async proxy, tensor-memory
                // stores (already waited for) to the MMA issuer in the even CTA. The same
                // proxy fence orders this warp's reads of the raw slot before its refill by TMA.
                fenceProxyAsync();
                tcgen05FenceBeforeSync();
                __syncwarp();
                if (lane == 0) {
                    mbarrierArrive(&bars->raw_empty[r]);
                    mbarrierArriveInCta(&bars->conv_done[s], 0);
                }
            }
        }
        if (!ok) { *abort_flag = 1; }
    } else {
        // ------------------------------------------------------------ drain / epilogue (warps 8..15)
        const int e                   = warp - kFirstEpilogue;
        const std::uint32_t lane_base = static_cast<std::uint32_t>(32 * (e & 3));
        const std::uint32_t col_half  = static_cast<std::uint32_t>(kHalfColumns * (e >> 2));
        const std::uint32_t tmem_row  = tmem_base + (lane_base << 16);
        std::uint32_t chunks          = 0;
        bool ok                       = true;
        for (std::uint32_t item = pair; item < num_items && ok; item += num_pairs) {
            const WorkItem w               = decodeItem(p, item, kPairRows);
            const std::uint32_t num_chunks = (w.k_blocks + p.chunk_k_blocks - 1) / p.chunk_k_blocks;
            const std::uint32_t row        = w.tile_m + rank * kCtaRows + lane_base + lane;
            const bool partial             = p.partials != nullptr;
            const float* out_base = partial ? p.partials + static_cast<std::uint64_t>(w.split) * p.m * p.n : p.d;
            const bool vector_ok =
                (p.n & 3) == 0 && (reinterpret_cast<std::uintptr_t>(out_base) & 15) == 0 &&
                (partial || (p.d_col_stride == 1 && (p.d_row_stride & 3) == 0)) &&
                (partial || p.c == nullptr ||
                 (p.c_col_stride == 1 && (p.c_row_stride & 3) == 0 && (reinterpret_cast<std::uintptr_t>(p.c) & 15) == 0));
            for (std::uint32_t chunk = 0; chunk < num_chunks && ok; ++chunk, ++chunks) {
                ok = mbarrierWait(&bars->acc_full, chunks & 1, abort_flag);
                if (!ok) { break; }
                tcgen05FenceAfterSync();
                const bool first = chunk == 0;
                const bool last  = chunk + 1 == num_chunks;
#pragma unroll
                for (int piece = 0; piece < kPieces; ++piece) {
                    float sum[16];
                    tmemLoad16(tmem_row + col_half + piece * 16, sum);
                    if (!first) {
                        float running[16];
                        tmemLoad16(tmem_row + kRunningColumn + col_half + piece * 16, running);
#pragma unroll
                        for (int j = 0; j < 16; ++j) { sum[j] += running[j]; }
                    }
                    if (piece == kPieces - 1) {
                        // This CTA's part of the chunk accumulator has been read.
                        tcgen05FenceBeforeSync();
                        __syncwarp();
                        if (lane == 0) { mbarrierArriveInCta(&bars->acc_empty, 0); }
                    }
                    if (last) {
                        writeRowSegment(p, w, row, w.tile_n + col_half + piece * 16, sum, vector_ok);
                    } else {
                        tmemStore16(tmem_row + kRunningColumn + col_half + piece * 16, sum);
                    }
                }
            }
        }
        if (!ok) { *abort_flag = 1; }
    }

    __syncthreads();
    if (*abort_flag != 0) {
        if (threadIdx.x == 0) {
            if (p.status != nullptr) { *p.status = 4; }
            // Copies that were armed but never consumed may still be landing.
            int never = 0;
            for (int r = 0; r < kRawSlots; ++r) {
                mbarrierWait(&bars->raw_full[r], 0, &never);
                mbarrierWait(&bars->raw_full[r], 1, &never);
            }
        }
        __syncthreads();
    }
    // The partner may still be signalling this CTA's barriers or (even CTA)
    // reading its operands: leave together.
    clusterBarrierArrive();
    clusterBarrierWait();
    if (warp == kMmaWarp) {
        tcgen05FenceAfterSync();
        tmemFreePair(tmem_base, kTmemColumns);
    }
}

}  // namespace

// Off unless FTCUDA_TF32_PAIR=1: measured on B200 (16384 x 4096 x 14336) the pair
// kernel reaches 164 TFLOP/s where the single-CTA kernel reaches 200+; with two
// stages and one chunk accumulator the cross-CTA round trips (converters ->
// issuer, drain -> issuer) are not hidden.
bool tensorPairEnabled() {
    const char* text = std::getenv("FTCUDA_TF32_PAIR");
    return text != nullptr && text[0] == '1';
}

int configureTensorPair(LaunchState& state, char* message, std::size_t capacity) {
    const FtcudaGemmDesc& desc = state.desc;
    const bool a_k_contiguous  = (state.variant & kVariantMaskA) == kVariantTmaAk;
    const bool b_k_contiguous  = (state.variant & kVariantFlagBk) != 0;
    const bool a_encoded =
        a_k_contiguous ? encodeTensorMap2d(&state.map_a, desc.a, desc.k, desc.m,
                                           static_cast<std::uint64_t>(desc.a_row_stride) * sizeof(float), kTileK, kCtaRows,
                                           kSwizzle128, message, capacity)
                       : encodeTensorMap2d(&state.map_a, desc.a, desc.m, desc.k,
                                           static_cast<std::uint64_t>(desc.a_col_stride) * sizeof(float), kCtaRows, kTileK,
                                           kSwizzleNone, message, capacity);
    if (!a_encoded) { return 1; }
    const bool b_encoded =
        b_k_contiguous ? encodeTensorMap2d(&state.map_b, desc.b, desc.k, desc.n,
                                           static_cast<std::uint64_t>(desc.b_col_stride) * sizeof(float), kTileK, kHalfN,
                                           kSwizzle128, message, capacity)
                       : encodeTensorMap2d(&state.map_b, desc.b, desc.n, desc.k,
                                           static_cast<std::uint64_t>(desc.b_row_stride) * sizeof(float), 32, kTileK,
                                           kSwizzle128Atom32, message, capacity);
    if (!b_encoded) { return 1; }
    state.block      = kThreads;
    state.smem_bytes = kSmemBytes;
    const cudaError_t error =
        cudaFuncSetAttribute(tensorGemm3xTf32Pair, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (error != cudaSuccess) {
        return fail(message, capacity, 1, "cudaFuncSetAttribute failed: %s", cudaGetErrorString(error));
    }
    return 0;
}

cudaError_t launchTensorPair(const LaunchState& state, const tf32x3::TensorParams& p, std::uint32_t items,
                             cudaStream_t stream) {
    cudaLaunchConfig_t config{};
    config.gridDim          = dim3(state.grid_x, 1, 1);
    config.blockDim         = dim3(state.block, 1, 1);
    config.dynamicSmemBytes = state.smem_bytes;
    config.stream           = stream;
    cudaLaunchAttribute attribute{};
    attribute.id               = cudaLaunchAttributeClusterDimension;
    attribute.val.clusterDim.x = 2;
    attribute.val.clusterDim.y = 1;
    attribute.val.clusterDim.z = 1;
    config.attrs               = &attribute;
    config.numAttrs            = 1;
    return cudaLaunchKernelEx(&config, tensorGemm3xTf32Pair, state.map_a, state.map_b, p, items);
}

}  // namespace ftcuda
