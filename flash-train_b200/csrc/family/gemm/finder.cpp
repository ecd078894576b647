#include "family/gemm/finder.hpp"

#include "ftcuda/ftcuda.h"
#include "primitive/cuda/gemm/cuda_gemm.hpp"

namespace ftrain {
namespace {

std::uint64_t ceilDiv(std::uint64_t x, std::uint64_t y) { return (x + y - 1) / y; }

}  // namespace

// Regime map on B200 (148 SMs; the count is queried, not assumed). The
// thresholds come from timing every kernel family on a grid of shapes
// (bench.py --workload finder_sweep) and keeping the Finder's first choice
// within about 1.4x of the fastest family everywhere on it:
//   * very few rows of A (m <= 32): B is streamed exactly once, the problem is
//     HBM-bound -> the few-rows kernel first -- unless B is so narrow that its
//     strips (128 columns, or 32 rows of a B given contiguous along K) times
//     the 8 K slices of a cluster leave most SMs without a CTA; then, with K
//     long enough to cut, the tensor-core split-K kernel goes first.
//   * from 33 rows on, with at least 128 columns: 3xTF32 on tcgen05 (its
//     128-row tile beats the SIMT kernel even when only a quarter full). If
//     the 128x192 tiles fill less than 90 % of the SMs' waves and K >= 2048,
//     the split-K variant (workspace needed) goes first so that K slices even
//     out the waves; the unsplit kernels follow for callers without workspace.
//     With a medium K (512 ... 2047) the split pays only while the tiles fill
//     under a quarter of a wave (two launches; the partial sums stay small).
//   * small outputs with a short K: exact-FP32 SIMT on 32x32 tiles ahead of the
//     tensor kernel (see below).
//   * everything else: exact-FP32 SIMT, split along K when its 128x128 tiles
//     leave most SMs idle and K >= 512.
// Every list ends with "Fp32Gemm", which needs no workspace and accepts every
// layout, so a caller walking the Plan by workspace budget always finds a
// runnable index.
std::vector<std::string> B200Heuristic::findCandidates(const GemmProblem& problem, const Constraints& constraints) {
    const GemmShape shape = problem.getShape();
    std::int32_t sms      = 148;
    if (ftcuda_device_sm_count(constraints.getDeviceId(), &sms, nullptr, 0) != 0 || sms <= 0) { sms = 148; }
    const std::uint64_t sm_count = static_cast<std::uint64_t>(sms);

    const char* simt         = cudaGemmName(FTCUDA_GEMM_SIMT);
    const char* tensor       = cudaGemmName(FTCUDA_GEMM_TF32X3);
    const char* tensor_split = cudaGemmName(FTCUDA_GEMM_TF32X3_SPLITK);
    const char* skinny       = cudaGemmName(FTCUDA_GEMM_SKINNY);
    const char* simt_split   = cudaGemmName(FTCUDA_GEMM_SIMT_SPLITK);

    const char* tensor_rows  = cudaGemmName(FTCUDA_GEMM_TF32X3_ROWS);

    if (shape.m * shape.n == 0) { return {simt}; }
    const bool b_along_k = problem.getLayout(GemmPort::kB).row_stride == 1 && shape.n > 1;
    // The tensor few-rows kernel (B as the tensor core's 128-row operand): one CTA per 128-column
    // strip and K slice, at most eight slices. Measured against the other families on B200:
    // it wins from 9 rows on for large B -- where the exact few-rows kernel changes to its 16-row form:
    // 22 against 27 us at 9 to 12 rows of 4096 x 4096 -- (from 17 rows whatever the size, K >= 1024), and up
    // to 64 rows, except where a narrow, deep problem leaves it too few CTAs: then the
    // split-K tensor kernel, which cuts K as finely as it likes, comes first.
    if (shape.m >= 9 && shape.m <= 64 && shape.n >= 128 && shape.k >= 256) {
        const std::uint64_t strips = ceilDiv(shape.n, 128);
        bool rows_first            = false;
        bool deep                  = false;  // too deep for eight K slices per strip
        if (shape.m <= 16) {
            rows_first = shape.k >= 1024 && shape.k * shape.n >= (8ULL << 20) && (!b_along_k || strips >= 32);
        } else if (shape.m <= 32) {
            rows_first = shape.k >= 2048 || (shape.k >= 1024 && strips >= 32);
        } else {
            rows_first = true;
        }
        deep = strips * 16 <= sm_count && shape.k >= 32768;
        if (deep && (rows_first || shape.k >= 32768)) { return {tensor_split, tensor_rows, skinny, tensor, simt_split, simt}; }
        if (rows_first) { return {tensor_rows, tensor_split, skinny, tensor, simt_split, simt}; }
    }
    if (shape.m <= 32 && shape.k >= 256) {
        const std::uint64_t strip      = b_along_k ? 32 : 128;
        const std::uint64_t few_ctas   = ceilDiv(shape.n, strip) * 8;  // CTAs the few-rows kernel can start
        // The more rows, the more arithmetic per CTA (from 17 rows on the kernel is
        // bound by the FP32 pipe and runs one CTA per SM), the more CTAs it needs.
        // Beyond 24 rows the tensor cores win whatever the width.
        const bool narrow = few_ctas * 4 <= sm_count || (few_ctas * 2 <= sm_count && shape.m > 8) ||
                            (few_ctas <= sm_count && shape.m > 16) || shape.m > 24;
        if (narrow && shape.k >= 2048) { return {tensor_split, skinny, simt_split, simt}; }
        return {skinny, simt_split, simt};
    }

    const std::uint64_t simt_tiles = ceilDiv(shape.m, 128) * ceilDiv(shape.n, 128);
    // Small outputs with a short K (64^3 ... 256^3, 384 x 256 x 320): the exact kernel runs them on 32 x 32
    // tiles -- many CTAs, a short K loop each -- in about 6 to 10 us of device time, where the tensor
    // kernel's pipeline set-up and cluster exchange cost over 20 (256^3: 10.3 against 22.2 us). The
    // condition mirrors the one under which the platform picks that tiling; up to about 48 M
    // multiply-adds -- 80 M when K is at most 512: 384 x 512 x 384 runs in 14.4 against 18.4 us -- the
    // exact kernel stays ahead (512^3: 24.6 against 18.0; 256 x 1024 x 256: 22.6 against 16.0).
    const std::uint64_t tiles64 = ceilDiv(shape.m, 64) * ceilDiv(shape.n, 64);
    const std::uint64_t tiles32 = ceilDiv(shape.m, 32) * ceilDiv(shape.n, 32);
    if (shape.m >= 33 && (shape.k <= 512 || (shape.k <= 1024 && tiles32 >= 32)) && tiles64 * 4 <= sm_count &&
        tiles32 <= 2 * sm_count && shape.m * shape.n * shape.k <= ((shape.k <= 512 ? 80ULL : 48ULL) << 20)) {
        if (shape.n >= 128 && shape.k >= 256) { return {simt, tensor}; }
        return {simt};
    }
    if (shape.m >= 33 && shape.n >= 128 && shape.k >= 256) {
        const std::uint64_t tiles = ceilDiv(shape.m, 128) * ceilDiv(shape.n, 192);
        const std::uint64_t waves = ceilDiv(tiles, sm_count);
        const bool ragged         = tiles * 10 < waves * sm_count * 9;  // the waves are under 90 % full overall
        // With few tiles the single-launch kernel cuts K over a thread-block cluster by itself. Under half
        // a wave of tiles that beats split-K with its second kernel whenever K is at most 2048 (one tile
        // of 128 x 1024 x 192: 16 against 21 us; 256 x 2048 x 2048: 25 against 27) and, up to a K of 4096,
        // from an eighth of a wave on (128 x 4096 x 4096, 22 tiles: 35 against 41 us; 8 tiles: 31 against
        // 27); deeper K or fewer tiles stay with split-K and its finer slices.
        if (tiles * 2 <= sm_count && shape.k >= 512 && (shape.k <= 2048 || (shape.k <= 4096 && tiles * 8 >= sm_count))) {
            return {tensor, tensor_split, simt_split, simt};
        }
        if (ragged && shape.k >= 2048) { return {tensor_split, tensor, simt_split, simt}; }
        // A medium K is worth cutting (two launches, partial sums re-read by the
        // second) only while the tiles fill under a quarter of a wave.
        if (shape.k >= 512 && tiles * 4 <= sm_count) { return {tensor_split, tensor, simt_split, simt}; }
        return {tensor, simt};
    }
    if (simt_tiles * 2 <= sm_count && shape.k >= 512) { return {simt_split, simt}; }
    return {simt};
}

}  // namespace ftrain
