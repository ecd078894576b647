#include "family/gemm/finder.hpp"

#include "ftcuda/ftcuda.h"
#include "primitive/cuda/gemm/cuda_gemm.hpp"

namespace ftrain {
namespace {

std::uint64_t ceilDiv(std::uint64_t x, std::uint64_t y) { return (x + y - 1) / y; }

}  // namespace

// Regime map on B200 (148 SMs; the count is queried, not assumed):
//   * very few rows of A (m <= 32): B is streamed exactly once, the problem is
//     HBM-bound -> the skinny kernel first.
//   * enough rows/columns to fill 128x192 tensor-core tiles: 3xTF32 on tcgen05.
//     If the last wave of those tiles would leave more than a tenth of the SMs
//     idle while K is long enough to cut, the split-K variant (workspace
//     needed) goes first so that K slices even out the waves; the unsplit
//     kernels follow for callers without workspace.
//   * everything else: exact-FP32 SIMT, split along K when its 128x128 tiles
//     leave most SMs idle and K is long.
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

    if (shape.m * shape.n == 0) { return {simt}; }
    if (shape.m <= 32 && shape.k >= 256) { return {skinny, simt_split, simt}; }

    const bool fills_tensor_tiles = shape.m >= 128 && shape.n >= 128 && shape.k >= 256;
    if (fills_tensor_tiles) {
        const std::uint64_t tiles = ceilDiv(shape.m, 128) * ceilDiv(shape.n, 192);
        const std::uint64_t waves = ceilDiv(tiles, sm_count);
        const bool ragged         = tiles * 10 < waves * sm_count * 9;  // last wave under 90 % full overall
        if (ragged && shape.k >= 8192) { return {tensor_split, tensor, simt_split, simt}; }
        return {tensor, simt};
    }
    const std::uint64_t simt_tiles = ceilDiv(shape.m, 128) * ceilDiv(shape.n, 128);
    if (simt_tiles * 2 <= sm_count && shape.k >= 2048) { return {simt_split, simt}; }
    return {simt};
}

}  // namespace ftrain
