// The GroupedABCDGemm family's Primitives on the CUDA platform: "GroupedFp32Gemm" (exact FP32, one
// launch of the exact kernels per group, no workspace) and "GroupedFp32Gemm3xTf32" (one persistent
// tensor-core launch over the tiles of all groups; its per-group table lives in the workspace).
// Both stand on the grouped entry points of ftcuda/ftcuda.h. The reference has no Primitive for this
// operation; the support checklist mirrors its Fp32Gemm's (src/primitive/hygon/gemm/fp32_gemm.cpp:27-62
// there) group by group.
#ifndef FTRAIN_PRIMITIVE_CUDA_GEMM_CUDA_GROUPED_GEMM_HPP_
#define FTRAIN_PRIMITIVE_CUDA_GEMM_CUDA_GROUPED_GEMM_HPP_

#include <cstdint>
#include <memory>
#include <vector>

#include "core/primitive.hpp"
#include "family/grouped_gemm/problem.hpp"
#include "ftcuda/ftcuda.h"

namespace ftrain {

const char* cudaGroupedGemmName(int kernel) noexcept;

// One raw descriptor per group (empty groups included, so that indices agree). alpha and beta are
// read from host memory when read_scalars is set.
std::vector<FtcudaGemmDesc> makeCudaGroupedDescs(const GroupedGemmProblem& problem, FTrainDeviceId device, bool read_scalars);

class CudaGroupedGemm final : public Primitive<GroupedGemmProblem> {
  public:
    explicit CudaGroupedGemm(int kernel) noexcept : kernel_(kernel) {}

    const char* getName() const noexcept override { return cudaGroupedGemmName(kernel_); }
    // A clone shares the configured launch (immutable once made); configuring the clone replaces it.
    std::unique_ptr<PrimitiveBase> clone() const override { return std::make_unique<CudaGroupedGemm>(*this); }
    Result isApplicable(const GroupedGemmProblem& problem, const Constraints& constraints) const override;
    std::uint64_t getRequiredWorkspaceBytes() const noexcept override { return workspace_bytes_; }
    void configure(const GroupedGemmProblem& problem) override;

  private:
    void executeImpl(const Resources& resources) override;

    int kernel_;
    std::uint64_t workspace_bytes_{0};
    std::shared_ptr<FtcudaGroupedGemmLaunch> launch_;  // null: nothing to launch
};

}  // namespace ftrain

#endif
