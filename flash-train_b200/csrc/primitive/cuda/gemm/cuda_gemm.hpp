// The Gemm family's Primitives on the CUDA platform.
//
// One host class serves every kernel family of the platform layer
// (ftcuda/ftcuda.h): the object knows its kernel id, asks the platform whether
// the kernel supports a problem, has it pre-build the launch (tile shape, grid,
// TMA descriptors) at configure time, and at execute time only forwards the
// stored launch. It takes the place of the reference's single Fp32Gemm
// Primitive (src/include/flash_train/primitive/hygon/gemm/fp32_gemm.hpp:29-53,
// src/primitive/hygon/gemm/fp32_gemm.cpp:20-81), and the kernel with id
// FTCUDA_GEMM_SIMT keeps that Primitive's name, "Fp32Gemm".
//
// Differences from the reference's support checklist: a, b, c and d may be
// strided views (index type INVALID with strides) as well as CONTINUOUS.
#ifndef FTRAIN_PRIMITIVE_CUDA_GEMM_CUDA_GEMM_HPP_
#define FTRAIN_PRIMITIVE_CUDA_GEMM_CUDA_GEMM_HPP_

#include <cstdint>
#include <memory>

#include "core/primitive.hpp"
#include "family/gemm/problem.hpp"
#include "ftcuda/ftcuda.h"

namespace ftrain {

// "Fp32Gemm", "Fp32Gemm3xTf32", "Fp32Gemm3xTf32SplitK", "Fp32GemmSkinny",
// "Fp32GemmSplitK" for the ids of ftcuda.h; nullptr for an unknown id.
const char* cudaGemmName(int kernel) noexcept;

// Translates a problem into the platform's raw descriptor. alpha and beta are
// read from host memory here, as in the reference (fp32_gemm.cpp:70-72).
FtcudaGemmDesc makeCudaGemmDesc(const GemmProblem& problem, FTrainDeviceId device, bool read_scalars);

class CudaGemm final : public Primitive<GemmProblem> {
  public:
    explicit CudaGemm(int kernel) noexcept : kernel_(kernel) {}

    const char* getName() const noexcept override { return cudaGemmName(kernel_); }
    std::unique_ptr<PrimitiveBase> clone() const override { return std::make_unique<CudaGemm>(*this); }
    Result isApplicable(const GemmProblem& problem, const Constraints& constraints) const override;
    std::uint64_t getRequiredWorkspaceBytes() const noexcept override { return workspace_bytes_; }
    // Binds to the calling thread's current device.
    void configure(const GemmProblem& problem) override;

  private:
    void executeImpl(const Resources& resources) override;

    int kernel_;
    bool empty_{true};  // nothing to launch (m * n == 0, or not configured)
    std::uint64_t workspace_bytes_{0};
    FtcudaGemmLaunch launch_{};
};

}  // namespace ftrain

#endif
