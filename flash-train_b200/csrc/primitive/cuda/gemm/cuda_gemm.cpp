#include "primitive/cuda/gemm/cuda_gemm.hpp"

#include <cstdint>

namespace ftrain {
namespace {

bool floatAligned(const void* address) noexcept {
    return reinterpret_cast<std::uintptr_t>(address) % alignof(float) == 0;  // null is aligned
}

constexpr GemmPort kAllPorts[]    = {GemmPort::kA, GemmPort::kB,     GemmPort::kC,
                                     GemmPort::kD, GemmPort::kAlpha, GemmPort::kBeta};
constexpr GemmPort kMatrixPorts[] = {GemmPort::kA, GemmPort::kB, GemmPort::kC, GemmPort::kD};

}  // namespace

const char* cudaGemmName(int kernel) noexcept {
    switch (kernel) {
        case FTCUDA_GEMM_SIMT: return "Fp32Gemm";
        case FTCUDA_GEMM_TF32X3: return "Fp32Gemm3xTf32";
        case FTCUDA_GEMM_TF32X3_SPLITK: return "Fp32Gemm3xTf32SplitK";
        case FTCUDA_GEMM_SKINNY: return "Fp32GemmSkinny";
        case FTCUDA_GEMM_SIMT_SPLITK: return "Fp32GemmSplitK";
        case FTCUDA_GEMM_TF32X3_ROWS: return "Fp32Gemm3xTf32FewRows";
        default: return nullptr;
    }
}

FtcudaGemmDesc makeCudaGemmDesc(const GemmProblem& problem, FTrainDeviceId device, bool read_scalars) {
    FtcudaGemmDesc desc{};
    desc.a = static_cast<const float*>(problem.getAddress(GemmPort::kA));
    desc.b = static_cast<const float*>(problem.getAddress(GemmPort::kB));
    desc.c = static_cast<const float*>(problem.getAddress(GemmPort::kC));
    desc.d = static_cast<float*>(problem.getAddress(GemmPort::kD));
    if (read_scalars) {
        desc.alpha = *static_cast<const float*>(problem.getAddress(GemmPort::kAlpha));
        desc.beta  = *static_cast<const float*>(problem.getAddress(GemmPort::kBeta));
    }
    const GemmShape shape = problem.getShape();
    desc.m                = shape.m;
    desc.n                = shape.n;
    desc.k                = shape.k;
    const MatrixLayout a  = problem.getLayout(GemmPort::kA);
    const MatrixLayout b  = problem.getLayout(GemmPort::kB);
    const MatrixLayout c  = problem.getLayout(GemmPort::kC);
    const MatrixLayout d  = problem.getLayout(GemmPort::kD);
    desc.a_row_stride     = a.row_stride;
    desc.a_col_stride     = a.col_stride;
    desc.b_row_stride     = b.row_stride;
    desc.b_col_stride     = b.col_stride;
    desc.c_row_stride     = c.row_stride;
    desc.c_col_stride     = c.col_stride;
    desc.d_row_stride     = d.row_stride;
    desc.d_col_stride     = d.col_stride;
    desc.device           = device;
    return desc;
}

// The checklist, in the reference's order and with its wording
// (fp32_gemm.cpp:27-62), followed by the platform's per-kernel rules.
Result CudaGemm::isApplicable(const GemmProblem& problem, const Constraints& constraints) const {
    if (problem.getComputeType() != FTRAIN_NUMERIC_TYPE_FP32) {
        return Result(FTRAIN_STATUS_UNSUPPORTED, "compute type is not fp32");
    }
    for (const GemmPort port : kAllPorts) {
        if (problem.getNumericType(port) != FTRAIN_NUMERIC_TYPE_FP32) {
            return Result(FTRAIN_STATUS_UNSUPPORTED, "an operand is not fp32");
        }
    }
    for (const GemmPort port : kMatrixPorts) {
        const FTrainIndexType index_type = problem.getIndexType(port);
        if (index_type != FTRAIN_INDEX_TYPE_CONTINUOUS && index_type != FTRAIN_INDEX_TYPE_INVALID) {
            return Result(FTRAIN_STATUS_UNSUPPORTED, "an operand is not continuously indexed");
        }
    }
    if (problem.getIndexType(GemmPort::kAlpha) != FTRAIN_INDEX_TYPE_CONTINUOUS ||
        problem.getIndexType(GemmPort::kBeta) != FTRAIN_INDEX_TYPE_CONTINUOUS) {
        return Result(FTRAIN_STATUS_UNSUPPORTED, "an operand is not continuously indexed");
    }
    for (const GemmPort port : kAllPorts) {
        if (!floatAligned(problem.getAddress(port))) {
            return Result(FTRAIN_STATUS_UNSUPPORTED, "an operand address is not float-aligned");
        }
    }
    if (!problem.hasEmptyOutput()) {
        const bool addressed = problem.getAddress(GemmPort::kD) != nullptr &&
                               (problem.getShape().k == 0 || (problem.getAddress(GemmPort::kA) != nullptr &&
                                                              problem.getAddress(GemmPort::kB) != nullptr));
        if (!addressed) { return Result(FTRAIN_STATUS_UNSUPPORTED, "a required operand address is null"); }
    }
    const FtcudaGemmDesc desc = makeCudaGemmDesc(problem, constraints.getDeviceId(), false);
    char reason[256];
    reason[0] = '\0';
    if (ftcuda_gemm_supports(kernel_, &desc, reason, sizeof reason) != 0) {
        return Result(FTRAIN_STATUS_UNSUPPORTED, reason);
    }
    return Result{};
}

void CudaGemm::configure(const GemmProblem& problem) {
    empty_           = problem.hasEmptyOutput();
    workspace_bytes_ = 0;
    if (empty_) { return; }
    const FtcudaGemmDesc desc = makeCudaGemmDesc(problem, getCurrentDeviceId(), true);
    char reason[256];
    reason[0] = '\0';
    if (ftcuda_gemm_configure(kernel_, &desc, &launch_, reason, sizeof reason) != 0) {
        throw Exception(FTRAIN_STATUS_INTERNAL_ERROR, "%s: configuring the launch failed: %s", getName(), reason);
    }
    workspace_bytes_ = ftcuda_gemm_workspace_bytes(&launch_);
}

void CudaGemm::executeImpl(const Resources& resources) {
    if (empty_) { return; }
    char reason[256];
    reason[0] = '\0';
    if (ftcuda_gemm_launch(&launch_, resources.getWorkspace(), resources.getWorkspaceBytes(), resources.getStream(),
                           reason, sizeof reason) != 0) {
        throw Exception(FTRAIN_STATUS_INTERNAL_ERROR, "FP32 GEMM kernel launch failed: %s", reason);
    }
}

}  // namespace ftrain
