#include "primitive/cuda/gemm/cuda_grouped_gemm.hpp"

#include <cstdint>

namespace ftrain {
namespace {

constexpr GroupedPort kPorts[] = {GroupedPort::kA, GroupedPort::kB, GroupedPort::kC, GroupedPort::kD};

bool floatAligned(const void* address) noexcept { return reinterpret_cast<std::uintptr_t>(address) % alignof(float) == 0; }

const float* groupAddress(const GroupedGemmProblem& problem, GroupedPort port, std::uint32_t group) noexcept {
    return problem.getGroup(port, group).address();
}

}  // namespace

const char* cudaGroupedGemmName(int kernel) noexcept {
    switch (kernel) {
        case FTCUDA_GROUPED_GEMM_EXACT: return "GroupedFp32Gemm";
        case FTCUDA_GROUPED_GEMM_TF32X3: return "GroupedFp32Gemm3xTf32";
        default: return nullptr;
    }
}

std::vector<FtcudaGemmDesc> makeCudaGroupedDescs(const GroupedGemmProblem& problem, FTrainDeviceId device, bool read_scalars) {
    float alpha = 0.0F, beta = 0.0F;
    if (read_scalars) {
        alpha = *static_cast<const float*>(problem.getAlpha().getMemory());
        beta  = *static_cast<const float*>(problem.getBeta().getMemory());
    }
    std::vector<FtcudaGemmDesc> descs(problem.getNumGroups());
    for (std::uint32_t g = 0; g < problem.getNumGroups(); ++g) {
        const GroupMatrix& a = problem.getGroup(GroupedPort::kA, g);
        const GroupMatrix& b = problem.getGroup(GroupedPort::kB, g);
        const GroupMatrix& c = problem.getGroup(GroupedPort::kC, g);
        const GroupMatrix& d = problem.getGroup(GroupedPort::kD, g);
        FtcudaGemmDesc& desc = descs[g];
        desc                 = FtcudaGemmDesc{};
        desc.a               = groupAddress(problem, GroupedPort::kA, g);
        desc.b               = groupAddress(problem, GroupedPort::kB, g);
        desc.c               = groupAddress(problem, GroupedPort::kC, g);
        desc.d               = const_cast<float*>(groupAddress(problem, GroupedPort::kD, g));
        desc.alpha           = alpha;
        desc.beta            = beta;
        desc.m               = static_cast<std::uint64_t>(a.rows);
        desc.k               = static_cast<std::uint64_t>(a.cols);
        desc.n               = static_cast<std::uint64_t>(b.cols);
        desc.a_row_stride    = a.row_stride;
        desc.a_col_stride    = a.col_stride;
        desc.b_row_stride    = b.row_stride;
        desc.b_col_stride    = b.col_stride;
        desc.c_row_stride    = c.row_stride;
        desc.c_col_stride    = c.col_stride;
        desc.d_row_stride    = d.row_stride;
        desc.d_col_stride    = d.col_stride;
        desc.device          = device;
    }
    return descs;
}

Result CudaGroupedGemm::isApplicable(const GroupedGemmProblem& problem, const Constraints& constraints) const {
    if (problem.getComputeType() != FTRAIN_NUMERIC_TYPE_FP32) { return Result(FTRAIN_STATUS_UNSUPPORTED, "compute type is not fp32"); }
    for (const GroupedPort port : kPorts) {
        const GroupedOperand& operand = problem.getOperand(port);
        if (operand.numeric_type != FTRAIN_NUMERIC_TYPE_FP32) { return Result(FTRAIN_STATUS_UNSUPPORTED, "an operand is not fp32"); }
        if (!operand.plainly_indexed) { return Result(FTRAIN_STATUS_UNSUPPORTED, "an operand's data is not continuously indexed"); }
        if (!operand.float_aligned) { return Result(FTRAIN_STATUS_UNSUPPORTED, "an operand address is not float-aligned"); }
    }
    for (const StorageView* scalar : {&problem.getAlpha(), &problem.getBeta()}) {
        if (scalar->getNumericType() != FTRAIN_NUMERIC_TYPE_FP32) { return Result(FTRAIN_STATUS_UNSUPPORTED, "an operand is not fp32"); }
        if (scalar->getIndexType() != FTRAIN_INDEX_TYPE_CONTINUOUS) {
            return Result(FTRAIN_STATUS_UNSUPPORTED, "an operand is not continuously indexed");
        }
        if (!floatAligned(scalar->getMemory())) { return Result(FTRAIN_STATUS_UNSUPPORTED, "an operand address is not float-aligned"); }
    }
    if (!problem.hasEmptyOutput()) {
        // d needs an address wherever it has elements, a and b wherever they are multiplied. A group whose
        // c has no address simply has no beta * C term.
        bool addressed = true;
        for (std::uint32_t g = 0; g < problem.getNumGroups(); ++g) {
            const GroupMatrix& a = problem.getGroup(GroupedPort::kA, g);
            const GroupMatrix& b = problem.getGroup(GroupedPort::kB, g);
            if (a.rows * b.cols == 0) { continue; }
            addressed = addressed && problem.getGroup(GroupedPort::kD, g).base != nullptr;
            if (a.cols != 0) { addressed = addressed && a.base != nullptr && b.base != nullptr; }
        }
        if (!addressed) { return Result(FTRAIN_STATUS_UNSUPPORTED, "a required operand address is null"); }
    }
    const std::vector<FtcudaGemmDesc> descs = makeCudaGroupedDescs(problem, constraints.getDeviceId(), false);
    char reason[256];
    reason[0] = '\0';
    if (ftcuda_grouped_gemm_supports(kernel_, descs.data(), static_cast<std::uint32_t>(descs.size()), reason, sizeof reason) != 0) {
        return Result(FTRAIN_STATUS_UNSUPPORTED, reason);
    }
    return Result{};
}

void CudaGroupedGemm::configure(const GroupedGemmProblem& problem) {
    launch_.reset();
    workspace_bytes_ = 0;
    if (problem.hasEmptyOutput()) { return; }
    const std::vector<FtcudaGemmDesc> descs = makeCudaGroupedDescs(problem, getCurrentDeviceId(), true);
    char reason[256];
    reason[0]                      = '\0';
    FtcudaGroupedGemmLaunch* made = nullptr;
    if (ftcuda_grouped_gemm_configure(kernel_, descs.data(), static_cast<std::uint32_t>(descs.size()), &made, reason, sizeof reason) != 0) {
        throw Exception(FTRAIN_STATUS_INTERNAL_ERROR, "%s: configuring the launch failed: %s", getName(), reason);
    }
    launch_.reset(made, [](FtcudaGroupedGemmLaunch* launch) { ftcuda_grouped_gemm_destroy(launch); });
    workspace_bytes_ = ftcuda_grouped_gemm_workspace_bytes(made);
}

void CudaGroupedGemm::executeImpl(const Resources& resources) {
    if (launch_ == nullptr) { return; }
    char reason[256];
    reason[0] = '\0';
    if (ftcuda_grouped_gemm_launch(launch_.get(), resources.getWorkspace(), resources.getWorkspaceBytes(), resources.getStream(), reason,
                                   sizeof reason) != 0) {
        throw Exception(FTRAIN_STATUS_INTERNAL_ERROR, "grouped FP32 GEMM kernel launch failed: %s", reason);
    }
}

}  // namespace ftrain
