#include "family/gemm/family.hpp"

#include "ftcuda/ftcuda.h"
#include "primitive/cuda/gemm/cuda_gemm.hpp"

namespace ftrain {

const GemmFamily::Roles& GemmFamily::getRoles() {
    static const Roles roles = [] {
        PatternBuilder builder;
        Roles made{};
        made.a     = builder.addOperand(OperandKind::kTensor);
        made.b     = builder.addOperand(OperandKind::kTensor);
        made.c     = builder.addOperand(OperandKind::kTensor);
        made.alpha = builder.addOperand(OperandKind::kTensor);
        made.beta  = builder.addOperand(OperandKind::kTensor);
        made.d     = builder.addOperand(OperandKind::kTensor);
        made.gemm  = builder.addOperation(OperationKind::kGemm, {made.a, made.b, made.c, made.alpha, made.beta}, {made.d});
        made.pattern = builder.build();
        return made;
    }();
    return roles;
}

std::vector<std::shared_ptr<const Primitive<GemmProblem>>> GemmFamily::makeRecords() {
    return {
        std::make_shared<CudaGemm>(FTCUDA_GEMM_SIMT),
        std::make_shared<CudaGemm>(FTCUDA_GEMM_TF32X3),
        std::make_shared<CudaGemm>(FTCUDA_GEMM_SKINNY),
        std::make_shared<CudaGemm>(FTCUDA_GEMM_TF32X3_SPLITK),
        std::make_shared<CudaGemm>(FTCUDA_GEMM_SIMT_SPLITK),
        std::make_shared<CudaGemm>(FTCUDA_GEMM_TF32X3_ROWS),
    };
}

GemmProblem GemmFamily::makeProblem(const Args& args) {
    const Roles& roles = getRoles();
    const auto tensor  = [&args](std::uint64_t role) { return std::get<Tensor>(*args.getOperand(role)); };
    return GemmProblem(tensor(roles.a), tensor(roles.b), tensor(roles.c), tensor(roles.d), tensor(roles.alpha),
                       tensor(roles.beta), args.getOpArgument(roles.gemm)->compute_type);
}

}  // namespace ftrain
