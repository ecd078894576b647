#include "family/grouped_gemm/family.hpp"

#include "ftcuda/ftcuda.h"
#include "primitive/cuda/gemm/cuda_grouped_gemm.hpp"

namespace ftrain {

const GroupedGemmFamily::Roles& GroupedGemmFamily::getRoles() {
    static const Roles roles = [] {
        PatternBuilder builder;
        Roles made{};
        made.a     = builder.addOperand(OperandKind::kGroupedTensor);
        made.b     = builder.addOperand(OperandKind::kGroupedTensor);
        made.c     = builder.addOperand(OperandKind::kGroupedTensor);
        made.alpha = builder.addOperand(OperandKind::kTensor);
        made.beta  = builder.addOperand(OperandKind::kTensor);
        made.d     = builder.addOperand(OperandKind::kGroupedTensor);
        made.gemm  = builder.addOperation(OperationKind::kGroupedABCDGemm, {made.a, made.b, made.c, made.alpha, made.beta}, {made.d});
        made.pattern = builder.build();
        return made;
    }();
    return roles;
}

std::vector<std::shared_ptr<const Primitive<GroupedGemmProblem>>> GroupedGemmFamily::makeRecords() {
    return {
        std::make_shared<CudaGroupedGemm>(FTCUDA_GROUPED_GEMM_EXACT),
        std::make_shared<CudaGroupedGemm>(FTCUDA_GROUPED_GEMM_TF32X3),
    };
}

GroupedGemmProblem GroupedGemmFamily::makeProblem(const Args& args) {
    const Roles& roles = getRoles();
    const auto grouped = [&args](std::uint64_t role) { return std::get<GroupedTensor>(*args.getOperand(role)); };
    const auto tensor  = [&args](std::uint64_t role) { return std::get<Tensor>(*args.getOperand(role)); };
    return GroupedGemmProblem(grouped(roles.a), grouped(roles.b), grouped(roles.c), grouped(roles.d), tensor(roles.alpha),
                              tensor(roles.beta), args.getOpArgument(roles.gemm)->compute_type);
}

std::vector<std::string> GroupedB200Heuristic::findCandidates(const GroupedGemmProblem&, const Constraints&) {
    return {cudaGroupedGemmName(FTCUDA_GROUPED_GEMM_TF32X3), cudaGroupedGemmName(FTCUDA_GROUPED_GEMM_EXACT)};
}

}  // namespace ftrain
