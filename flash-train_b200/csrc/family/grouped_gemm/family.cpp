#include "family/grouped_gemm/family.hpp"

#include "ftcuda/ftcuda.h"
#include "primitive/cuda/gemm/cuda_grouped_gemm.hpp"

namespace ftrain {
namespace {

GroupedGemmRoles buildRoles(OperationKind operation) {
    const OperandKind grouped = OperandKind::kGroupedTensor;
    const OperandKind list    = OperandKind::kTensorList;
    const OperandKind a_kind  = operation == OperationKind::kGroupedBCDGemm ? list : grouped;
    const OperandKind cd_kind = operation == OperationKind::kGroupedABGemm ? list : grouped;
    PatternBuilder builder;
    GroupedGemmRoles made{};
    made.a       = builder.addOperand(a_kind);
    made.b       = builder.addOperand(grouped);
    made.c       = builder.addOperand(cd_kind);
    made.alpha   = builder.addOperand(OperandKind::kTensor);
    made.beta    = builder.addOperand(OperandKind::kTensor);
    made.d       = builder.addOperand(cd_kind);
    made.gemm    = builder.addOperation(operation, {made.a, made.b, made.c, made.alpha, made.beta}, {made.d});
    made.pattern = builder.build();
    return made;
}

}  // namespace

template<OperationKind kOperation>
const GroupedGemmRoles& GroupedGemmFamilyOf<kOperation>::getRoles() {
    static const GroupedGemmRoles roles = buildRoles(kOperation);
    return roles;
}

template<OperationKind kOperation>
std::vector<std::shared_ptr<const Primitive<GroupedGemmProblem>>> GroupedGemmFamilyOf<kOperation>::makeRecords() {
    return {
        std::make_shared<CudaGroupedGemm>(FTCUDA_GROUPED_GEMM_EXACT),
        std::make_shared<CudaGroupedGemm>(FTCUDA_GROUPED_GEMM_TF32X3),
    };
}

template<OperationKind kOperation>
GroupedGemmProblem GroupedGemmFamilyOf<kOperation>::makeProblem(const Args& args) {
    const GroupedGemmRoles& roles = getRoles();
    const auto tensor             = [&args](std::uint64_t role) { return std::get<Tensor>(*args.getOperand(role)); };
    return GroupedGemmProblem(*args.getOperand(roles.a), *args.getOperand(roles.b), *args.getOperand(roles.c), *args.getOperand(roles.d),
                              tensor(roles.alpha), tensor(roles.beta), args.getOpArgument(roles.gemm)->compute_type);
}

template struct GroupedGemmFamilyOf<OperationKind::kGroupedABCDGemm>;
template struct GroupedGemmFamilyOf<OperationKind::kGroupedBCDGemm>;
template struct GroupedGemmFamilyOf<OperationKind::kGroupedABGemm>;

std::vector<std::string> GroupedB200Heuristic::findCandidates(const GroupedGemmProblem&, const Constraints&) {
    return {cudaGroupedGemmName(FTCUDA_GROUPED_GEMM_TF32X3), cudaGroupedGemmName(FTCUDA_GROUPED_GEMM_EXACT)};
}

}  // namespace ftrain
