// What the grouped-GEMM families hand to their engines: supported Pattern, Primitive catalogue,
// Problem factory -- one family per grouped operation of the public API. The operations exist in
// the reference's public API without an engine (include/flash_train/common.h:248-306,
// src/engine.cpp:25-27 there); here each has one.
#ifndef FTRAIN_FAMILY_GROUPED_GEMM_FAMILY_HPP_
#define FTRAIN_FAMILY_GROUPED_GEMM_FAMILY_HPP_

#include <memory>
#include <string>
#include <vector>

#include "core/constraints.hpp"
#include "core/ops_args.hpp"
#include "core/pattern.hpp"
#include "core/primitive.hpp"
#include "family/grouped_gemm/problem.hpp"

namespace ftrain {

// The supported graph and the indices its builder assigned: four matrix operands, two Tensor
// scalars, one operation node with inputs (a, b, c, alpha, beta) and output d
// (src/include/flash_train/operation/gemm.hpp:80-150 there).
struct GroupedGemmRoles {
    Pattern pattern;
    std::uint64_t a, b, c, d, alpha, beta, gemm;
};

// kOperation selects the storage family of each operand:
//   kGroupedABCDGemm  a, b, c, d GroupedTensors
//   kGroupedBCDGemm   a a TensorList; b, c, d GroupedTensors
//   kGroupedABGemm    a, b GroupedTensors; c, d TensorLists
template<OperationKind kOperation>
struct GroupedGemmFamilyOf {
    using Problem = GroupedGemmProblem;

    static const GroupedGemmRoles& getRoles();
    static Pattern makePattern() { return getRoles().pattern; }
    // Registration order = fallback preference: the exact-FP32, workspace-free Primitive first.
    static std::vector<std::shared_ptr<const Primitive<GroupedGemmProblem>>> makeRecords();
    static GroupedGemmProblem makeProblem(const Args& args);
};

using GroupedGemmFamily    = GroupedGemmFamilyOf<OperationKind::kGroupedABCDGemm>;
using GroupedBcdGemmFamily = GroupedGemmFamilyOf<OperationKind::kGroupedBCDGemm>;
using GroupedAbGemmFamily  = GroupedGemmFamilyOf<OperationKind::kGroupedABGemm>;

// The tensor-core Primitive first wherever it applies (it is one launch for all groups), the exact
// one behind it so that a caller without a workspace still finds a runnable index.
struct GroupedB200Heuristic final {
    static const char* getName() { return "GroupedB200Heuristic"; }
    static std::vector<std::string> findCandidates(const GroupedGemmProblem& problem, const Constraints& constraints);
};

}  // namespace ftrain

#endif
