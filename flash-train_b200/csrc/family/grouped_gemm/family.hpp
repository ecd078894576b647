// What the GroupedABCDGemm family hands to its engine: supported Pattern, Primitive catalogue,
// Problem factory. The operation exists in the reference's public API without an engine
// (include/flash_train/common.h:248-266, src/engine.cpp:25-27 there); here it has one.
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

struct GroupedGemmFamily {
    using Problem = GroupedGemmProblem;

    // Four GroupedTensor operands, two Tensor scalars, one GroupedABCDGemm node with inputs
    // (a, b, c, alpha, beta) and output d (src/include/flash_train/operation/gemm.hpp:80-104 there).
    struct Roles {
        Pattern pattern;
        std::uint64_t a, b, c, d, alpha, beta, gemm;
    };
    static const Roles& getRoles();
    static Pattern makePattern() { return getRoles().pattern; }

    // Registration order = fallback preference: the exact-FP32, workspace-free Primitive first.
    static std::vector<std::shared_ptr<const Primitive<GroupedGemmProblem>>> makeRecords();
    static GroupedGemmProblem makeProblem(const Args& args);
};

// The tensor-core Primitive first wherever it applies (it is one launch for all groups), the exact
// one behind it so that a caller without a workspace still finds a runnable index.
struct GroupedB200Heuristic final {
    static const char* getName() { return "GroupedB200Heuristic"; }
    static std::vector<std::string> findCandidates(const GroupedGemmProblem& problem, const Constraints& constraints);
};

}  // namespace ftrain

#endif
