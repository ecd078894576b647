// What the Gemm family hands to its engine: supported Pattern, Primitive
// catalogue, Problem factory. Reference: src/include/flash_train/family/gemm/family.hpp:20-72,
// src/family/gemm/family.cpp:13-15.
#ifndef FTRAIN_FAMILY_GEMM_FAMILY_HPP_
#define FTRAIN_FAMILY_GEMM_FAMILY_HPP_

#include <memory>
#include <vector>

#include "core/ops_args.hpp"
#include "core/pattern.hpp"
#include "core/primitive.hpp"
#include "family/gemm/problem.hpp"

namespace ftrain {

struct GemmFamily {
    using Problem = GemmProblem;

    // The supported graph and the indices its builder assigned: six Tensor
    // operands and one Gemm node with inputs (a, b, c, alpha, beta), output d.
    struct Roles {
        Pattern pattern;
        std::uint64_t a, b, c, d, alpha, beta, gemm;
    };
    static const Roles& getRoles();

    static Pattern makePattern() { return getRoles().pattern; }

    // Registration order = fallback preference when no Finder contributes:
    // the exact-FP32, workspace-free kernel comes first.
    static std::vector<std::shared_ptr<const Primitive<GemmProblem>>> makeRecords();

    static GemmProblem makeProblem(const Args& args);
};

}  // namespace ftrain

#endif
