// Selection policies of the Gemm family.
//
// The reference ships only a placeholder that names nothing
// (src/include/flash_train/family/gemm/finder.hpp:21-25), which makes its engine
// fall back to registration order. B200Heuristic is the real policy of this
// build: it ranks the CUDA Primitives by problem regime (see finder.cpp).
#ifndef FTRAIN_FAMILY_GEMM_FINDER_HPP_
#define FTRAIN_FAMILY_GEMM_FINDER_HPP_

#include <string>
#include <vector>

#include "core/constraints.hpp"
#include "family/gemm/problem.hpp"

namespace ftrain {

struct B200Heuristic final {
    static const char* getName() { return "B200Heuristic"; }
    // Primitive names, best first. The engine keeps the applicable ones.
    static std::vector<std::string> findCandidates(const GemmProblem& problem, const Constraints& constraints);
};

// Kept so that FTRAIN_DISABLED_FINDERS=B200Heuristic reproduces the
// reference's behaviour: no opinion, registration order decides.
struct RegistrationOrderFinder final {
    static const char* getName() { return "RegistrationOrder"; }
    static std::vector<std::string> findCandidates(const GemmProblem&, const Constraints&) { return {}; }
};

}  // namespace ftrain

#endif
