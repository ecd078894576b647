// The one place that lists the engines this library ships
// (reference: src/engine.cpp:25-27).
#include <memory>
#include <vector>

#include "core/engine.hpp"
#include "family/gemm/family.hpp"
#include "family/gemm/finder.hpp"
#include "family/grouped_gemm/family.hpp"

namespace ftrain {

std::vector<std::shared_ptr<OpsEngineBase>> makeBuiltinOpsEngines() {
    // The reference registers the Gemm engine only; the GroupedABCDGemm engine is this build's addition
    // (its other two grouped operations, with TensorList operands, stay without one, as there).
    return {std::make_shared<OpsEngine<GemmFamily, B200Heuristic, RegistrationOrderFinder>>(),
            std::make_shared<OpsEngine<GroupedGemmFamily, GroupedB200Heuristic>>()};
}

}  // namespace ftrain
