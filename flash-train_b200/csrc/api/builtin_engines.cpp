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
    // The reference registers the Gemm engine only; the three grouped-GEMM engines are this build's addition
    // (its public API declares the operations, include/flash_train/common.h:248-306 there).
    return {std::make_shared<OpsEngine<GemmFamily, B200Heuristic, RegistrationOrderFinder>>(),
            std::make_shared<OpsEngine<GroupedGemmFamily, GroupedB200Heuristic>>(),
            std::make_shared<OpsEngine<GroupedBcdGemmFamily, GroupedB200Heuristic>>(),
            std::make_shared<OpsEngine<GroupedAbGemmFamily, GroupedB200Heuristic>>()};
}

}  // namespace ftrain
