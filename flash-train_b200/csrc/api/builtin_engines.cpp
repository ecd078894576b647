// The one place that lists the engines this library ships
// (reference: src/engine.cpp:25-27).
#include <memory>
#include <vector>

#include "core/engine.hpp"
#include "family/gemm/family.hpp"
#include "family/gemm/finder.hpp"

namespace ftrain {

std::vector<std::shared_ptr<OpsEngineBase>> makeBuiltinOpsEngines() {
    return {std::make_shared<OpsEngine<GemmFamily, B200Heuristic, RegistrationOrderFinder>>()};
}

}  // namespace ftrain
