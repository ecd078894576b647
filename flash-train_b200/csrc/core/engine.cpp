#include "core/engine.hpp"

#include <utility>

namespace ftrain {

OpsEngineBase::OpsEngineBase(Pattern pattern) : pattern_(std::move(pattern)) {}

OpsEngineBase::~OpsEngineBase() = default;

Plan OpsEngineBase::createPlan(const Args& args) const {
    const FTrainDeviceId device = getCurrentDeviceId();
    return Plan(createPrimitives(args, Constraints{device}), device);
}

}  // namespace ftrain
