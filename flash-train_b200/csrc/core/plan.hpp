// Plan: the configured Primitives selected for one call, best first, bound to
// the device they were configured on.
// Reference: src/include/flash_train/plan.hpp:21-57, src/plan.cpp:12-55.
#ifndef FTRAIN_CORE_PLAN_HPP_
#define FTRAIN_CORE_PLAN_HPP_

#include <cstdint>
#include <memory>
#include <vector>

#include "core/primitive.hpp"

namespace ftrain {

class Plan final {
  public:
    // An empty list or a null entry throws Exception(FTRAIN_STATUS_INVALID_ARGUMENT).
    Plan(std::vector<std::unique_ptr<PrimitiveBase>>&& primitives, FTrainDeviceId device_id);

    std::uint64_t getNumPrimitives() const noexcept { return primitives_.size(); }
    // An index out of range throws Exception(FTRAIN_STATUS_INVALID_ARGUMENT).
    const char* getPrimitiveName(std::uint64_t index) const;
    std::uint64_t getPrimitiveRequiredWorkspaceBytes(std::uint64_t index) const;

    // The hot call of a training loop: checks, in this order, that the calling
    // thread is on the Plan's device and that the index exists (each failing
    // with FTRAIN_STATUS_INVALID_ARGUMENT before anything is dispatched), then
    // hands the caller's workspace and stream to that one Primitive.
    void execute(std::uint64_t index, void* workspace, std::uint64_t workspace_bytes, FTrainStream stream);

  private:
    PrimitiveBase& at(std::uint64_t index) const;

    FTrainDeviceId device_id_;
    std::vector<std::unique_ptr<PrimitiveBase>> primitives_;
};

}  // namespace ftrain

#endif
