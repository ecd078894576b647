#include "core/plan.hpp"

#include <utility>

namespace ftrain {

Plan::Plan(std::vector<std::unique_ptr<PrimitiveBase>>&& primitives, FTrainDeviceId device_id)
    : device_id_(device_id), primitives_(std::move(primitives)) {
    if (primitives_.empty()) { throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "Plan requires at least one Primitive"); }
    for (const auto& primitive : primitives_) {
        if (primitive == nullptr) { throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "Plan Primitive must not be null"); }
    }
}

PrimitiveBase& Plan::at(std::uint64_t index) const {
    if (index >= primitives_.size()) {
        throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "Plan primitive index %llu is out of range for %llu primitives",
                        static_cast<unsigned long long>(index), static_cast<unsigned long long>(primitives_.size()));
    }
    return *primitives_[index];
}

const char* Plan::getPrimitiveName(std::uint64_t index) const { return at(index).getName(); }

std::uint64_t Plan::getPrimitiveRequiredWorkspaceBytes(std::uint64_t index) const {
    return at(index).getRequiredWorkspaceBytes();
}

void Plan::execute(std::uint64_t index, void* workspace, std::uint64_t workspace_bytes, FTrainStream stream) {
    const FTrainDeviceId current = getCurrentDeviceId();
    if (current != device_id_) {
        throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT,
                        "Plan was created for device %d but the calling thread uses device %d",
                        static_cast<int>(device_id_), static_cast<int>(current));
    }
    at(index).execute(Resources{workspace, workspace_bytes, stream});
}

}  // namespace ftrain
