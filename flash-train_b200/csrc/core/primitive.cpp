#include "core/primitive.hpp"

namespace ftrain {

PrimitiveBase::~PrimitiveBase() = default;

void PrimitiveBase::execute(const Resources& resources) {
    const std::uint64_t required = getRequiredWorkspaceBytes();
    if (resources.getWorkspaceBytes() < required) {
        throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "Primitive requires %llu workspace bytes but received %llu",
                        static_cast<unsigned long long>(required),
                        static_cast<unsigned long long>(resources.getWorkspaceBytes()));
    }
    if (required != 0 && resources.getWorkspace() == nullptr) {
        throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "Primitive requires a non-null workspace for %llu bytes",
                        static_cast<unsigned long long>(required));
    }
    executeImpl(resources);
}

}  // namespace ftrain
