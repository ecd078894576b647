#include "core/primitive.hpp"

namespace ftrain {

PrimitiveBase::~PrimitiveBase() = default;

void PrimitiveBase::execute(const Resources& resources) {
    const std::uint64_t required = getRequiredWorkspaceBytes();
    if (resources.getWorkspaceBytes() < required) {
        throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "the workspace holds %llu bytes; this Primitive needs %llu",
                        static_cast<unsigned long long>(resources.getWorkspaceBytes()),
                        static_cast<unsigned long long>(required));
    }
    if (required != 0 && resources.getWorkspace() == nullptr) {
        throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "this Primitive needs a workspace of %llu bytes, got a null pointer",
                        static_cast<unsigned long long>(required));
    }
    executeImpl(resources);
}

}  // namespace ftrain
