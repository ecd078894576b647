#include "api/api_support.hpp"

namespace ftrain {
namespace {

Result& lastResult() noexcept {
    static thread_local Result slot;
    return slot;
}

}  // namespace

const Result& getLastResult() noexcept { return lastResult(); }
void clearLastResult() noexcept { lastResult().clear(); }
void setLastResult(FTrainStatus status, const char* message) noexcept { lastResult().set(status, message); }

void requireNonNull(const void* pointer, const char* function, const char* what) {
    if (pointer == nullptr) { throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "%s: %s must not be null", function, what); }
}

}  // namespace ftrain

extern "C" FTrainStatus ftrainGetLastStatus(void) { return ftrain::getLastResult().getStatus(); }

extern "C" const char* ftrainGetLastMessage(void) { return ftrain::getLastResult().getMessage(); }
