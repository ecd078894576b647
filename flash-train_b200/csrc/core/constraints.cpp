#include "core/constraints.hpp"

#include "core/error.hpp"
#include "ftcuda/ftcuda.h"

namespace ftrain {

FTrainDeviceId getCurrentDeviceId() {
    std::int32_t device = 0;
    char reason[160];
    if (ftcuda_current_device(&device, reason, sizeof reason) != 0) {
        throw Exception(FTRAIN_STATUS_INTERNAL_ERROR, "cudaGetDevice failed: %s", reason);
    }
    return device;
}

}  // namespace ftrain
