// Runtime constraints of one selection: the device it runs on.
// Reference: src/include/flash_train/constraints.hpp:19-36, src/constraints.cpp:15-26.
#ifndef FTRAIN_CORE_CONSTRAINTS_HPP_
#define FTRAIN_CORE_CONSTRAINTS_HPP_

#include <cstdint>
#include <vector>

#include "flash_train/common.h"

namespace ftrain {

// The calling thread's current CUDA device, asked of the platform layer
// (ftcuda_current_device). A runtime failure throws
// Exception(FTRAIN_STATUS_INTERNAL_ERROR).
FTrainDeviceId getCurrentDeviceId();

class Constraints final {
  public:
    explicit Constraints(FTrainDeviceId device_id) noexcept : device_id_(device_id) {}
    FTrainDeviceId getDeviceId() const noexcept { return device_id_; }
    // Everything here that can change a selection must appear in these tokens:
    // a cache hit bypasses the Finders and the applicability checks.
    std::vector<std::uint64_t> getConstraintsKey() const {
        return {static_cast<std::uint64_t>(static_cast<std::uint32_t>(device_id_))};
    }

  private:
    FTrainDeviceId device_id_;
};

}  // namespace ftrain

#endif
