#include "core/tensor.hpp"

#include <cstdio>

#include "core/error.hpp"

namespace ftrain {
namespace {

// A per-group metadata array must be rank one with one entry per group.
void requireGroupVector(const StorageView& view, std::uint32_t num_groups, const char* what, long index) {
    const Extents& dims = view.getDims();
    char label[48];
    if (index < 0) {
        std::snprintf(label, sizeof label, "%s", what);
    } else {
        std::snprintf(label, sizeof label, "%s[%ld]", what, index);
    }
    if (dims.size() != 1) {
        throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "GroupedTensor %s rank %zu must be 1", label, dims.size());
    }
    if (dims[0] != static_cast<std::int64_t>(num_groups)) {
        throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "GroupedTensor %s length %lld must match num_groups %u", label,
                        static_cast<long long>(dims[0]), static_cast<unsigned>(num_groups));
    }
}

}  // namespace

GroupedTensor::GroupedTensor(std::uint32_t num_groups, StorageView&& data, std::optional<StorageView>&& offsets,
                             std::vector<StorageView>&& dim_sizes, std::vector<StorageView>&& strides)
    : num_groups_(num_groups), data_(std::move(data)), offsets_(std::move(offsets)), dim_sizes_(std::move(dim_sizes)),
      strides_(std::move(strides)) {
    const std::size_t rank = data_.getDims().size();
    if (!dim_sizes_.empty() && dim_sizes_.size() != rank) {
        throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT,
                        "GroupedTensor dim_sizes count %zu must be zero or match data rank %zu", dim_sizes_.size(), rank);
    }
    if (!strides_.empty() && strides_.size() != rank) {
        throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT,
                        "GroupedTensor strides count %zu must be zero or match data rank %zu", strides_.size(), rank);
    }
    if (offsets_.has_value()) { requireGroupVector(*offsets_, num_groups_, "offsets", -1); }
    for (std::size_t axis = 0; axis < dim_sizes_.size(); ++axis) {
        requireGroupVector(dim_sizes_[axis], num_groups_, "dim_sizes", static_cast<long>(axis));
    }
    for (std::size_t axis = 0; axis < strides_.size(); ++axis) {
        requireGroupVector(strides_[axis], num_groups_, "strides", static_cast<long>(axis));
    }
}

}  // namespace ftrain
