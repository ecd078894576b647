// Argument value types for the three operand storage families.
//
// Tensor = one view; TensorList = ordered views; GroupedTensor = data view plus
// optional per-group offsets / dimension sizes / strides. Shape rules for
// GroupedTensor follow the reference (src/tensor.cpp:9-62). Only Tensor is used
// by a registered engine; the other two exist so the Args setters of the public
// API behave as in the reference.
#ifndef FTRAIN_CORE_TENSOR_HPP_
#define FTRAIN_CORE_TENSOR_HPP_

#include <cstdint>
#include <optional>
#include <utility>
#include <vector>

#include "core/storage_view.hpp"

namespace ftrain {

class Tensor final {
  public:
    explicit Tensor(StorageView&& view) noexcept : view_(std::move(view)) {}
    const StorageView& getStorageView() const noexcept { return view_; }

  private:
    StorageView view_;
};

class TensorList final {
  public:
    explicit TensorList(std::vector<StorageView>&& views) noexcept : views_(std::move(views)) {}
    const std::vector<StorageView>& getStorageViews() const noexcept { return views_; }

  private:
    std::vector<StorageView> views_;
};

class GroupedTensor final {
  public:
    // dim_sizes / strides: empty, or one rank-1 view of num_groups entries per
    // data dimension. offsets: absent, or a rank-1 view of num_groups entries.
    // Throws Exception(FTRAIN_STATUS_INVALID_ARGUMENT) otherwise.
    GroupedTensor(std::uint32_t num_groups, StorageView&& data, std::optional<StorageView>&& offsets,
                  std::vector<StorageView>&& dim_sizes, std::vector<StorageView>&& strides);

    std::uint32_t getNumGroups() const noexcept { return num_groups_; }
    const StorageView& getData() const noexcept { return data_; }
    const std::optional<StorageView>& getOffsets() const noexcept { return offsets_; }
    const std::vector<StorageView>& getDimSizes() const noexcept { return dim_sizes_; }
    const std::vector<StorageView>& getStrides() const noexcept { return strides_; }

  private:
    std::uint32_t num_groups_;
    StorageView data_;
    std::optional<StorageView> offsets_;
    std::vector<StorageView> dim_sizes_;
    std::vector<StorageView> strides_;
};

}  // namespace ftrain

#endif
