// Validated, metadata-owning copy of an FTrainStorageView.
//
// Validation rules are the reference's (src/storage_view.cpp:9-52, pinned by
// tests/storage_view_test.cpp:30-251): real numeric type, known index type,
// scalar needs memory, dims present and non-negative, and exactly one layout
// source (strides <=> index_type INVALID). Stride values are not validated.
//
// Unlike the reference's std::vector members, extents live in an inline buffer
// for rank <= 4, so copying a matrix or scalar view never touches the heap:
// the one-shot ftrainGemm path builds six of these per call.
#ifndef FTRAIN_CORE_STORAGE_VIEW_HPP_
#define FTRAIN_CORE_STORAGE_VIEW_HPP_

#include <cstddef>
#include <cstdint>
#include <memory>

#include "flash_train/common.h"

namespace ftrain {

// A fixed-length int64 sequence with small-size inline storage.
class Extents final {
  public:
    Extents() noexcept = default;
    Extents(const std::int64_t* values, std::size_t count);
    Extents(const Extents& other);
    Extents& operator=(const Extents& other);
    Extents(Extents&& other) noexcept;
    Extents& operator=(Extents&& other) noexcept;

    std::size_t size() const noexcept { return size_; }
    bool empty() const noexcept { return size_ == 0; }
    const std::int64_t* data() const noexcept { return heap_ ? heap_.get() : inline_; }
    const std::int64_t* begin() const noexcept { return data(); }
    const std::int64_t* end() const noexcept { return data() + size_; }
    std::int64_t operator[](std::size_t index) const noexcept { return data()[index]; }

    bool operator==(const Extents& other) const noexcept;
    bool operator!=(const Extents& other) const noexcept { return !(*this == other); }

  private:
    static constexpr std::size_t kInline = 4;
    std::size_t size_{0};
    std::int64_t inline_[kInline]{};
    std::unique_ptr<std::int64_t[]> heap_;
};

class StorageView final {
  public:
    // Throws Exception(FTRAIN_STATUS_INVALID_ARGUMENT) on a rule violation.
    explicit StorageView(const FTrainStorageView& view);

    void* getMemory() const noexcept { return memory_; }
    const Extents& getDims() const noexcept { return dims_; }
    // Empty unless the view's layout comes from strides (index type INVALID).
    const Extents& getStrides() const noexcept { return strides_; }
    FTrainNumericType getNumericType() const noexcept { return numeric_type_; }
    FTrainIndexType getIndexType() const noexcept { return index_type_; }
    bool isHostMemory() const noexcept { return is_host_memory_; }

  private:
    void* memory_;
    Extents dims_;
    Extents strides_;
    FTrainNumericType numeric_type_;
    FTrainIndexType index_type_;
    bool is_host_memory_;
};

}  // namespace ftrain

#endif
