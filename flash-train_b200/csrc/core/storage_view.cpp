#include "core/storage_view.hpp"

#include <algorithm>
#include <utility>

#include "core/error.hpp"

namespace ftrain {

Extents::Extents(const std::int64_t* values, std::size_t count) : size_(count) {
    std::int64_t* target = inline_;
    if (count > kInline) {
        heap_  = std::make_unique<std::int64_t[]>(count);
        target = heap_.get();
    }
    std::copy(values, values + count, target);
}

Extents::Extents(const Extents& other) : Extents(other.data(), other.size_) {}

Extents& Extents::operator=(const Extents& other) {
    if (this != &other) {
        Extents copy(other);
        *this = std::move(copy);
    }
    return *this;
}

Extents::Extents(Extents&& other) noexcept : size_(other.size_), heap_(std::move(other.heap_)) {
    std::copy(other.inline_, other.inline_ + kInline, inline_);
    other.size_ = 0;
}

Extents& Extents::operator=(Extents&& other) noexcept {
    if (this != &other) {
        size_ = other.size_;
        heap_ = std::move(other.heap_);
        std::copy(other.inline_, other.inline_ + kInline, inline_);
        other.size_ = 0;
    }
    return *this;
}

bool Extents::operator==(const Extents& other) const noexcept {
    return size_ == other.size_ && std::equal(begin(), end(), other.begin());
}

StorageView::StorageView(const FTrainStorageView& view)
    : memory_(view.memory), numeric_type_(view.numeric_type), index_type_(view.index_type),
      is_host_memory_(view.is_host_memory) {
    const std::size_t rank = view.num_dims;
    if (numeric_type_ == FTRAIN_NUMERIC_TYPE_INVALID || numeric_type_ >= FTRAIN_NUMERIC_TYPE_COUNT) {
        throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "StorageView numeric_type %u is invalid",
                        static_cast<unsigned>(numeric_type_));
    }
    if (index_type_ >= FTRAIN_INDEX_TYPE_COUNT) {
        throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "StorageView index_type %u is unknown",
                        static_cast<unsigned>(index_type_));
    }
    if (rank == 0 && view.memory == nullptr) {
        throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "StorageView memory must not be null for a scalar");
    }
    if (rank != 0 && view.dims == nullptr) {
        throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "StorageView dims must not be null when num_dims is %zu", rank);
    }
    const bool strided = index_type_ == FTRAIN_INDEX_TYPE_INVALID;
    if (strided && view.strides == nullptr) {
        throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "StorageView requires strides or a non-invalid index_type");
    }
    if (!strided && view.strides != nullptr) {
        throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT,
                        "StorageView strides must be null when index_type %u defines a predefined layout",
                        static_cast<unsigned>(index_type_));
    }
    for (std::size_t axis = 0; axis < rank; ++axis) {
        if (view.dims[axis] < 0) {
            throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "StorageView dimension %zu must be non-negative, got %lld",
                            axis, static_cast<long long>(view.dims[axis]));
        }
    }
    if (rank == 0) { return; }
    dims_ = Extents(view.dims, rank);
    if (strided) { strides_ = Extents(view.strides, rank); }
}

}  // namespace ftrain
