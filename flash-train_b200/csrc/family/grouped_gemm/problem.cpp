#include "family/grouped_gemm/problem.hpp"

#include <cstring>
#include <limits>
#include <utility>

#include "core/error.hpp"

namespace ftrain {
namespace {

constexpr const char* kPortNames[4] = {"a", "b", "c", "d"};

// Entry `group` of a per-group metadata array in host memory.
std::int64_t readEntry(const StorageView& view, std::uint32_t group, const char* port, const char* what) {
    if (!view.isHostMemory()) {
        throw Exception(FTRAIN_STATUS_UNSUPPORTED, "GroupedGemm: %s of %s must be in host memory (the tile lists are built on the host)",
                        what, port);
    }
    if (view.getMemory() == nullptr) {
        throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "GroupedGemm: %s of %s has no memory", what, port);
    }
    const unsigned char* base = static_cast<const unsigned char*>(view.getMemory());
    switch (view.getNumericType()) {
        case FTRAIN_NUMERIC_TYPE_INT64: {
            std::int64_t value;
            std::memcpy(&value, base + 8 * static_cast<std::size_t>(group), sizeof value);
            return value;
        }
        case FTRAIN_NUMERIC_TYPE_UINT64: {
            std::uint64_t value;
            std::memcpy(&value, base + 8 * static_cast<std::size_t>(group), sizeof value);
            if (value > static_cast<std::uint64_t>(std::numeric_limits<std::int64_t>::max())) {
                throw Exception(FTRAIN_STATUS_OVERFLOW, "GroupedGemm: %s of %s does not fit 63 bits", what, port);
            }
            return static_cast<std::int64_t>(value);
        }
        case FTRAIN_NUMERIC_TYPE_INT32: {
            std::int32_t value;
            std::memcpy(&value, base + 4 * static_cast<std::size_t>(group), sizeof value);
            return value;
        }
        case FTRAIN_NUMERIC_TYPE_UINT32: {
            std::uint32_t value;
            std::memcpy(&value, base + 4 * static_cast<std::size_t>(group), sizeof value);
            return value;
        }
        default:
            throw Exception(FTRAIN_STATUS_UNSUPPORTED, "GroupedGemm: %s of %s must be an int64, uint64, int32 or uint32 array", what,
                            port);
    }
}

bool productOverflows(std::uint64_t x, std::uint64_t y) noexcept {
    return y != 0 && x > std::numeric_limits<std::uint64_t>::max() / sizeof(float) / y;
}

}  // namespace

GroupedGemmProblem::GroupedGemmProblem(GroupedTensor a, GroupedTensor b, GroupedTensor c, GroupedTensor d, Tensor alpha,
                                       Tensor beta, FTrainNumericType compute_type)
    : tensors_{std::move(a), std::move(b), std::move(c), std::move(d)}, alpha_(std::move(alpha)), beta_(std::move(beta)),
      compute_type_(compute_type), num_groups_(tensors_[0].getNumGroups()) {
    for (int port = 0; port < 4; ++port) {
        const GroupedTensor& tensor = tensors_[port];
        if (tensor.getData().getDims().size() != 2) {
            throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "GroupedGemm: a, b, c and d must be rank-two GroupedTensors");
        }
        if (tensor.getNumGroups() != num_groups_) {
            throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "GroupedGemm: %s has %u groups but a has %u", kPortNames[port],
                            static_cast<unsigned>(tensor.getNumGroups()), static_cast<unsigned>(num_groups_));
        }
    }
    if (!alpha_.getStorageView().getDims().empty() || !beta_.getStorageView().getDims().empty()) {
        throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "GroupedGemm: alpha and beta must be scalars (rank zero)");
    }
    for (int port = 0; port < 4; ++port) {
        if (tensors_[port].getData().isHostMemory()) {
            throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "GroupedGemm: the data of a, b, c and d must live in device memory");
        }
    }
    if (!alpha_.getStorageView().isHostMemory() || !beta_.getStorageView().isHostMemory()) {
        throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "GroupedGemm: alpha and beta must live in host memory");
    }

    // Decode the per-group metadata once; the kernels' tile lists and the key are made from it.
    for (int port = 0; port < 4; ++port) {
        const GroupedTensor& tensor = tensors_[port];
        if (tensor.getDimSizes().size() != 2) {
            throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "GroupedGemm: %s needs dim_sizes for both dimensions", kPortNames[port]);
        }
        const bool strided  = tensor.getStrides().size() == 2;
        const bool has_base = tensor.getOffsets().has_value();
        if (!has_base && tensor.getData().getIndexType() != FTRAIN_INDEX_TYPE_GROUPED_CONTINUOUS) {
            throw Exception(FTRAIN_STATUS_UNSUPPORTED,
                            "GroupedGemm: %s has no offsets and its data is not indexed GROUPED_CONTINUOUS", kPortNames[port]);
        }
        std::vector<GroupMatrix>& groups = groups_[port];
        groups.resize(num_groups_);
        std::int64_t running = 0;  // dense packing when no offsets are given
        for (std::uint32_t g = 0; g < num_groups_; ++g) {
            GroupMatrix& matrix = groups[g];
            matrix.rows         = readEntry(tensor.getDimSizes()[0], g, kPortNames[port], "dim_sizes[0]");
            matrix.cols         = readEntry(tensor.getDimSizes()[1], g, kPortNames[port], "dim_sizes[1]");
            if (matrix.rows < 0 || matrix.cols < 0) {
                throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "GroupedGemm: group %u of %s has a negative extent",
                                static_cast<unsigned>(g), kPortNames[port]);
            }
            if (productOverflows(static_cast<std::uint64_t>(matrix.rows), static_cast<std::uint64_t>(matrix.cols))) {
                throw Exception(FTRAIN_STATUS_OVERFLOW, "GroupedGemm: the byte size of group %u of %s does not fit 64 bits",
                                static_cast<unsigned>(g), kPortNames[port]);
            }
            matrix.row_stride = strided ? readEntry(tensor.getStrides()[0], g, kPortNames[port], "strides[0]") : matrix.cols;
            matrix.col_stride = strided ? readEntry(tensor.getStrides()[1], g, kPortNames[port], "strides[1]") : 1;
            matrix.offset     = has_base ? readEntry(*tensor.getOffsets(), g, kPortNames[port], "offsets") : running;
            if (matrix.offset < 0) {
                throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "GroupedGemm: group %u of %s has a negative offset",
                                static_cast<unsigned>(g), kPortNames[port]);
            }
            running += matrix.rows * matrix.cols;
        }
    }
    for (std::uint32_t g = 0; g < num_groups_; ++g) {
        const GroupMatrix& ga = groups_[0][g];
        const GroupMatrix& gb = groups_[1][g];
        if (ga.cols != gb.rows) {
            throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "GroupedGemm: in group %u a has %lld columns but b has %lld rows",
                            static_cast<unsigned>(g), static_cast<long long>(ga.cols), static_cast<long long>(gb.rows));
        }
        for (const int port : {2, 3}) {
            const GroupMatrix& out = groups_[port][g];
            if (out.rows != ga.rows || out.cols != gb.cols) {
                throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "GroupedGemm: in group %u %s must be %lld-by-%lld like the product of a and b",
                                static_cast<unsigned>(g), kPortNames[port], static_cast<long long>(ga.rows),
                                static_cast<long long>(gb.cols));
            }
        }
        output_elements_ += static_cast<std::uint64_t>(ga.rows) * static_cast<std::uint64_t>(gb.cols);
    }
}

bool GroupedGemmProblem::isInPlace() const noexcept {
    if (getData(GroupedPort::kC).getMemory() != getData(GroupedPort::kD).getMemory()) { return false; }
    for (std::uint32_t g = 0; g < num_groups_; ++g) {
        if (groups_[2][g].offset != groups_[3][g].offset) { return false; }
    }
    return true;
}

std::vector<std::uint64_t> GroupedGemmProblem::getProblemKey() const {
    std::vector<std::uint64_t> key;
    key.reserve(4 * (3 + 5 * static_cast<std::size_t>(num_groups_)) + 3);
    key.push_back(num_groups_);
    for (int port = 0; port < 4; ++port) {
        const StorageView& data = tensors_[port].getData();
        const void* memory      = data.getMemory();
        key.push_back(static_cast<std::uint64_t>(data.getNumericType()) | static_cast<std::uint64_t>(data.getIndexType()) << 8);
        key.push_back(memory != nullptr ? 1U : 0U);
        key.push_back(memory != nullptr ? reinterpret_cast<std::uintptr_t>(memory) & 15U : 0U);
        for (const GroupMatrix& matrix : groups_[port]) {
            for (const std::int64_t value : {matrix.offset, matrix.rows, matrix.cols, matrix.row_stride, matrix.col_stride}) {
                key.push_back(static_cast<std::uint64_t>(value));
            }
        }
    }
    for (const StorageView* scalar : {&alpha_.getStorageView(), &beta_.getStorageView()}) {
        key.push_back(static_cast<std::uint64_t>(scalar->getNumericType()) | static_cast<std::uint64_t>(scalar->getIndexType()) << 8 |
                      (scalar->getMemory() != nullptr ? 1ULL << 16 : 0ULL) |
                      (reinterpret_cast<std::uintptr_t>(scalar->getMemory()) & 3U) << 24);
    }
    key.push_back(static_cast<std::uint64_t>(compute_type_));
    key.push_back(isInPlace() ? 1U : 0U);
    return key;
}

}  // namespace ftrain
