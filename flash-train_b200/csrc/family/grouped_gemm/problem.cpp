#include "family/grouped_gemm/problem.hpp"

#include <cstring>
#include <limits>
#include <utility>
#include <variant>

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

bool floatAligned(const void* address) noexcept { return reinterpret_cast<std::uintptr_t>(address) % alignof(float) == 0; }

void checkExtents(const GroupMatrix& matrix, std::uint32_t group, const char* port) {
    if (matrix.rows < 0 || matrix.cols < 0) {
        throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "GroupedGemm: group %u of %s has a negative extent", static_cast<unsigned>(group), port);
    }
    if (productOverflows(static_cast<std::uint64_t>(matrix.rows), static_cast<std::uint64_t>(matrix.cols))) {
        throw Exception(FTRAIN_STATUS_OVERFLOW, "GroupedGemm: the byte size of group %u of %s does not fit 64 bits",
                        static_cast<unsigned>(group), port);
    }
}

GroupedOperand decodeGrouped(const GroupedTensor& tensor, const char* port) {
    GroupedOperand operand;
    const StorageView& data = tensor.getData();
    if (data.getDims().size() != 2) {
        throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "GroupedGemm: a, b, c and d must be rank two (%s is not)", port);
    }
    if (tensor.getDimSizes().size() != 2) {
        throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "GroupedGemm: %s needs dim_sizes for both dimensions", port);
    }
    const bool strided  = tensor.getStrides().size() == 2;
    const bool has_base = tensor.getOffsets().has_value();
    if (!has_base && data.getIndexType() != FTRAIN_INDEX_TYPE_GROUPED_CONTINUOUS) {
        throw Exception(FTRAIN_STATUS_UNSUPPORTED, "GroupedGemm: %s has no offsets and its data is not indexed GROUPED_CONTINUOUS", port);
    }
    operand.is_list          = false;
    operand.numeric_type     = data.getNumericType();
    operand.plainly_indexed  = data.getIndexType() == FTRAIN_INDEX_TYPE_GROUPED_CONTINUOUS || data.getIndexType() == FTRAIN_INDEX_TYPE_CONTINUOUS;
    operand.in_device_memory = !data.isHostMemory();
    operand.any_memory       = data.getMemory() != nullptr;
    operand.all_memory       = data.getMemory() != nullptr;
    operand.float_aligned    = floatAligned(data.getMemory());
    operand.groups.resize(tensor.getNumGroups());
    std::int64_t running = 0;  // dense packing when no offsets are given
    for (std::uint32_t g = 0; g < tensor.getNumGroups(); ++g) {
        GroupMatrix& matrix = operand.groups[g];
        matrix.base         = data.getMemory();
        matrix.rows         = readEntry(tensor.getDimSizes()[0], g, port, "dim_sizes[0]");
        matrix.cols         = readEntry(tensor.getDimSizes()[1], g, port, "dim_sizes[1]");
        checkExtents(matrix, g, port);
        matrix.row_stride = strided ? readEntry(tensor.getStrides()[0], g, port, "strides[0]") : matrix.cols;
        matrix.col_stride = strided ? readEntry(tensor.getStrides()[1], g, port, "strides[1]") : 1;
        matrix.offset     = has_base ? readEntry(*tensor.getOffsets(), g, port, "offsets") : running;
        if (matrix.offset < 0) {
            throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "GroupedGemm: group %u of %s has a negative offset", static_cast<unsigned>(g), port);
        }
        running += matrix.rows * matrix.cols;
    }
    return operand;
}

GroupedOperand decodeList(const TensorList& list, const char* port) {
    GroupedOperand operand;
    const std::vector<StorageView>& views = list.getStorageViews();
    operand.is_list    = true;
    operand.all_memory = true;
    operand.groups.resize(views.size());
    for (std::size_t g = 0; g < views.size(); ++g) {
        const StorageView& view = views[g];
        if (view.getDims().size() != 2) {
            throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "GroupedGemm: a, b, c and d must be rank two (entry %zu of %s is not)", g, port);
        }
        GroupMatrix& matrix = operand.groups[g];
        matrix.base         = view.getMemory();
        matrix.offset       = 0;
        matrix.rows         = view.getDims()[0];
        matrix.cols         = view.getDims()[1];
        checkExtents(matrix, static_cast<std::uint32_t>(g), port);
        const bool strided = view.getIndexType() == FTRAIN_INDEX_TYPE_INVALID && view.getStrides().size() == 2;
        matrix.row_stride  = strided ? view.getStrides()[0] : matrix.cols;
        matrix.col_stride  = strided ? view.getStrides()[1] : 1;
        if (g == 0) {
            operand.numeric_type = view.getNumericType();
        } else if (operand.numeric_type != view.getNumericType()) {
            operand.numeric_type = FTRAIN_NUMERIC_TYPE_INVALID;
        }
        operand.plainly_indexed  = operand.plainly_indexed && (strided || view.getIndexType() == FTRAIN_INDEX_TYPE_CONTINUOUS);
        operand.in_device_memory = operand.in_device_memory && !view.isHostMemory();
        operand.any_memory       = operand.any_memory || view.getMemory() != nullptr;
        operand.all_memory       = operand.all_memory && (view.getMemory() != nullptr || matrix.rows * matrix.cols == 0);
        operand.float_aligned    = operand.float_aligned && floatAligned(view.getMemory());
    }
    if (views.empty()) { operand.numeric_type = FTRAIN_NUMERIC_TYPE_FP32; }  // nothing to disagree with
    return operand;
}

GroupedOperand decode(const OperandValue& value, const char* port) {
    if (const GroupedTensor* grouped = std::get_if<GroupedTensor>(&value)) { return decodeGrouped(*grouped, port); }
    if (const TensorList* list = std::get_if<TensorList>(&value)) { return decodeList(*list, port); }
    throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "GroupedGemm: %s must be a GroupedTensor or a TensorList", port);
}

}  // namespace

GroupedGemmProblem::GroupedGemmProblem(const OperandValue& a, const OperandValue& b, const OperandValue& c, const OperandValue& d,
                                       Tensor alpha, Tensor beta, FTrainNumericType compute_type)
    : operands_{decode(a, "a"), decode(b, "b"), decode(c, "c"), decode(d, "d")}, alpha_(std::move(alpha)), beta_(std::move(beta)),
      compute_type_(compute_type) {
    num_groups_ = static_cast<std::uint32_t>(operands_[0].groups.size());
    for (int port = 1; port < 4; ++port) {
        if (operands_[port].groups.size() != num_groups_) {
            throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "GroupedGemm: %s has %zu groups but a has %u", kPortNames[port],
                            operands_[port].groups.size(), static_cast<unsigned>(num_groups_));
        }
    }
    if (!alpha_.getStorageView().getDims().empty() || !beta_.getStorageView().getDims().empty()) {
        throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "GroupedGemm: alpha and beta must be scalars (rank zero)");
    }
    for (int port = 0; port < 4; ++port) {
        if (!operands_[port].in_device_memory) {
            throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "GroupedGemm: the data of a, b, c and d must live in device memory");
        }
    }
    if (!alpha_.getStorageView().isHostMemory() || !beta_.getStorageView().isHostMemory()) {
        throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "GroupedGemm: alpha and beta must live in host memory");
    }
    for (std::uint32_t g = 0; g < num_groups_; ++g) {
        const GroupMatrix& ga = operands_[0].groups[g];
        const GroupMatrix& gb = operands_[1].groups[g];
        if (ga.cols != gb.rows) {
            throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "GroupedGemm: in group %u a has %lld columns but b has %lld rows",
                            static_cast<unsigned>(g), static_cast<long long>(ga.cols), static_cast<long long>(gb.rows));
        }
        for (const int port : {2, 3}) {
            const GroupMatrix& out = operands_[port].groups[g];
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
    for (std::uint32_t g = 0; g < num_groups_; ++g) {
        if (operands_[2].groups[g].address() != operands_[3].groups[g].address()) { return false; }
    }
    return true;
}

std::vector<std::uint64_t> GroupedGemmProblem::getProblemKey() const {
    std::vector<std::uint64_t> key;
    key.reserve(4 * (2 + 6 * static_cast<std::size_t>(num_groups_)) + 5);
    key.push_back(num_groups_);
    for (const GroupedOperand& operand : operands_) {
        key.push_back((operand.is_list ? 1U : 0U) | static_cast<std::uint64_t>(operand.numeric_type) << 8 |
                      (operand.plainly_indexed ? 1ULL << 16 : 0ULL) | (operand.float_aligned ? 1ULL << 17 : 0ULL));
        for (const GroupMatrix& matrix : operand.groups) {
            const float* address = matrix.address();
            key.push_back(address != nullptr ? 1U + ((reinterpret_cast<std::uintptr_t>(address) & 15U) << 1) : 0U);
            for (const std::int64_t value : {matrix.rows, matrix.cols, matrix.row_stride, matrix.col_stride}) {
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
