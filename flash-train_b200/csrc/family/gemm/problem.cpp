#include "family/gemm/problem.hpp"

#include <limits>
#include <utility>

#include "core/error.hpp"

namespace ftrain {
namespace {

constexpr GemmPort kMatrices[] = {GemmPort::kA, GemmPort::kB, GemmPort::kC, GemmPort::kD};
constexpr GemmPort kScalars[]  = {GemmPort::kAlpha, GemmPort::kBeta};

// Token layout of one view inside the problem key: a fixed head of four words
// followed by the extents and (for strided views) the strides.
//   word 0  numeric type | index type << 8 | rank << 16 | stride count << 24
//   word 1  1 when the view has memory, else 0
//   word 2  address modulo 16 (0 without memory)
//   word 3  number of words that follow (extents + strides)
// The head carries both lengths, so two keys can only be equal when every
// view has the same rank and stride count and the same values in them.
constexpr std::size_t kHeadWords = 4;
constexpr std::size_t kKeyWords  = 6 * (kHeadWords + 4) + 2;  // six views of rank <= 2, compute type, aliasing

void appendView(std::vector<std::uint64_t>& key, const StorageView& view) {
    const auto& dims    = view.getDims();
    const auto& strides = view.getStrides();
    const void* memory  = view.getMemory();
    key.push_back(static_cast<std::uint64_t>(view.getNumericType()) | static_cast<std::uint64_t>(view.getIndexType()) << 8 |
                  static_cast<std::uint64_t>(dims.size()) << 16 | static_cast<std::uint64_t>(strides.size()) << 24);
    key.push_back(memory != nullptr ? 1U : 0U);
    key.push_back(memory != nullptr ? reinterpret_cast<std::uintptr_t>(memory) & 15U : 0U);
    key.push_back(dims.size() + strides.size());
    for (const std::int64_t extent : dims) { key.push_back(static_cast<std::uint64_t>(extent)); }
    for (const std::int64_t stride : strides) { key.push_back(static_cast<std::uint64_t>(stride)); }
}

// x * y * sizeof(float) does not fit 64 bits.
bool byteCountOverflows(std::uint64_t x, std::uint64_t y) noexcept {
    return y != 0 && x > std::numeric_limits<std::uint64_t>::max() / sizeof(float) / y;
}

}  // namespace

// The checks come in the reference's order (src/family/gemm/problem.cpp:13-56 there): which status
// a doubly wrong call gets depends on it. Rank, then placement, then shapes, then size.
GemmProblem::GemmProblem(Tensor a, Tensor b, Tensor c, Tensor d, Tensor alpha, Tensor beta,
                         FTrainNumericType compute_type)
    : ports_{std::move(a), std::move(b), std::move(c), std::move(d), std::move(alpha), std::move(beta)},
      compute_type_(compute_type) {
    for (const GemmPort port : kMatrices) {
        if (getView(port).getDims().size() != 2) {
            throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "Gemm: a, b, c and d must be matrices (rank two)");
        }
    }
    for (const GemmPort port : kScalars) {
        if (!getView(port).getDims().empty()) {
            throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "Gemm: alpha and beta must be scalars (rank zero)");
        }
    }
    for (const GemmPort port : kMatrices) {
        if (getView(port).isHostMemory()) {
            throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "Gemm: a, b, c and d must live in device memory");
        }
    }
    for (const GemmPort port : kScalars) {
        if (!getView(port).isHostMemory()) {
            throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "Gemm: alpha and beta must live in host memory");
        }
    }

    const auto& a_dims = getView(GemmPort::kA).getDims();
    const auto& b_dims = getView(GemmPort::kB).getDims();
    shape_.m           = static_cast<std::uint64_t>(a_dims[0]);
    shape_.k           = static_cast<std::uint64_t>(a_dims[1]);
    shape_.n           = static_cast<std::uint64_t>(b_dims[1]);
    if (a_dims[1] != b_dims[0]) {
        throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "Gemm: a has %lld columns but b has %lld rows",
                        static_cast<long long>(a_dims[1]), static_cast<long long>(b_dims[0]));
    }
    for (const GemmPort port : {GemmPort::kC, GemmPort::kD}) {
        const auto& dims = getView(port).getDims();
        if (dims[0] != a_dims[0] || dims[1] != b_dims[1]) {
            throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "Gemm: c and d must be %lld-by-%lld like the product of a and b",
                            static_cast<long long>(a_dims[0]), static_cast<long long>(b_dims[1]));
        }
    }
    if (byteCountOverflows(shape_.m, shape_.k) || byteCountOverflows(shape_.k, shape_.n) ||
        byteCountOverflows(shape_.m, shape_.n)) {
        throw Exception(FTRAIN_STATUS_OVERFLOW, "Gemm: the byte size of a matrix does not fit 64 bits");
    }
}

MatrixLayout GemmProblem::getLayout(GemmPort port) const noexcept {
    const StorageView& view = getView(port);
    if (view.getDims().size() != 2) { return MatrixLayout{0, 0}; }
    if (view.getIndexType() == FTRAIN_INDEX_TYPE_CONTINUOUS) { return MatrixLayout{view.getDims()[1], 1}; }
    if (view.getIndexType() == FTRAIN_INDEX_TYPE_INVALID && view.getStrides().size() == 2) {
        return MatrixLayout{view.getStrides()[0], view.getStrides()[1]};
    }
    return MatrixLayout{0, 0};
}

std::vector<std::uint64_t> GemmProblem::getProblemKey() const {
    std::vector<std::uint64_t> key;
    key.reserve(kKeyWords);
    for (const Tensor& port : ports_) { appendView(key, port.getStorageView()); }
    key.push_back(static_cast<std::uint64_t>(compute_type_));
    key.push_back(isInPlace() ? 1U : 0U);
    return key;
}

}  // namespace ftrain
