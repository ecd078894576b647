#include "family/gemm/problem.hpp"

#include <limits>
#include <utility>

#include "core/error.hpp"

namespace ftrain {

GemmProblem::GemmProblem(Tensor a, Tensor b, Tensor c, Tensor d, Tensor alpha, Tensor beta,
                         FTrainNumericType compute_type)
    : ports_{std::move(a), std::move(b), std::move(c), std::move(d), std::move(alpha), std::move(beta)},
      compute_type_(compute_type) {
    const StorageView& av = getView(GemmPort::kA);
    const StorageView& bv = getView(GemmPort::kB);
    const StorageView& cv = getView(GemmPort::kC);
    const StorageView& dv = getView(GemmPort::kD);
    const StorageView& alpha_v = getView(GemmPort::kAlpha);
    const StorageView& beta_v  = getView(GemmPort::kBeta);

    if (av.getDims().size() != 2 || bv.getDims().size() != 2 || cv.getDims().size() != 2 || dv.getDims().size() != 2) {
        throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "Gemm requires rank-two a, b, c, and d Tensors");
    }
    if (!alpha_v.getDims().empty() || !beta_v.getDims().empty()) {
        throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "Gemm requires scalar alpha and beta Tensors");
    }
    if (av.isHostMemory() || bv.isHostMemory() || cv.isHostMemory() || dv.isHostMemory()) {
        throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "Gemm requires a, b, c, and d in device memory");
    }
    if (!alpha_v.isHostMemory() || !beta_v.isHostMemory()) {
        throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "Gemm requires alpha and beta in host memory");
    }

    shape_ = GemmShape{static_cast<std::uint64_t>(av.getDims()[0]), static_cast<std::uint64_t>(bv.getDims()[1]),
                       static_cast<std::uint64_t>(av.getDims()[1])};
    if (av.getDims()[1] != bv.getDims()[0]) {
        throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "Gemm a column count %lld does not match b row count %lld",
                        static_cast<long long>(av.getDims()[1]), static_cast<long long>(bv.getDims()[0]));
    }
    const std::int64_t rows = av.getDims()[0];
    const std::int64_t cols = bv.getDims()[1];
    if (cv.getDims()[0] != rows || cv.getDims()[1] != cols || dv.getDims()[0] != rows || dv.getDims()[1] != cols) {
        throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "Gemm c and d shapes must both be m-by-n");
    }

    const std::uint64_t budget = std::numeric_limits<std::uint64_t>::max() / sizeof(float);
    const auto overflows       = [budget](std::uint64_t x, std::uint64_t y) { return y != 0 && x > budget / y; };
    if (overflows(shape_.m, shape_.k) || overflows(shape_.k, shape_.n) || overflows(shape_.m, shape_.n)) {
        throw Exception(FTRAIN_STATUS_OVERFLOW, "Gemm matrix byte size overflows uint64_t");
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
    key.reserve(96);
    std::uint64_t field = 0;
    for (const Tensor& port : ports_) {
        const StorageView& view = port.getStorageView();
        const bool present      = view.getMemory() != nullptr;
        key.push_back(++field);
        key.push_back(view.getNumericType());
        key.push_back(++field);
        key.push_back(view.getIndexType());
        key.push_back(++field);
        key.push_back(present ? 1 : 0);
        key.push_back(++field);
        key.push_back(present ? reinterpret_cast<std::uintptr_t>(view.getMemory()) % 16 : 0);
        key.push_back(++field);
        key.push_back(view.getDims().size());
        for (const std::int64_t dim : view.getDims()) { key.push_back(static_cast<std::uint64_t>(dim)); }
        key.push_back(++field);
        key.push_back(view.getStrides().size());
        for (const std::int64_t stride : view.getStrides()) { key.push_back(static_cast<std::uint64_t>(stride)); }
    }
    key.push_back(++field);
    key.push_back(compute_type_);
    key.push_back(++field);
    key.push_back(isInPlace() ? 1 : 0);
    return key;
}

}  // namespace ftrain
