// GemmProblem: one validated D = alpha*A*B + beta*C call, as a checklist of
// properties a Primitive decides support on.
//
// Validation and getters follow the reference (src/family/gemm/problem.cpp:13-56,
// src/include/flash_train/family/gemm/problem.hpp:35-118): a, b, c, d rank two in
// device memory; alpha, beta scalars in host memory; a's columns = b's rows;
// c and d m-by-n; every matrix byte count fits 64 bits.
//
// Two additions for this platform:
//   * getLayout(): row/column strides in elements for a, b, c, d, derived from
//     either layout source (CONTINUOUS = dense row-major, or the view's
//     strides), because the CUDA kernels accept strided views;
//   * getProblemKey() records each address modulo 16 (the reference records
//     modulo 4, problem.cpp:75-76): 16-byte alignment decides whether a matrix
//     can be fetched by TMA, and a cache hit skips the applicability check.
#ifndef FTRAIN_FAMILY_GEMM_PROBLEM_HPP_
#define FTRAIN_FAMILY_GEMM_PROBLEM_HPP_

#include <cstdint>
#include <vector>

#include "core/tensor.hpp"

namespace ftrain {

struct GemmShape {
    std::uint64_t m;
    std::uint64_t n;
    std::uint64_t k;
};

// Element strides of a rank-two view.
struct MatrixLayout {
    std::int64_t row_stride;
    std::int64_t col_stride;
};

enum class GemmPort : int { kA = 0, kB, kC, kD, kAlpha, kBeta };

class GemmProblem final {
  public:
    // Throws Exception with FTRAIN_STATUS_INVALID_ARGUMENT or FTRAIN_STATUS_OVERFLOW.
    GemmProblem(Tensor a, Tensor b, Tensor c, Tensor d, Tensor alpha, Tensor beta, FTrainNumericType compute_type);

    GemmShape getShape() const noexcept { return shape_; }
    bool hasEmptyOutput() const noexcept { return shape_.m * shape_.n == 0; }
    FTrainNumericType getComputeType() const noexcept { return compute_type_; }

    const StorageView& getView(GemmPort port) const noexcept { return ports_[static_cast<int>(port)].getStorageView(); }
    FTrainNumericType getNumericType(GemmPort port) const noexcept { return getView(port).getNumericType(); }
    FTrainIndexType getIndexType(GemmPort port) const noexcept { return getView(port).getIndexType(); }
    void* getAddress(GemmPort port) const noexcept { return getView(port).getMemory(); }

    // Only for kA..kD, and only when the port's index type is CONTINUOUS or
    // INVALID (strides given); other predefined layouts return {0, 0}.
    MatrixLayout getLayout(GemmPort port) const noexcept;

    // c and d are the same address: D is accumulated in place.
    bool isInPlace() const noexcept { return getAddress(GemmPort::kC) == getAddress(GemmPort::kD); }

    // Everything that can change which Primitive applies or wins, as tokens: per
    // view a fixed head (types, rank and stride count packed into one word;
    // has-memory; address modulo 16; length of the tail) and then its extents and
    // strides, after the six views the compute type and the in-place flag. The
    // heads carry the lengths, so distinct descriptions cannot alias. Addresses
    // enter only through null-ness, alignment class and aliasing.
    std::vector<std::uint64_t> getProblemKey() const;

  private:
    Tensor ports_[6];
    FTrainNumericType compute_type_;
    GemmShape shape_{};
};

}  // namespace ftrain

#endif
