// GroupedGemmProblem: one validated GroupedABCDGemm call,
//     D_g = alpha * A_g * B_g + beta * C_g   for every group g,
// over four GroupedTensors and two host scalars.
//
// The reference declares the operation and its operand family in its public API
// (include/flash_train/common.h:248-266, 394-430 there; operation node in
// src/include/flash_train/operation/gemm.hpp:80-104) but registers no engine for it
// (src/engine.cpp:25-27), so what a group "is" is taken from the GroupedTensor contract of the
// public header: element (i, j) of group g lies at logical element
//     offsets[g] + i * strides[0][g] + j * strides[1][g]
// from data.memory, for 0 <= i < dim_sizes[0][g], 0 <= j < dim_sizes[1][g].
//
// What this family accepts (anything else is INVALID_ARGUMENT when the description contradicts
// itself, UNSUPPORTED when it is merely something no Primitive here handles):
//   * a, b, c, d: rank-two GroupedTensors with the same number of groups; data in device memory
//     (c's data may be null: no beta * C term);
//   * dim_sizes present for all four, as INT64 / UINT64 / INT32 / UINT32 arrays in HOST memory
//     (the tile lists of the kernels are built on the host when the Plan is made);
//   * offsets and strides optional, host arrays of the same types. Without strides a group is
//     dense row-major; without offsets the groups follow one another densely
//     (FTRAIN_INDEX_TYPE_GROUPED_CONTINUOUS);
//   * per group: a is m x k, b is k x n, c and d are m x n. Empty groups are allowed.
#ifndef FTRAIN_FAMILY_GROUPED_GEMM_PROBLEM_HPP_
#define FTRAIN_FAMILY_GROUPED_GEMM_PROBLEM_HPP_

#include <cstdint>
#include <vector>

#include "core/tensor.hpp"

namespace ftrain {

// One group's matrix as the kernels see it: element offset from the data address, extents and
// element strides.
struct GroupMatrix {
    std::int64_t offset;
    std::int64_t rows, cols;
    std::int64_t row_stride, col_stride;
};

enum class GroupedPort : int { kA = 0, kB, kC, kD };

class GroupedGemmProblem final {
  public:
    // Throws Exception: INVALID_ARGUMENT for contradictory descriptions, UNSUPPORTED for metadata
    // this family cannot read (device-resident or of another numeric type), OVERFLOW when a group's
    // byte size does not fit 64 bits.
    GroupedGemmProblem(GroupedTensor a, GroupedTensor b, GroupedTensor c, GroupedTensor d, Tensor alpha, Tensor beta,
                       FTrainNumericType compute_type);

    std::uint32_t getNumGroups() const noexcept { return num_groups_; }
    FTrainNumericType getComputeType() const noexcept { return compute_type_; }
    const GroupedTensor& getTensor(GroupedPort port) const noexcept { return tensors_[static_cast<int>(port)]; }
    const StorageView& getData(GroupedPort port) const noexcept { return getTensor(port).getData(); }
    const StorageView& getAlpha() const noexcept { return alpha_.getStorageView(); }
    const StorageView& getBeta() const noexcept { return beta_.getStorageView(); }
    // Group g of a port, decoded from the host metadata.
    const GroupMatrix& getGroup(GroupedPort port, std::uint32_t group) const noexcept {
        return groups_[static_cast<int>(port)][group];
    }
    bool hasEmptyOutput() const noexcept { return output_elements_ == 0; }
    // c and d describe the same memory group by group: D is accumulated in place.
    bool isInPlace() const noexcept;

    // Everything that can change which Primitive applies or wins: per tensor the data view's
    // types, null-ness and alignment class, then every group's offset, extents and strides;
    // compute type and the in-place flag last.
    std::vector<std::uint64_t> getProblemKey() const;

  private:
    GroupedTensor tensors_[4];
    Tensor alpha_, beta_;
    FTrainNumericType compute_type_;
    std::uint32_t num_groups_;
    std::vector<GroupMatrix> groups_[4];
    std::uint64_t output_elements_{0};
};

}  // namespace ftrain

#endif
