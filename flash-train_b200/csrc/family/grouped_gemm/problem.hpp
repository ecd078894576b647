// GroupedGemmProblem: one validated grouped GEMM call,
//     D_g = alpha * A_g * B_g + beta * C_g   for every group g,
// for the three grouped operations of the public API: GroupedABCDGemm (a, b, c, d GroupedTensors),
// GroupedBCDGemm (a a TensorList) and GroupedABGemm (c and d TensorLists).
//
// The reference declares the operations and their operand families in its public API
// (include/flash_train/common.h:248-306, 376-430 there; operation nodes in
// src/include/flash_train/operation/gemm.hpp:80-150) but registers no engine for any of them
// (src/engine.cpp:25-27), so what a group "is" is taken from the contracts of the public header:
//   * GroupedTensor: element (i, j) of group g lies at logical element
//         offsets[g] + i * strides[0][g] + j * strides[1][g]
//     from data.memory, for 0 <= i < dim_sizes[0][g], 0 <= j < dim_sizes[1][g];
//   * TensorList: group g is the list's g-th view, an ordinary rank-two matrix view.
//
// What this family accepts (anything else is INVALID_ARGUMENT when the description contradicts
// itself, UNSUPPORTED when it is merely something no Primitive here handles):
//   * a, b, c, d: rank two, the same number of groups, data in device memory (every c may be
//     null: no beta * C term);
//   * GroupedTensor: dim_sizes present, as INT64 / UINT64 / INT32 / UINT32 arrays in HOST memory
//     (the tile lists of the kernels are built on the host when the Plan is made); offsets and
//     strides optional, host arrays of the same types. Without strides a group is dense row-major;
//     without offsets the groups follow one another densely (FTRAIN_INDEX_TYPE_GROUPED_CONTINUOUS);
//   * per group: a is m x k, b is k x n, c and d are m x n. Empty groups are allowed.
#ifndef FTRAIN_FAMILY_GROUPED_GEMM_PROBLEM_HPP_
#define FTRAIN_FAMILY_GROUPED_GEMM_PROBLEM_HPP_

#include <cstdint>
#include <vector>

#include "core/ops_args.hpp"
#include "core/tensor.hpp"

namespace ftrain {

// One group's matrix as the kernels see it: address, extents and element strides.
struct GroupMatrix {
    const void* base;     // data address of the operand the group lives in (null: no memory)
    std::int64_t offset;  // elements from `base`
    std::int64_t rows, cols;
    std::int64_t row_stride, col_stride;
    const float* address() const noexcept { return base == nullptr ? nullptr : static_cast<const float*>(base) + offset; }
};

// One operand (a, b, c or d), decoded: a GroupedTensor or a TensorList.
struct GroupedOperand {
    bool is_list = false;
    // Common to all of the operand's views: INVALID (0) when a TensorList mixes types.
    FTrainNumericType numeric_type = FTRAIN_NUMERIC_TYPE_INVALID;
    bool plainly_indexed           = true;   // every view is CONTINUOUS / GROUPED_CONTINUOUS or carries strides
    bool in_device_memory          = true;
    bool any_memory                = false;  // some group has an address
    bool all_memory                = true;   // every group with elements has one
    bool float_aligned             = true;
    std::vector<GroupMatrix> groups;
};

enum class GroupedPort : int { kA = 0, kB, kC, kD };

class GroupedGemmProblem final {
  public:
    // Each operand is the GroupedTensor or TensorList stored in the Args (a plain Tensor is rejected).
    // Throws Exception: INVALID_ARGUMENT for contradictory descriptions, UNSUPPORTED for metadata
    // this family cannot read (device-resident or of another numeric type), OVERFLOW when a group's
    // byte size does not fit 64 bits.
    GroupedGemmProblem(const OperandValue& a, const OperandValue& b, const OperandValue& c, const OperandValue& d, Tensor alpha,
                       Tensor beta, FTrainNumericType compute_type);

    std::uint32_t getNumGroups() const noexcept { return num_groups_; }
    FTrainNumericType getComputeType() const noexcept { return compute_type_; }
    const GroupedOperand& getOperand(GroupedPort port) const noexcept { return operands_[static_cast<int>(port)]; }
    const StorageView& getAlpha() const noexcept { return alpha_.getStorageView(); }
    const StorageView& getBeta() const noexcept { return beta_.getStorageView(); }
    const GroupMatrix& getGroup(GroupedPort port, std::uint32_t group) const noexcept { return getOperand(port).groups[group]; }
    bool hasEmptyOutput() const noexcept { return output_elements_ == 0; }
    // c and d describe the same memory group by group: D is accumulated in place.
    bool isInPlace() const noexcept;

    // Everything that can change which Primitive applies or wins: per operand its kind and type
    // summary, then every group's null-ness, alignment class, extents and strides; the scalars'
    // description, compute type and the in-place flag last.
    std::vector<std::uint64_t> getProblemKey() const;

  private:
    GroupedOperand operands_[4];
    Tensor alpha_, beta_;
    FTrainNumericType compute_type_;
    std::uint32_t num_groups_{0};
    std::uint64_t output_elements_{0};
};

}  // namespace ftrain

#endif
