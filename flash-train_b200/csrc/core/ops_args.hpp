// Ops (a matched Pattern) and Args (one call's concrete values).
//
// Behaviour follows the reference (src/include/flash_train/ops_args.hpp:25-112,
// src/ops_args.cpp:431-657): constructing an Ops matches the user's Pattern
// against a supported Pattern -- insertion order of operands, operations and
// consumers is irrelevant, port order is significant -- and records, for every
// user role id, the supported role it plays. Args then stores values in
// supported-role slots while callers keep addressing them by their own ids.
//
// Structure differs from the reference: the matched schema is one immutable
// object shared (by reference count) between the Ops and every Args made from
// it, so ftrainArgsCreate allocates only the two slot arrays; and matching is a
// single colour-pruned backtracking search.
#ifndef FTRAIN_CORE_OPS_ARGS_HPP_
#define FTRAIN_CORE_OPS_ARGS_HPP_

#include <cstddef>
#include <cstdint>
#include <memory>
#include <optional>
#include <variant>
#include <vector>

#include "core/pattern.hpp"
#include "core/tensor.hpp"

namespace ftrain {

using OperandValue = std::variant<Tensor, TensorList, GroupedTensor>;

// Per-call attributes of one operation. Every operation kind of the public
// API carries exactly a compute type.
struct OperationValue {
    OperationKind kind;
    FTrainNumericType compute_type;
};

// Returns, for each user operand / operation index, the supported-Pattern index
// it corresponds to, or nullopt when the two graphs are not isomorphic.
struct RoleMapping {
    std::vector<std::uint64_t> operand;
    std::vector<std::uint64_t> op;
};
std::optional<RoleMapping> matchPatterns(const Pattern& user, const Pattern& supported);

// What an Args needs to know about its Ops; immutable once built.
struct OpsSchema {
    PatternKey key;
    RoleMapping user_to_supported;
    std::vector<OperandKind> operand_kinds;  // indexed by supported operand
    std::vector<OperationKind> op_kinds;     // indexed by supported operation
};

class Args;

class Ops final {
  public:
    // Throws Exception(FTRAIN_STATUS_UNSUPPORTED) when the graphs differ.
    Ops(const Pattern& user_pattern, const Pattern& supported_pattern);

    const PatternKey& getPatternKey() const noexcept { return schema_->key; }
    // Every slot of the returned Args is unset.
    Args makeArgs() const;

  private:
    std::shared_ptr<const OpsSchema> schema_;
};

class Args final {
  public:
    const PatternKey& getPatternKey() const noexcept { return schema_->key; }
    std::uint64_t getNumOperands() const noexcept { return operands_.size(); }
    std::uint64_t getNumOps() const noexcept { return op_values_.size(); }
    bool isComplete() const noexcept;

    // Slot access by SUPPORTED role index (what a family uses). Out of range
    // throws Exception(FTRAIN_STATUS_INVALID_ARGUMENT).
    const std::optional<OperandValue>& getOperand(std::uint64_t supported_operand) const;
    const std::optional<OperationValue>& getOpArgument(std::uint64_t supported_op) const;

    // Setters by USER role index. An id out of range, or a role of another
    // storage family / operation kind, throws
    // Exception(FTRAIN_STATUS_INVALID_ARGUMENT) and leaves the Args unchanged.
    void setOperand(std::uint64_t user_operand, OperandKind kind, OperandValue&& value);
    void setOperation(std::uint64_t user_op, OperationValue value);

  private:
    friend class Ops;
    explicit Args(std::shared_ptr<const OpsSchema> schema);

    std::shared_ptr<const OpsSchema> schema_;
    std::vector<std::optional<OperandValue>> operands_;
    std::vector<std::optional<OperationValue>> op_values_;
};

}  // namespace ftrain

#endif
