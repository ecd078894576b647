// Compute-graph topology: builder, validated Pattern and its canonical key.
//
// A Pattern is a bipartite graph of operands (Tensor / TensorList /
// GroupedTensor roles) and operations with ORDERED input and output ports.
// Behaviour follows the reference (src/include/flash_train/pattern.hpp:112-192,
// src/pattern.cpp:140-295): the builder only appends; build() validates ids,
// port uniqueness, single producer and acyclicity, then derives a structural
// colouring whose sorted colours form the PatternKey. Two graphs that differ
// only in the order their pieces were added get equal keys; port order matters.
#ifndef FTRAIN_CORE_PATTERN_HPP_
#define FTRAIN_CORE_PATTERN_HPP_

#include <cstddef>
#include <cstdint>
#include <vector>

namespace ftrain {

enum class OperandKind : std::uint8_t { kTensor, kTensorList, kGroupedTensor };

enum class OperationKind : std::uint16_t { kGemm, kGroupedABCDGemm, kGroupedBCDGemm, kGroupedABGemm };

// Index value meaning "no such node".
constexpr std::uint64_t kNoNode = ~std::uint64_t{0};

// One use of an operand by an operation port.
struct PortRef {
    std::uint64_t op;
    std::uint64_t port;
    bool operator==(const PortRef& other) const noexcept { return op == other.op && port == other.port; }
};

struct OperationNode {
    OperationKind kind;
    std::vector<std::uint64_t> inputs;   // operand indices, port order
    std::vector<std::uint64_t> outputs;  // operand indices, port order
};

struct OperandNode {
    OperandKind kind;
    PortRef producer{kNoNode, 0};    // producer.op == kNoNode: graph input
    std::vector<PortRef> consumers;  // unordered
    bool hasProducer() const noexcept { return producer.op != kNoNode; }
};

// Order-independent structural fingerprint; compared token by token.
class PatternKey final {
  public:
    PatternKey() = default;
    explicit PatternKey(std::vector<std::uint64_t>&& tokens) noexcept;

    bool operator==(const PatternKey& other) const noexcept { return hash_ == other.hash_ && tokens_ == other.tokens_; }
    bool operator!=(const PatternKey& other) const noexcept { return !(*this == other); }
    std::size_t getHash() const noexcept { return hash_; }

  private:
    std::vector<std::uint64_t> tokens_;
    std::size_t hash_{0};
};

struct PatternKeyHasher {
    std::size_t operator()(const PatternKey& key) const noexcept { return key.getHash(); }
};

class Pattern final {
  public:
    const PatternKey& getKey() const noexcept { return key_; }
    std::uint64_t getNumOperands() const noexcept { return operands_.size(); }
    std::uint64_t getNumOps() const noexcept { return ops_.size(); }
    // Out-of-range indices throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT).
    const OperandNode& getOperandNode(std::uint64_t index) const;
    const OperationNode& getOpNode(std::uint64_t index) const;
    // Structurally indistinguishable nodes share a colour; colours are
    // comparable across Patterns.
    const std::vector<std::uint64_t>& getOperandColors() const noexcept { return operand_colors_; }
    const std::vector<std::uint64_t>& getOpColors() const noexcept { return op_colors_; }

  private:
    friend class PatternBuilder;
    std::vector<OperandNode> operands_;
    std::vector<OperationNode> ops_;
    std::vector<std::uint64_t> operand_colors_;
    std::vector<std::uint64_t> op_colors_;
    PatternKey key_;
};

class PatternBuilder final {
  public:
    // Both return the new node's 0-based index within its own sequence.
    std::uint64_t addOperand(OperandKind kind);
    std::uint64_t addOperation(OperationKind kind, std::vector<std::uint64_t> inputs,
                               std::vector<std::uint64_t> outputs);

    // Throws Exception(FTRAIN_STATUS_INVALID_ARGUMENT) naming the offending
    // operation and port; the builder is unchanged either way.
    Pattern build() const;

  private:
    std::vector<OperandKind> operand_kinds_;
    std::vector<OperationNode> ops_;
};

}  // namespace ftrain

#endif
