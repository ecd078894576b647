#include "core/pattern.hpp"

#include <algorithm>
#include <utility>

#include "core/error.hpp"

namespace ftrain {
namespace {

// 64-bit mixing step (splitmix64 finaliser) used for colours and key hashes.
std::uint64_t mix(std::uint64_t state, std::uint64_t value) noexcept {
    std::uint64_t z = state + 0x9E3779B97F4A7C15ULL + value;
    z               = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
    z               = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
    return z ^ (z >> 31);
}

std::size_t countDistinct(const std::vector<std::uint64_t>& a, const std::vector<std::uint64_t>& b) {
    std::vector<std::uint64_t> all(a);
    all.insert(all.end(), b.begin(), b.end());
    std::sort(all.begin(), all.end());
    return static_cast<std::size_t>(std::unique(all.begin(), all.end()) - all.begin());
}

constexpr std::uint64_t kOperandTag = 0x4F50444E;  // distinguishes the two node classes
constexpr std::uint64_t kOpTag      = 0x4F504E44;

// One round of colour refinement: every node's new colour hashes its old
// colour with its neighbours' old colours -- consumers as a sorted multiset
// (their order carries no meaning), ports in port order (it does).
void refine(const std::vector<OperandNode>& operands, const std::vector<OperationNode>& ops,
            std::vector<std::uint64_t>& operand_colors, std::vector<std::uint64_t>& op_colors) {
    std::vector<std::uint64_t> next_operand(operands.size());
    std::vector<std::uint64_t> next_op(ops.size());
    std::vector<std::pair<std::uint64_t, std::uint64_t>> uses;
    for (std::size_t i = 0; i < operands.size(); ++i) {
        const OperandNode& node = operands[i];
        std::uint64_t h         = mix(kOperandTag, operand_colors[i]);
        h                       = mix(h, static_cast<std::uint64_t>(node.kind));
        if (node.hasProducer()) {
            h = mix(h, 1);
            h = mix(h, node.producer.port);
            h = mix(h, op_colors[node.producer.op]);
        } else {
            h = mix(h, 0);
        }
        uses.clear();
        for (const PortRef& use : node.consumers) { uses.emplace_back(use.port, op_colors[use.op]); }
        std::sort(uses.begin(), uses.end());
        h = mix(h, uses.size());
        for (const auto& use : uses) { h = mix(mix(h, use.first), use.second); }
        next_operand[i] = h;
    }
    for (std::size_t i = 0; i < ops.size(); ++i) {
        const OperationNode& node = ops[i];
        std::uint64_t h           = mix(kOpTag, op_colors[i]);
        h                         = mix(h, static_cast<std::uint64_t>(node.kind));
        h                         = mix(h, node.inputs.size());
        for (const std::uint64_t operand : node.inputs) { h = mix(h, operand_colors[operand]); }
        h = mix(h, node.outputs.size());
        for (const std::uint64_t operand : node.outputs) { h = mix(h, operand_colors[operand]); }
        next_op[i] = h;
    }
    operand_colors.swap(next_operand);
    op_colors.swap(next_op);
}

}  // namespace

PatternKey::PatternKey(std::vector<std::uint64_t>&& tokens) noexcept : tokens_(std::move(tokens)) {
    std::uint64_t h = mix(0, tokens_.size());
    for (const std::uint64_t token : tokens_) { h = mix(h, token); }
    hash_ = static_cast<std::size_t>(h);
}

const OperandNode& Pattern::getOperandNode(std::uint64_t index) const {
    if (index >= operands_.size()) {
        throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "Pattern operand index %llu is out of range for %zu operands",
                        static_cast<unsigned long long>(index), operands_.size());
    }
    return operands_[index];
}

const OperationNode& Pattern::getOpNode(std::uint64_t index) const {
    if (index >= ops_.size()) {
        throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "Pattern operation index %llu is out of range for %zu operations",
                        static_cast<unsigned long long>(index), ops_.size());
    }
    return ops_[index];
}

std::uint64_t PatternBuilder::addOperand(OperandKind kind) {
    operand_kinds_.push_back(kind);
    return operand_kinds_.size() - 1;
}

std::uint64_t PatternBuilder::addOperation(OperationKind kind, std::vector<std::uint64_t> inputs,
                                           std::vector<std::uint64_t> outputs) {
    ops_.push_back(OperationNode{kind, std::move(inputs), std::move(outputs)});
    return ops_.size() - 1;
}

Pattern PatternBuilder::build() const {
    const std::size_t num_operands = operand_kinds_.size();
    Pattern pattern;
    pattern.operands_.resize(num_operands);
    for (std::size_t i = 0; i < num_operands; ++i) { pattern.operands_[i].kind = operand_kinds_[i]; }

    // Wiring: ids in range, no operand twice among one operation's inputs or
    // outputs, no output that is also an input, one producer per operand.
    for (std::size_t op = 0; op < ops_.size(); ++op) {
        const OperationNode& node = ops_[op];
        for (std::size_t port = 0; port < node.inputs.size(); ++port) {
            const std::uint64_t operand = node.inputs[port];
            if (operand >= num_operands) {
                throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT,
                                "Operation %zu input port %zu references out-of-range operand %llu for %zu operands", op,
                                port, static_cast<unsigned long long>(operand), num_operands);
            }
            if (std::find(node.inputs.begin(), node.inputs.begin() + static_cast<std::ptrdiff_t>(port), operand) !=
                node.inputs.begin() + static_cast<std::ptrdiff_t>(port)) {
                throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "Operation %zu repeats operand %llu across input ports",
                                op, static_cast<unsigned long long>(operand));
            }
            pattern.operands_[operand].consumers.push_back(PortRef{op, port});
        }
        for (std::size_t port = 0; port < node.outputs.size(); ++port) {
            const std::uint64_t operand = node.outputs[port];
            if (operand >= num_operands) {
                throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT,
                                "Operation %zu output port %zu references out-of-range operand %llu for %zu operands",
                                op, port, static_cast<unsigned long long>(operand), num_operands);
            }
            if (std::find(node.inputs.begin(), node.inputs.end(), operand) != node.inputs.end()) {
                throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT,
                                "Operation %zu output port %zu reuses operand %llu from an input port", op, port,
                                static_cast<unsigned long long>(operand));
            }
            if (std::find(node.outputs.begin(), node.outputs.begin() + static_cast<std::ptrdiff_t>(port), operand) !=
                node.outputs.begin() + static_cast<std::ptrdiff_t>(port)) {
                throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "Operation %zu repeats operand %llu across output ports",
                                op, static_cast<unsigned long long>(operand));
            }
            if (pattern.operands_[operand].hasProducer()) {
                throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT,
                                "Operation %zu output port %zu reuses operand %llu that already has a producer", op, port,
                                static_cast<unsigned long long>(operand));
            }
            pattern.operands_[operand].producer = PortRef{op, port};
        }
    }

    // Acyclicity by topological peeling over "consumes what the other produces".
    std::vector<std::size_t> pending(ops_.size(), 0);
    for (std::size_t op = 0; op < ops_.size(); ++op) {
        for (const std::uint64_t operand : ops_[op].inputs) {
            if (pattern.operands_[operand].hasProducer()) { ++pending[op]; }
        }
    }
    std::vector<std::size_t> ready;
    for (std::size_t op = 0; op < ops_.size(); ++op) {
        if (pending[op] == 0) { ready.push_back(op); }
    }
    std::size_t peeled = 0;
    while (!ready.empty()) {
        const std::size_t op = ready.back();
        ready.pop_back();
        ++peeled;
        for (const std::uint64_t produced : ops_[op].outputs) {
            for (const PortRef& use : pattern.operands_[produced].consumers) {
                if (--pending[use.op] == 0) { ready.push_back(use.op); }
            }
        }
    }
    if (peeled != ops_.size()) {
        for (std::size_t op = 0; op < ops_.size(); ++op) {
            if (pending[op] == 0) { continue; }
            for (const std::uint64_t operand : ops_[op].inputs) {
                const OperandNode& source = pattern.operands_[operand];
                if (source.hasProducer() && pending[source.producer.op] != 0) {
                    throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT,
                                    "Operation %zu input port participates in a dependency cycle through operand %llu",
                                    op, static_cast<unsigned long long>(operand));
                }
            }
        }
        throw Exception(FTRAIN_STATUS_INTERNAL_ERROR, "Cycle detection peeled %zu of %zu operations but named no edge",
                        peeled, ops_.size());
    }

    pattern.ops_ = ops_;

    // Colour refinement to a stable partition (at most one round per node).
    pattern.operand_colors_.assign(num_operands, 0);
    pattern.op_colors_.assign(ops_.size(), 0);
    const std::size_t num_nodes = num_operands + ops_.size();
    std::size_t classes         = 0;
    for (std::size_t round = 0; round <= num_nodes; ++round) {
        refine(pattern.operands_, pattern.ops_, pattern.operand_colors_, pattern.op_colors_);
        const std::size_t refined = countDistinct(pattern.operand_colors_, pattern.op_colors_);
        if (refined == classes || refined == num_nodes) { break; }
        classes = refined;
    }

    std::vector<std::uint64_t> tokens(pattern.operand_colors_);
    tokens.insert(tokens.end(), pattern.op_colors_.begin(), pattern.op_colors_.end());
    std::sort(tokens.begin(), tokens.end());
    pattern.key_ = PatternKey(std::move(tokens));
    return pattern;
}

}  // namespace ftrain
