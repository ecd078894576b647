#include "core/ops_args.hpp"

#include <algorithm>
#include <utility>

#include "core/error.hpp"

namespace ftrain {
namespace {

// Backtracking isomorphism search over operations. Mapping one user operation
// onto a supported one fixes, port by port, the operands on its ports; the
// search keeps both directions of the operand map and undoes them on retreat.
// Colours from Pattern::build() prune candidates: isomorphic nodes always share
// a colour, so only same-colour pairs are tried.
class Search final {
  public:
    Search(const Pattern& user, const Pattern& supported)
        : user_(user), supported_(supported), operand_fwd_(user.getNumOperands(), kNoNode),
          operand_bwd_(supported.getNumOperands(), kNoNode), op_fwd_(user.getNumOps(), kNoNode),
          op_taken_(supported.getNumOps(), false) {}

    bool run() {
        if (user_.getNumOperands() != supported_.getNumOperands() || user_.getNumOps() != supported_.getNumOps()) {
            return false;
        }
        return placeOp(0) && placeLooseOperands();
    }

    RoleMapping take() { return RoleMapping{std::move(operand_fwd_), std::move(op_fwd_)}; }

  private:
    bool placeOp(std::uint64_t user_op) {
        if (user_op == user_.getNumOps()) { return true; }
        const OperationNode& u = user_.getOpNode(user_op);
        for (std::uint64_t candidate = 0; candidate < supported_.getNumOps(); ++candidate) {
            if (op_taken_[candidate]) { continue; }
            if (user_.getOpColors()[user_op] != supported_.getOpColors()[candidate]) { continue; }
            const OperationNode& s = supported_.getOpNode(candidate);
            if (u.kind != s.kind || u.inputs.size() != s.inputs.size() || u.outputs.size() != s.outputs.size()) {
                continue;
            }
            const std::size_t mark = trail_.size();
            if (bindPorts(u.inputs, s.inputs) && bindPorts(u.outputs, s.outputs)) {
                op_taken_[candidate] = true;
                op_fwd_[user_op]     = candidate;
                if (placeOp(user_op + 1)) { return true; }
                op_taken_[candidate] = false;
                op_fwd_[user_op]     = kNoNode;
            }
            unwind(mark);
        }
        return false;
    }

    bool bindPorts(const std::vector<std::uint64_t>& user_ports, const std::vector<std::uint64_t>& supported_ports) {
        for (std::size_t port = 0; port < user_ports.size(); ++port) {
            if (!bindOperand(user_ports[port], supported_ports[port])) { return false; }
        }
        return true;
    }

    bool bindOperand(std::uint64_t u, std::uint64_t s) {
        if (operand_fwd_[u] != kNoNode || operand_bwd_[s] != kNoNode) {
            return operand_fwd_[u] == s && operand_bwd_[s] == u;
        }
        const OperandNode& un = user_.getOperandNode(u);
        const OperandNode& sn = supported_.getOperandNode(s);
        if (un.kind != sn.kind || un.hasProducer() != sn.hasProducer() ||
            un.consumers.size() != sn.consumers.size() ||
            (un.hasProducer() && un.producer.port != sn.producer.port)) {
            return false;
        }
        operand_fwd_[u] = s;
        operand_bwd_[s] = u;
        trail_.push_back(u);
        return true;
    }

    void unwind(std::size_t mark) {
        while (trail_.size() > mark) {
            const std::uint64_t u         = trail_.back();
            operand_bwd_[operand_fwd_[u]] = kNoNode;
            operand_fwd_[u]               = kNoNode;
            trail_.pop_back();
        }
    }

    // Operands wired to no operation are interchangeable within a kind: pair
    // them in index order.
    bool placeLooseOperands() {
        for (std::uint64_t u = 0; u < user_.getNumOperands(); ++u) {
            if (operand_fwd_[u] != kNoNode) { continue; }
            bool placed = false;
            for (std::uint64_t s = 0; s < supported_.getNumOperands() && !placed; ++s) {
                if (operand_bwd_[s] != kNoNode) { continue; }
                const OperandNode& sn = supported_.getOperandNode(s);
                if (sn.kind != user_.getOperandNode(u).kind || sn.hasProducer() || !sn.consumers.empty()) { continue; }
                operand_fwd_[u] = s;
                operand_bwd_[s] = u;
                placed          = true;
            }
            if (!placed) { return false; }
        }
        return true;
    }

    const Pattern& user_;
    const Pattern& supported_;
    std::vector<std::uint64_t> operand_fwd_;
    std::vector<std::uint64_t> operand_bwd_;
    std::vector<std::uint64_t> op_fwd_;
    std::vector<bool> op_taken_;
    std::vector<std::uint64_t> trail_;
};

}  // namespace

std::optional<RoleMapping> matchPatterns(const Pattern& user, const Pattern& supported) {
    Search search(user, supported);
    if (!search.run()) { return std::nullopt; }
    return search.take();
}

Ops::Ops(const Pattern& user_pattern, const Pattern& supported_pattern) {
    std::optional<RoleMapping> mapping;
    if (user_pattern.getKey() == supported_pattern.getKey()) { mapping = matchPatterns(user_pattern, supported_pattern); }
    if (!mapping.has_value()) {
        throw Exception(FTRAIN_STATUS_UNSUPPORTED, "Ops: user Pattern does not match the supported Pattern");
    }
    auto schema               = std::make_shared<OpsSchema>();
    schema->key               = user_pattern.getKey();
    schema->user_to_supported = std::move(*mapping);
    for (std::uint64_t i = 0; i < supported_pattern.getNumOperands(); ++i) {
        schema->operand_kinds.push_back(supported_pattern.getOperandNode(i).kind);
    }
    for (std::uint64_t i = 0; i < supported_pattern.getNumOps(); ++i) {
        schema->op_kinds.push_back(supported_pattern.getOpNode(i).kind);
    }
    schema_ = std::move(schema);
}

Args Ops::makeArgs() const { return Args(schema_); }

Args::Args(std::shared_ptr<const OpsSchema> schema)
    : schema_(std::move(schema)), operands_(schema_->operand_kinds.size()), op_values_(schema_->op_kinds.size()) {}

bool Args::isComplete() const noexcept {
    for (const auto& slot : operands_) {
        if (!slot.has_value()) { return false; }
    }
    for (const auto& slot : op_values_) {
        if (!slot.has_value()) { return false; }
    }
    return true;
}

const std::optional<OperandValue>& Args::getOperand(std::uint64_t supported_operand) const {
    if (supported_operand >= operands_.size()) {
        throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "Supported OperandValue role index %llu is out of range [0, %zu)",
                        static_cast<unsigned long long>(supported_operand), operands_.size());
    }
    return operands_[supported_operand];
}

const std::optional<OperationValue>& Args::getOpArgument(std::uint64_t supported_op) const {
    if (supported_op >= op_values_.size()) {
        throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "Supported Op role index %llu is out of range [0, %zu)",
                        static_cast<unsigned long long>(supported_op), op_values_.size());
    }
    return op_values_[supported_op];
}

void Args::setOperand(std::uint64_t user_operand, OperandKind kind, OperandValue&& value) {
    const std::vector<std::uint64_t>& map = schema_->user_to_supported.operand;
    if (user_operand >= map.size()) {
        throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "User OperandValue role index %llu is out of range [0, %zu)",
                        static_cast<unsigned long long>(user_operand), map.size());
    }
    const std::uint64_t slot = map[user_operand];
    if (slot >= operands_.size()) {
        throw Exception(FTRAIN_STATUS_INTERNAL_ERROR, "Ops operand role mapping contains out-of-range slot %llu",
                        static_cast<unsigned long long>(slot));
    }
    if (schema_->operand_kinds[slot] != kind) {
        throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "User OperandValue role %llu has a different storage family",
                        static_cast<unsigned long long>(user_operand));
    }
    operands_[slot] = std::move(value);
}

void Args::setOperation(std::uint64_t user_op, OperationValue value) {
    const std::vector<std::uint64_t>& map = schema_->user_to_supported.op;
    if (user_op >= map.size()) {
        throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "User Op role index %llu is out of range [0, %zu)",
                        static_cast<unsigned long long>(user_op), map.size());
    }
    const std::uint64_t slot = map[user_op];
    if (slot >= op_values_.size()) {
        throw Exception(FTRAIN_STATUS_INTERNAL_ERROR, "Ops operation role mapping contains out-of-range slot %llu",
                        static_cast<unsigned long long>(slot));
    }
    if (schema_->op_kinds[slot] != value.kind) {
        throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "User Op role %llu has a different operation kind",
                        static_cast<unsigned long long>(user_op));
    }
    op_values_[slot] = value;
}

}  // namespace ftrain
