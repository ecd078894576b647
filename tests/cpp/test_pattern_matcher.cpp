// Pattern validation, the order-independent key, and matching.
// Behaviours pinned by the reference's tests/pattern_test.cpp and
// tests/matcher_test.cpp:235-574 (insertion order ignored, port order
// significant, disconnected and symmetric components, a case that needs
// backtracking).
#include <algorithm>
#include <numeric>
#include <random>

#include "core/ops_args.hpp"
#include "mini_test.hpp"

using namespace ftrain;

namespace {

// Gemm node: inputs (a, b, c, alpha, beta), output d.
std::uint64_t addGemm(PatternBuilder& builder, std::uint64_t a, std::uint64_t b, std::uint64_t c, std::uint64_t d,
                      std::uint64_t alpha, std::uint64_t beta, OperationKind kind = OperationKind::kGemm) {
    return builder.addOperation(kind, {a, b, c, alpha, beta}, {d});
}

Pattern singleGemm(const std::vector<int>& order) {
    // order: a permutation of the positions at which roles a,b,c,alpha,beta,d are added.
    PatternBuilder builder;
    std::uint64_t role[6];
    for (int slot = 0; slot < 6; ++slot) {
        role[order[slot]] = builder.addOperand(OperandKind::kTensor);
    }
    addGemm(builder, role[0], role[1], role[2], role[5], role[3], role[4]);
    return builder.build();
}

// Two chained Gemms: d1 feeds the second one's `a` port (or `b` port).
Pattern chained(bool into_b, bool second_first) {
    PatternBuilder builder;
    std::uint64_t t[11];
    for (auto& id : t) { id = builder.addOperand(OperandKind::kTensor); }
    const auto first  = [&] { addGemm(builder, t[0], t[1], t[2], t[3], t[4], t[5]); };
    const auto second = [&] {
        if (into_b) {
            addGemm(builder, t[6], t[3], t[7], t[8], t[9], t[10]);
        } else {
            addGemm(builder, t[3], t[6], t[7], t[8], t[9], t[10]);
        }
    };
    if (second_first) {
        second();
        first();
    } else {
        first();
        second();
    }
    return builder.build();
}

}  // namespace

TEST(builder_numbers_nodes_from_zero) {
    PatternBuilder builder;
    CHECK_EQ(builder.addOperand(OperandKind::kTensor), std::uint64_t{0});
    CHECK_EQ(builder.addOperand(OperandKind::kTensorList), std::uint64_t{1});
    CHECK_EQ(builder.addOperand(OperandKind::kGroupedTensor), std::uint64_t{2});
    for (int i = 0; i < 4; ++i) { builder.addOperand(OperandKind::kTensor); }
    CHECK_EQ(addGemm(builder, 0, 3, 4, 5, 6, 1), std::uint64_t{0});  // operations count separately
}

TEST(build_reports_wiring_errors) {
    {
        PatternBuilder builder;
        for (int i = 0; i < 6; ++i) { builder.addOperand(OperandKind::kTensor); }
        addGemm(builder, 0, 1, 2, 9, 3, 4);  // output id out of range
        CHECK_THROWS_STATUS(builder.build(), FTRAIN_STATUS_INVALID_ARGUMENT);
    }
    {
        PatternBuilder builder;
        for (int i = 0; i < 6; ++i) { builder.addOperand(OperandKind::kTensor); }
        addGemm(builder, 0, 0, 2, 5, 3, 4);  // operand repeated across inputs
        CHECK_THROWS_STATUS(builder.build(), FTRAIN_STATUS_INVALID_ARGUMENT);
    }
    {
        PatternBuilder builder;
        for (int i = 0; i < 6; ++i) { builder.addOperand(OperandKind::kTensor); }
        addGemm(builder, 0, 1, 2, 2, 3, 4);  // output is also an input
        CHECK_THROWS_STATUS(builder.build(), FTRAIN_STATUS_INVALID_ARGUMENT);
    }
    {
        PatternBuilder builder;
        for (int i = 0; i < 11; ++i) { builder.addOperand(OperandKind::kTensor); }
        addGemm(builder, 0, 1, 2, 3, 4, 5);
        addGemm(builder, 6, 7, 8, 3, 9, 10);  // second producer for operand 3
        CHECK_THROWS_STATUS(builder.build(), FTRAIN_STATUS_INVALID_ARGUMENT);
    }
    {
        PatternBuilder builder;  // two operations feeding each other
        for (int i = 0; i < 10; ++i) { builder.addOperand(OperandKind::kTensor); }
        addGemm(builder, 9, 1, 2, 3, 4, 5);
        addGemm(builder, 3, 6, 7, 9, 8, 0);
        CHECK_THROWS_STATUS(builder.build(), FTRAIN_STATUS_INVALID_ARGUMENT);
    }
    PatternBuilder empty;
    const Pattern nothing = empty.build();
    CHECK_EQ(nothing.getNumOperands(), std::uint64_t{0});
    CHECK_THROWS_STATUS(nothing.getOperandNode(0), FTRAIN_STATUS_INVALID_ARGUMENT);
    CHECK_THROWS_STATUS(nothing.getOpNode(0), FTRAIN_STATUS_INVALID_ARGUMENT);
}

TEST(key_ignores_insertion_order) {
    const Pattern canonical = singleGemm({0, 1, 2, 3, 4, 5});
    std::vector<int> order  = {0, 1, 2, 3, 4, 5};
    std::mt19937 rng(7);
    for (int trial = 0; trial < 20; ++trial) {
        std::shuffle(order.begin(), order.end(), rng);
        const Pattern shuffled = singleGemm(order);
        CHECK(shuffled.getKey() == canonical.getKey());
        CHECK_EQ(shuffled.getKey().getHash(), canonical.getKey().getHash());
        const auto mapping = matchPatterns(shuffled, canonical);
        CHECK(mapping.has_value());
        if (mapping.has_value()) {
            // The operand added at position `slot` plays role order[slot] (a,b,c,alpha,beta,d = 0..5), and the
            // canonical builder added its roles in exactly that order.
            for (int slot = 0; slot < 6; ++slot) { CHECK_EQ(mapping->operand[slot], static_cast<std::uint64_t>(order[slot])); }
        }
    }
    CHECK(chained(false, false).getKey() == chained(false, true).getKey());
}

TEST(key_respects_port_order_and_kinds) {
    CHECK(chained(false, false).getKey() != chained(true, false).getKey());
    CHECK(!matchPatterns(chained(false, false), chained(true, false)).has_value());
    PatternBuilder grouped;
    std::uint64_t g[4];
    for (auto& id : g) { id = grouped.addOperand(OperandKind::kGroupedTensor); }
    const std::uint64_t alpha = grouped.addOperand(OperandKind::kTensor);
    const std::uint64_t beta  = grouped.addOperand(OperandKind::kTensor);
    addGemm(grouped, g[0], g[1], g[2], g[3], alpha, beta, OperationKind::kGroupedABCDGemm);
    CHECK(grouped.build().getKey() != singleGemm({0, 1, 2, 3, 4, 5}).getKey());
    // A dangling extra operand changes the structure.
    PatternBuilder extra;
    std::uint64_t t[7];
    for (auto& id : t) { id = extra.addOperand(OperandKind::kTensor); }
    addGemm(extra, t[0], t[1], t[2], t[5], t[3], t[4]);
    CHECK(extra.build().getKey() != singleGemm({0, 1, 2, 3, 4, 5}).getKey());
}

TEST(symmetric_and_disconnected_components_match) {
    // Two independent Gemms plus two loose operands, built in different orders.
    const auto make = [](bool reversed) {
        PatternBuilder builder;
        std::vector<std::uint64_t> t(14);
        for (auto& id : t) { id = builder.addOperand(OperandKind::kTensor); }
        if (reversed) { std::reverse(t.begin(), t.end()); }
        addGemm(builder, t[0], t[1], t[2], t[3], t[4], t[5]);
        addGemm(builder, t[6], t[7], t[8], t[9], t[10], t[11]);
        return builder.build();
    };
    const Pattern left  = make(false);
    const Pattern right = make(true);
    CHECK(left.getKey() == right.getKey());
    const auto mapping = matchPatterns(left, right);
    CHECK(mapping.has_value());
    if (mapping.has_value()) {
        std::vector<std::uint64_t> image = mapping->operand;
        std::sort(image.begin(), image.end());
        for (std::uint64_t i = 0; i < image.size(); ++i) { CHECK_EQ(image[i], i); }  // a bijection
        // Each user operation's ports map onto the ports of its image.
        for (std::uint64_t op = 0; op < left.getNumOps(); ++op) {
            const OperationNode& u = left.getOpNode(op);
            const OperationNode& s = right.getOpNode(mapping->op[op]);
            for (std::size_t port = 0; port < u.inputs.size(); ++port) {
                CHECK_EQ(mapping->operand[u.inputs[port]], s.inputs[port]);
            }
            CHECK_EQ(mapping->operand[u.outputs[0]], s.outputs[0]);
        }
    }
}

TEST(matching_backtracks_when_colours_tie) {
    // A ring-free "ladder" whose two middle operations are structurally alike
    // until their far ends are considered: producer -> {left, right} -> two sinks
    // where only one sink feeds a final operation. Colours separate them after
    // refinement, and the search must still find the one consistent assignment
    // whichever candidate it tries first.
    const auto make = [](bool swap_branches) {
        PatternBuilder builder;
        std::vector<std::uint64_t> t(26);
        for (auto& id : t) { id = builder.addOperand(OperandKind::kTensor); }
        const auto gemm = [&](int base, std::uint64_t a_operand, std::uint64_t out) {
            addGemm(builder, a_operand, t[base], t[base + 1], out, t[base + 2], t[base + 3]);
        };
        gemm(0, t[4], t[5]);                              // root: produces t5
        const int first = swap_branches ? 10 : 6;
        const int other = swap_branches ? 6 : 10;
        gemm(first, t[5], t[first + 4 == 10 ? 14 : 15]);  // branch
        gemm(other, t[5], t[other + 4 == 10 ? 14 : 15]);  // branch
        gemm(16, t[14], t[20]);                           // only the t14 branch continues
        return builder.build();
    };
    const Pattern one = make(false);
    const Pattern two = make(true);
    CHECK(one.getKey() == two.getKey());
    CHECK(matchPatterns(one, two).has_value());
    CHECK(matchPatterns(two, one).has_value());
}

TEST(ops_rejects_a_different_graph) {
    const Pattern supported = singleGemm({0, 1, 2, 3, 4, 5});
    CHECK_THROWS_STATUS(Ops(chained(false, false), supported), FTRAIN_STATUS_UNSUPPORTED);
    const Ops matched(singleGemm({5, 4, 3, 2, 1, 0}), supported);
    CHECK(matched.getPatternKey() == supported.getKey());
}
