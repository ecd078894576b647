// Selection cache and engine selection semantics, with mock Family / Finder /
// Primitive policy types injected at the template level.
// Behaviours pinned by the reference's tests/cache/cache_test.cpp:35-234 and
// tests/engine/engine_test.cpp:276-555.
#include <atomic>
#include <string>
#include <thread>
#include <type_traits>

#include "core/engine.hpp"
#include "fake_platform.hpp"
#include "mini_test.hpp"

using namespace ftrain;

// ------------------------------------------------------------------ cache

static_assert(std::is_trivially_copyable<CacheKey>::value, "CacheKey must be trivially copyable");

TEST(cache_key_depends_on_group_boundary) {
    CHECK(CacheKey({2}, {3, 5, 8}) != CacheKey({2, 3}, {5, 8}));
    CHECK(CacheKey({2}, {3, 5, 8}) == CacheKey({2}, {3, 5, 8}));
    CHECK(CacheKey({}, {1}) != CacheKey({1}, {}));
    CHECK(CacheKey({7}, {1, 2}) != CacheKey({7}, {2, 1}));
    CHECK(CacheKey({0}, {1}) != CacheKey({1}, {1}));  // another device
}

TEST(cache_first_publish_wins) {
    MemoryPrimitiveCache cache(16, 1);
    const CacheKey key({0}, {1, 2, 3});
    CHECK(!cache.find(key).has_value());
    cache.publish(key, {2, 0});
    cache.publish(key, {1});
    const auto found = cache.find(key);
    CHECK(found.has_value() && *found == (std::vector<std::size_t>{2, 0}));
    CHECK_EQ(cache.getSize(), static_cast<std::size_t>(1));
    CHECK_THROWS_STATUS(cache.publish(CacheKey({0}, {9}), {}), FTRAIN_STATUS_INVALID_ARGUMENT);
    CHECK_THROWS_STATUS(MemoryPrimitiveCache(0), FTRAIN_STATUS_INVALID_ARGUMENT);
    CHECK_THROWS_STATUS(MemoryPrimitiveCache(4, 0), FTRAIN_STATUS_INVALID_ARGUMENT);
}

TEST(cache_evicts_least_hit_entries) {
    // One shard of four entries: a fifth key evicts the coldest one.
    MemoryPrimitiveCache small(4, 1);
    for (std::uint64_t i = 0; i < 4; ++i) { small.publish(CacheKey({0}, {i}), {static_cast<std::size_t>(i)}); }
    for (std::uint64_t i = 0; i < 4; ++i) {
        if (i != 2) { small.find(CacheKey({0}, {i})); }
    }
    small.publish(CacheKey({0}, {99}), {7});
    CHECK_EQ(small.getSize(), static_cast<std::size_t>(4));
    CHECK(!small.find(CacheKey({0}, {2})).has_value());
    CHECK(small.find(CacheKey({0}, {99})).has_value());
    // Sixteen entries: a full shard sheds an eighth (two) of them at once.
    MemoryPrimitiveCache batch(16, 1);
    for (std::uint64_t i = 0; i < 16; ++i) { batch.publish(CacheKey({0}, {i}), {1}); }
    for (std::uint64_t i = 2; i < 16; ++i) { batch.find(CacheKey({0}, {i})); }
    batch.publish(CacheKey({0}, {100}), {1});
    CHECK_EQ(batch.getSize(), static_cast<std::size_t>(15));
    CHECK(!batch.find(CacheKey({0}, {0})).has_value() && !batch.find(CacheKey({0}, {1})).has_value());
}

TEST(cache_is_safe_under_concurrent_use) {
    MemoryPrimitiveCache cache(100000);
    std::atomic<int> wrong{0};
    std::vector<std::thread> workers;
    for (int worker = 0; worker < 8; ++worker) {
        workers.emplace_back([&, worker] {
            for (std::uint64_t i = 0; i < 2000; ++i) {
                const CacheKey key({0}, {i % 500});
                cache.publish(key, {static_cast<std::size_t>(i % 500), static_cast<std::size_t>(worker)});
                const auto found = cache.find(key);
                if (!found.has_value() || (*found)[0] != i % 500) { ++wrong; }
            }
        });
    }
    for (auto& worker : workers) { worker.join(); }
    CHECK_EQ(wrong.load(), 0);
    CHECK_EQ(cache.getSize(), static_cast<std::size_t>(500));
}

TEST(name_lists_and_switches_parse_like_the_reference) {
    const auto names = parseNameList(" Fp32Gemm ,\tOther,, ,Third");
    CHECK_EQ(names.size(), static_cast<std::size_t>(3));
    CHECK(names.count("Fp32Gemm") == 1 && names.count("Other") == 1 && names.count("Third") == 1);
    CHECK(parseNameList(nullptr).empty() && parseNameList("").empty());
    CHECK(!parseSwitch(nullptr) && !parseSwitch("") && !parseSwitch(" 0 ") && !parseSwitch("\t"));
    CHECK(parseSwitch("1") && parseSwitch("true") && parseSwitch(" 00 "));
    CHECK(isPrimitiveAllowed("a", {}, {}) && !isPrimitiveAllowed("a", {}, {"a"}));
    CHECK(isPrimitiveAllowed("a", {"a"}, {}) && !isPrimitiveAllowed("b", {"a"}, {}) && !isPrimitiveAllowed("a", {"a"}, {"a"}));
}

// ------------------------------------------------------------------ engine with mocks

namespace {

struct Counters {
    std::atomic<int> applicable_calls{0};
    std::atomic<int> configure_calls{0};
    std::atomic<int> finder_calls{0};
};

Counters& counters() {
    static Counters value;
    return value;
}

struct MockProblem {
    std::uint64_t size;
    void* address;
    std::vector<std::uint64_t> getProblemKey() const { return {1, size}; }  // the address is not part of the key
};

struct MockPrimitive final : Primitive<MockProblem> {
    MockPrimitive(const char* name, std::uint64_t max_size, std::uint64_t workspace)
        : name_(name), max_size_(max_size), workspace_(workspace) {}
    const char* getName() const noexcept override { return name_; }
    std::unique_ptr<PrimitiveBase> clone() const override { return std::make_unique<MockPrimitive>(*this); }
    std::uint64_t getRequiredWorkspaceBytes() const noexcept override { return workspace_; }
    Result isApplicable(const MockProblem& problem, const Constraints&) const override {
        ++counters().applicable_calls;
        if (problem.size > max_size_) { return Result(FTRAIN_STATUS_UNSUPPORTED, "too large"); }
        return Result{};
    }
    void configure(const MockProblem& problem) override {
        ++counters().configure_calls;
        bound_address = problem.address;
    }
    void executeImpl(const Resources&) override {}

    void* bound_address = nullptr;

  private:
    const char* name_;
    std::uint64_t max_size_;
    std::uint64_t workspace_;
};

Pattern mockPattern(int extra_operands) {
    PatternBuilder builder;
    std::uint64_t t[6];
    for (auto& id : t) { id = builder.addOperand(OperandKind::kTensor); }
    builder.addOperation(OperationKind::kGemm, {t[0], t[1], t[2], t[3], t[4]}, {t[5]});
    for (int i = 0; i < extra_operands; ++i) { builder.addOperand(OperandKind::kTensorList); }
    return builder.build();
}

struct MockFamily {
    using Problem = MockProblem;
    static Pattern makePattern() { return mockPattern(1); }
    static std::vector<std::shared_ptr<const Primitive<MockProblem>>> makeRecords() {
        return {std::make_shared<MockPrimitive>("small", 10, 0), std::make_shared<MockPrimitive>("medium", 100, 64),
                std::make_shared<MockPrimitive>("large", 1000, 0)};
    }
    static MockProblem makeProblem(const Args& args) {
        // The problem size travels in the first dimension of operand 0; its address rebinds per Args.
        const auto& view = std::get<Tensor>(*args.getOperand(0)).getStorageView();
        if (view.getDims()[0] == 13) { throw Exception(FTRAIN_STATUS_OVERFLOW, "unlucky size"); }
        return MockProblem{static_cast<std::uint64_t>(view.getDims()[0]), view.getMemory()};
    }
};

struct ReversingFinder {
    static const char* getName() { return "Reversing"; }
    static std::vector<std::string> findCandidates(const MockProblem&, const Constraints&) {
        ++counters().finder_calls;
        return {"large", "ghost", "medium", "small"};  // "ghost" matches no record
    }
};

struct EmptyFinder {
    static const char* getName() { return "Empty"; }
    static std::vector<std::string> findCandidates(const MockProblem&, const Constraints&) {
        ++counters().finder_calls;
        return {};
    }
};

struct SmallOnlyFinder {
    static const char* getName() { return "SmallOnly"; }
    static std::vector<std::string> findCandidates(const MockProblem&, const Constraints&) {
        ++counters().finder_calls;
        return {"small"};
    }
};

struct UnreachableFinder {
    static const char* getName() { return "Unreachable"; }
    static std::vector<std::string> findCandidates(const MockProblem&, const Constraints&) {
        throw Exception(FTRAIN_STATUS_INTERNAL_ERROR, "a Finder after the contributing one must not be asked");
    }
};

// Args for the mock pattern with operand 0 shaped (size, 1) at `address`.
Args makeArgs(const Pattern& supported, std::int64_t size, void* address, bool complete = true) {
    const Ops ops(supported, supported);
    Args args = ops.makeArgs();
    float cell = 0;
    for (std::uint64_t role = 0; role < 6; ++role) {
        if (!complete && role == 3) { continue; }
        const std::int64_t dims[2] = {role == 0 ? size : 1, 1};
        FTrainStorageView view{role == 0 ? address : &cell, dims, nullptr, 2, FTRAIN_NUMERIC_TYPE_FP32,
                               FTRAIN_INDEX_TYPE_CONTINUOUS, false};
        args.setOperand(role, OperandKind::kTensor, Tensor(StorageView(view)));
    }
    args.setOperand(6, OperandKind::kTensorList, TensorList({}));
    args.setOperation(0, OperationValue{OperationKind::kGemm, FTRAIN_NUMERIC_TYPE_FP32});
    return args;
}

std::vector<std::string> names(const std::vector<std::unique_ptr<PrimitiveBase>>& primitives) {
    std::vector<std::string> out;
    for (const auto& primitive : primitives) { out.emplace_back(primitive->getName()); }
    return out;
}

void resetCounters() {
    counters().applicable_calls = 0;
    counters().configure_calls  = 0;
    counters().finder_calls     = 0;
}

}  // namespace

TEST(engine_falls_back_to_registration_order) {
    resetCounters();
    const OpsEngine<MockFamily, EmptyFinder> engine;
    float cell = 0;
    const auto all = engine.createPrimitives(makeArgs(engine.getPattern(), 5, &cell), Constraints{0});
    CHECK(names(all) == (std::vector<std::string>{"small", "medium", "large"}));
    const auto some = engine.createPrimitives(makeArgs(engine.getPattern(), 50, &cell), Constraints{0});
    CHECK(names(some) == (std::vector<std::string>{"medium", "large"}));
    CHECK_EQ(some[0]->getRequiredWorkspaceBytes(), std::uint64_t{64});
}

TEST(engine_first_contributing_finder_is_the_selection) {
    resetCounters();
    const OpsEngine<MockFamily, EmptyFinder, ReversingFinder, UnreachableFinder> engine;
    float cell = 0;
    const auto chosen = engine.createPrimitives(makeArgs(engine.getPattern(), 50, &cell), Constraints{0});
    // "small" is offered by the Finder but not applicable at size 50; unknown names are skipped.
    CHECK(names(chosen) == (std::vector<std::string>{"large", "medium"}));
    CHECK_EQ(counters().finder_calls.load(), 2);
}

TEST(engine_does_not_recheck_what_a_finder_already_offered) {
    resetCounters();
    const OpsEngine<MockFamily, SmallOnlyFinder> engine;
    float cell = 0;
    // "small" is rejected at size 50, the Finder contributes nothing, and the
    // registration walk offers only the two records not yet seen.
    const auto chosen = engine.createPrimitives(makeArgs(engine.getPattern(), 50, &cell), Constraints{0});
    CHECK(names(chosen) == (std::vector<std::string>{"medium", "large"}));
    CHECK_EQ(counters().applicable_calls.load(), 3);
}

TEST(engine_cache_hit_skips_selection_but_reconfigures) {
    resetCounters();
    const OpsEngine<MockFamily, ReversingFinder> engine;
    float first_cell = 0, second_cell = 0;
    const auto first = engine.createPrimitives(makeArgs(engine.getPattern(), 7, &first_cell), Constraints{0});
    const int applicable_after_first = counters().applicable_calls.load();
    const int finder_after_first     = counters().finder_calls.load();
    const int configure_after_first  = counters().configure_calls.load();
    CHECK_EQ(engine.getCacheSize(), static_cast<std::size_t>(1));
    const auto second = engine.createPrimitives(makeArgs(engine.getPattern(), 7, &second_cell), Constraints{0});
    CHECK(names(second) == names(first));
    CHECK_EQ(counters().applicable_calls.load(), applicable_after_first);  // no extra applicability checks
    CHECK_EQ(counters().finder_calls.load(), finder_after_first);          // no extra Finder calls
    CHECK_EQ(counters().configure_calls.load(), configure_after_first + static_cast<int>(second.size()));
    // Each Plan's clones are bound to its own Args' addresses.
    CHECK(static_cast<MockPrimitive&>(*first[0]).bound_address == &first_cell);
    CHECK(static_cast<MockPrimitive&>(*second[0]).bound_address == &second_cell);
    CHECK(first[0].get() != second[0].get());
    // Another size or another device is another cache entry.
    engine.createPrimitives(makeArgs(engine.getPattern(), 8, &first_cell), Constraints{0});
    engine.createPrimitives(makeArgs(engine.getPattern(), 7, &first_cell), Constraints{1});
    CHECK_EQ(engine.getCacheSize(), static_cast<std::size_t>(3));
}

TEST(engine_error_statuses) {
    const OpsEngine<MockFamily, EmptyFinder> engine;
    float cell = 0;
    try {
        engine.createPrimitives(makeArgs(engine.getPattern(), 5000, &cell), Constraints{0});
        CHECK(false);
    } catch (const Exception& error) {
        CHECK_EQ(static_cast<int>(error.getResult().getStatus()), static_cast<int>(FTRAIN_STATUS_UNSUPPORTED));
        const std::string text = error.what();
        CHECK(text.find("No Primitive supports the supplied Args and runtime constraints (") == 0);
        CHECK(text.find("small: too large; medium: too large; large: too large") != std::string::npos);
    }
    CHECK_THROWS_STATUS(engine.createPrimitives(makeArgs(engine.getPattern(), 5, &cell, false), Constraints{0}),
                        FTRAIN_STATUS_INVALID_ARGUMENT);  // incomplete Args
    CHECK_THROWS_STATUS(engine.createPrimitives(makeArgs(engine.getPattern(), 13, &cell), Constraints{0}),
                        FTRAIN_STATUS_OVERFLOW);  // the family's own validation
    const Pattern other = mockPattern(2);
    const Ops other_ops(other, other);
    CHECK_THROWS_STATUS(engine.createPrimitives(other_ops.makeArgs(), Constraints{0}), FTRAIN_STATUS_INVALID_ARGUMENT);
}

namespace {

struct DuplicateNameFamily : MockFamily {
    static std::vector<std::shared_ptr<const Primitive<MockProblem>>> makeRecords() {
        return {std::make_shared<MockPrimitive>("same", 10, 0), std::make_shared<MockPrimitive>("same", 20, 0)};
    }
};

struct NullRecordFamily : MockFamily {
    static std::vector<std::shared_ptr<const Primitive<MockProblem>>> makeRecords() { return {nullptr}; }
};

}  // namespace

TEST(engine_rejects_bad_catalogues) {
    using Duplicate = OpsEngine<DuplicateNameFamily>;
    using Null      = OpsEngine<NullRecordFamily>;
    CHECK_THROWS_STATUS(Duplicate(), FTRAIN_STATUS_INVALID_ARGUMENT);
    CHECK_THROWS_STATUS(Null(), FTRAIN_STATUS_INVALID_ARGUMENT);
}

TEST(engine_is_safe_for_concurrent_plan_creation) {
    const OpsEngine<MockFamily, ReversingFinder> engine;
    std::atomic<int> wrong{0};
    std::vector<std::thread> workers;
    for (int worker = 0; worker < 8; ++worker) {
        workers.emplace_back([&, worker] {
            float cell = 0;
            for (int i = 0; i < 200; ++i) {
                const std::int64_t size = 1 + (i % 5) * 20 + (worker % 2);
                const auto chosen       = engine.createPrimitives(makeArgs(engine.getPattern(), size, &cell), Constraints{0});
                if (chosen.empty() || std::string(chosen[0]->getName()) != "large") { ++wrong; }
            }
        });
    }
    for (auto& worker : workers) { worker.join(); }
    CHECK_EQ(wrong.load(), 0);
}

TEST(create_plan_binds_the_current_device) {
    fake::reset();
    fake::state().device = 3;
    const OpsEngine<MockFamily, EmptyFinder> engine;
    float cell = 0;
    Plan plan  = engine.createPlan(makeArgs(engine.getPattern(), 5, &cell));
    CHECK_EQ(plan.getNumPrimitives(), std::uint64_t{3});
    plan.execute(0, nullptr, 0, nullptr);
    fake::state().device = 4;
    try {
        plan.execute(0, nullptr, 0, nullptr);
        CHECK(false);
    } catch (const Exception& error) {
        CHECK_EQ(static_cast<int>(error.getResult().getStatus()), static_cast<int>(FTRAIN_STATUS_INVALID_ARGUMENT));
        CHECK(std::string(error.what()).find("calling thread uses device 4") != std::string::npos);
    }
    fake::state().device_query_fails = true;
    CHECK_THROWS_STATUS(engine.createPlan(makeArgs(engine.getPattern(), 5, &cell)), FTRAIN_STATUS_INTERNAL_ERROR);
    fake::reset();
}
