// GemmProblem validation, the CUDA Primitives' support checklist (on fake
// addresses: nothing is launched), Plan dispatch and the B200 Finder.
// Behaviours pinned by the reference's tests/primitive/hygon/gemm/fp32_gemm_test.cpp:90-196,
// tests/plan_test.cpp:69-148, tests/primitive_test.cpp:70-103 and
// tests/family/gemm/gemm_test.cpp:34-56.
#include <array>
#include <cstring>
#include <string>

#include "core/handle.hpp"
#include "core/plan.hpp"
#include "fake_platform.hpp"
#include "family/gemm/family.hpp"
#include "family/gemm/finder.hpp"
#include "mini_test.hpp"
#include "primitive/cuda/gemm/cuda_gemm.hpp"

using namespace ftrain;

namespace {

float g_alpha = 1.5F;
float g_beta  = 0.25F;

struct ViewSpec {
    void* memory;
    std::int64_t rows, cols;
    FTrainNumericType type  = FTRAIN_NUMERIC_TYPE_FP32;
    FTrainIndexType index   = FTRAIN_INDEX_TYPE_CONTINUOUS;
    const std::int64_t* strides = nullptr;
    bool host               = false;
};

Tensor matrix(const ViewSpec& spec) {
    const std::int64_t dims[2] = {spec.rows, spec.cols};
    return Tensor(StorageView(FTrainStorageView{spec.memory, dims, spec.strides, 2, spec.type, spec.index, spec.host}));
}

Tensor scalar(float* value, bool host = true, FTrainNumericType type = FTRAIN_NUMERIC_TYPE_FP32,
              FTrainIndexType index = FTRAIN_INDEX_TYPE_CONTINUOUS) {
    return Tensor(StorageView(FTrainStorageView{value, nullptr, nullptr, 0, type, index, host}));
}

void* address(std::uintptr_t value) { return reinterpret_cast<void*>(value); }

// A well-formed m x k x n problem on made-up 256-byte aligned device addresses.
GemmProblem problem(std::int64_t m, std::int64_t k, std::int64_t n, FTrainNumericType compute = FTRAIN_NUMERIC_TYPE_FP32) {
    return GemmProblem(matrix({address(0x10000), m, k}), matrix({address(0x20000), k, n}), matrix({address(0x30000), m, n}),
                       matrix({address(0x40000), m, n}), scalar(&g_alpha), scalar(&g_beta), compute);
}

std::string reason(const Result& result) { return result.getMessage(); }

}  // namespace

TEST(problem_validation_statuses) {
    const GemmProblem fine = problem(4, 3, 5);
    CHECK_EQ(fine.getShape().m, std::uint64_t{4});
    CHECK_EQ(fine.getShape().k, std::uint64_t{3});
    CHECK_EQ(fine.getShape().n, std::uint64_t{5});
    CHECK(!fine.hasEmptyOutput() && !fine.isInPlace());
    const auto a = [] { return matrix({address(0x100), 4, 3}); };
    const auto b = [] { return matrix({address(0x200), 3, 5}); };
    const auto c = [] { return matrix({address(0x300), 4, 5}); };
    const auto d = [] { return matrix({address(0x400), 4, 5}); };
    const std::int64_t cube[3] = {2, 2, 2};
    float cell = 0;
    const Tensor rank3(StorageView(FTrainStorageView{&cell, cube, nullptr, 3, FTRAIN_NUMERIC_TYPE_FP32, FTRAIN_INDEX_TYPE_CONTINUOUS, false}));
    CHECK_THROWS_STATUS(GemmProblem(rank3, b(), c(), d(), scalar(&g_alpha), scalar(&g_beta), FTRAIN_NUMERIC_TYPE_FP32),
                        FTRAIN_STATUS_INVALID_ARGUMENT);
    CHECK_THROWS_STATUS(GemmProblem(a(), b(), c(), d(), matrix({&cell, 1, 1}), scalar(&g_beta), FTRAIN_NUMERIC_TYPE_FP32),
                        FTRAIN_STATUS_INVALID_ARGUMENT);  // alpha is not a scalar
    CHECK_THROWS_STATUS(GemmProblem(matrix({address(0x100), 4, 3, FTRAIN_NUMERIC_TYPE_FP32, FTRAIN_INDEX_TYPE_CONTINUOUS, nullptr, true}),
                                    b(), c(), d(), scalar(&g_alpha), scalar(&g_beta), FTRAIN_NUMERIC_TYPE_FP32),
                        FTRAIN_STATUS_INVALID_ARGUMENT);  // a in host memory
    CHECK_THROWS_STATUS(GemmProblem(a(), b(), c(), d(), scalar(&g_alpha, false), scalar(&g_beta), FTRAIN_NUMERIC_TYPE_FP32),
                        FTRAIN_STATUS_INVALID_ARGUMENT);  // alpha in device memory
    CHECK_THROWS_STATUS(GemmProblem(a(), matrix({address(0x200), 4, 5}), c(), d(), scalar(&g_alpha), scalar(&g_beta), FTRAIN_NUMERIC_TYPE_FP32),
                        FTRAIN_STATUS_INVALID_ARGUMENT);  // a's columns != b's rows
    CHECK_THROWS_STATUS(GemmProblem(a(), b(), matrix({address(0x300), 5, 4}), d(), scalar(&g_alpha), scalar(&g_beta), FTRAIN_NUMERIC_TYPE_FP32),
                        FTRAIN_STATUS_INVALID_ARGUMENT);  // c is not m x n
    const std::int64_t huge = INT64_MAX;
    CHECK_THROWS_STATUS(GemmProblem(matrix({nullptr, huge, huge}), matrix({nullptr, huge, huge}), matrix({nullptr, huge, huge}),
                                    matrix({nullptr, huge, huge}), scalar(&g_alpha), scalar(&g_beta), FTRAIN_NUMERIC_TYPE_FP32),
                        FTRAIN_STATUS_OVERFLOW);
}

TEST(problem_key_covers_what_selection_depends_on) {
    const auto key = [](const GemmProblem& p) { return p.getProblemKey(); };
    const GemmProblem base = problem(128, 64, 96);
    CHECK(key(base) == key(problem(128, 64, 96)));
    CHECK(key(base) != key(problem(128, 64, 100)));
    CHECK(key(base) != key(problem(128, 64, 96, FTRAIN_NUMERIC_TYPE_FP64)));
    // Other addresses with the same alignment class, null-ness and aliasing: same key.
    const GemmProblem moved(matrix({address(0x50000), 128, 64}), matrix({address(0x60000), 64, 96}), matrix({address(0x70000), 128, 96}),
                            matrix({address(0x80000), 128, 96}), scalar(&g_alpha), scalar(&g_beta), FTRAIN_NUMERIC_TYPE_FP32);
    CHECK(key(base) == key(moved));
    // Alignment class (modulo 16), a null C, and in-place C == D each change it.
    const GemmProblem shifted(matrix({address(0x10004), 128, 64}), matrix({address(0x20000), 64, 96}), matrix({address(0x30000), 128, 96}),
                              matrix({address(0x40000), 128, 96}), scalar(&g_alpha), scalar(&g_beta), FTRAIN_NUMERIC_TYPE_FP32);
    CHECK(key(base) != key(shifted));
    const GemmProblem no_c(matrix({address(0x10000), 128, 64}), matrix({address(0x20000), 64, 96}), matrix({nullptr, 128, 96}),
                           matrix({address(0x40000), 128, 96}), scalar(&g_alpha), scalar(&g_beta), FTRAIN_NUMERIC_TYPE_FP32);
    CHECK(key(base) != key(no_c));
    const GemmProblem in_place(matrix({address(0x10000), 128, 64}), matrix({address(0x20000), 64, 96}), matrix({address(0x40000), 128, 96}),
                               matrix({address(0x40000), 128, 96}), scalar(&g_alpha), scalar(&g_beta), FTRAIN_NUMERIC_TYPE_FP32);
    CHECK(in_place.isInPlace() && key(base) != key(in_place));
    // A strided view of the same shape is another key, and its layout is read from the strides.
    const std::int64_t transposed[2] = {1, 128};
    const GemmProblem strided(matrix({address(0x10000), 128, 64, FTRAIN_NUMERIC_TYPE_FP32, FTRAIN_INDEX_TYPE_INVALID, transposed}),
                              matrix({address(0x20000), 64, 96}), matrix({address(0x30000), 128, 96}), matrix({address(0x40000), 128, 96}),
                              scalar(&g_alpha), scalar(&g_beta), FTRAIN_NUMERIC_TYPE_FP32);
    CHECK(key(base) != key(strided));
    CHECK_EQ(strided.getLayout(GemmPort::kA).row_stride, std::int64_t{1});
    CHECK_EQ(strided.getLayout(GemmPort::kA).col_stride, std::int64_t{128});
    CHECK_EQ(base.getLayout(GemmPort::kA).row_stride, std::int64_t{64});
    CHECK_EQ(base.getLayout(GemmPort::kB).col_stride, std::int64_t{1});
}

TEST(fp32_gemm_checklist) {
    fake::reset();
    const CudaGemm primitive(FTCUDA_GEMM_SIMT);
    const Constraints device0{0};
    CHECK_EQ(std::string(primitive.getName()), std::string("Fp32Gemm"));
    CHECK_EQ(primitive.getRequiredWorkspaceBytes(), std::uint64_t{0});
    CHECK(primitive.isApplicable(problem(4, 3, 5), device0).isSuccess());
    CHECK_EQ(reason(primitive.isApplicable(problem(4, 3, 5, FTRAIN_NUMERIC_TYPE_FP64), device0)), std::string("compute type is not fp32"));
    const auto with_a = [&](const ViewSpec& a_spec) {
        return GemmProblem(matrix(a_spec), matrix({address(0x20000), 3, 5}), matrix({address(0x30000), 4, 5}),
                           matrix({address(0x40000), 4, 5}), scalar(&g_alpha), scalar(&g_beta), FTRAIN_NUMERIC_TYPE_FP32);
    };
    CHECK_EQ(reason(primitive.isApplicable(with_a({address(0x10000), 4, 3, FTRAIN_NUMERIC_TYPE_FP16}), device0)),
             std::string("an operand is not fp32"));
    CHECK_EQ(reason(primitive.isApplicable(with_a({address(0x10000), 4, 3, FTRAIN_NUMERIC_TYPE_FP32, FTRAIN_INDEX_TYPE_GROUPED_CONTINUOUS}), device0)),
             std::string("an operand is not continuously indexed"));
    CHECK_EQ(reason(primitive.isApplicable(with_a({address(0x10002), 4, 3}), device0)), std::string("an operand address is not float-aligned"));
    CHECK_EQ(reason(primitive.isApplicable(with_a({nullptr, 4, 3}), device0)), std::string("a required operand address is null"));
    // Strided views are accepted by this build (the reference's only kernel rejects them).
    const std::int64_t transposed[2] = {1, 4};
    CHECK(primitive.isApplicable(with_a({address(0x10000), 4, 3, FTRAIN_NUMERIC_TYPE_FP32, FTRAIN_INDEX_TYPE_INVALID, transposed}), device0).isSuccess());
    // A null C is fine; a null D is not.
    const GemmProblem no_c(matrix({address(0x10000), 4, 3}), matrix({address(0x20000), 3, 5}), matrix({nullptr, 4, 5}),
                           matrix({address(0x40000), 4, 5}), scalar(&g_alpha), scalar(&g_beta), FTRAIN_NUMERIC_TYPE_FP32);
    CHECK(primitive.isApplicable(no_c, device0).isSuccess());
    const GemmProblem no_d(matrix({address(0x10000), 4, 3}), matrix({address(0x20000), 3, 5}), matrix({address(0x30000), 4, 5}),
                           matrix({nullptr, 4, 5}), scalar(&g_alpha), scalar(&g_beta), FTRAIN_NUMERIC_TYPE_FP32);
    CHECK_EQ(reason(primitive.isApplicable(no_d, device0)), std::string("a required operand address is null"));
    // K == 0 needs neither A nor B; an empty output needs no address at all.
    const GemmProblem zero_depth(matrix({nullptr, 4, 0}), matrix({nullptr, 0, 5}), matrix({address(0x30000), 4, 5}),
                                 matrix({address(0x40000), 4, 5}), scalar(&g_alpha), scalar(&g_beta), FTRAIN_NUMERIC_TYPE_FP32);
    CHECK(primitive.isApplicable(zero_depth, device0).isSuccess());
    const GemmProblem empty(matrix({nullptr, 0, 3}), matrix({nullptr, 3, 5}), matrix({nullptr, 0, 5}), matrix({nullptr, 0, 5}),
                            scalar(&g_alpha), scalar(&g_beta), FTRAIN_NUMERIC_TYPE_FP32);
    CHECK(empty.hasEmptyOutput() && primitive.isApplicable(empty, device0).isSuccess());
    // Scalars must be FP32 and plainly indexed too.
    const GemmProblem half_alpha(matrix({address(0x10000), 4, 3}), matrix({address(0x20000), 3, 5}), matrix({address(0x30000), 4, 5}),
                                 matrix({address(0x40000), 4, 5}), scalar(&g_alpha, true, FTRAIN_NUMERIC_TYPE_FP16), scalar(&g_beta),
                                 FTRAIN_NUMERIC_TYPE_FP32);
    CHECK_EQ(reason(primitive.isApplicable(half_alpha, device0)), std::string("an operand is not fp32"));
}

TEST(configured_clone_is_independent_and_reads_scalars_at_configure) {
    fake::reset();
    const CudaGemm prototype(FTCUDA_GEMM_SIMT);
    std::unique_ptr<PrimitiveBase> clone = prototype.clone();
    g_alpha = 2.0F;
    g_beta  = -1.0F;
    static_cast<Primitive<GemmProblem>&>(*clone).configure(problem(4, 3, 5));
    g_alpha = 99.0F;  // changing the host scalars after configure must not matter
    int token = 0;
    clone->execute(Resources{nullptr, 0, reinterpret_cast<FTrainStream>(&token)});
    CHECK_EQ(fake::state().launches.size(), static_cast<std::size_t>(1));
    const fake::LaunchRecord& launch = fake::state().launches[0];
    CHECK_EQ(launch.kernel, static_cast<int>(FTCUDA_GEMM_SIMT));
    CHECK(launch.stream == &token);
    CHECK_EQ(launch.desc.alpha, 2.0F);
    CHECK_EQ(launch.desc.beta, -1.0F);
    CHECK_EQ(launch.desc.m, std::uint64_t{4});
    CHECK_EQ(launch.desc.a_row_stride, std::int64_t{3});
    CHECK(launch.desc.a == address(0x10000) && launch.desc.d == address(0x40000));
    // The prototype stays unconfigured: executing it launches nothing.
    CudaGemm untouched(FTCUDA_GEMM_SIMT);
    untouched.execute(Resources{nullptr, 0, nullptr});
    CHECK_EQ(fake::state().launches.size(), static_cast<std::size_t>(1));
    // An empty problem configures to a no-op.
    std::unique_ptr<PrimitiveBase> nothing = prototype.clone();
    static_cast<Primitive<GemmProblem>&>(*nothing).configure(GemmProblem(
        matrix({nullptr, 0, 3}), matrix({nullptr, 3, 5}), matrix({nullptr, 0, 5}), matrix({nullptr, 0, 5}), scalar(&g_alpha),
        scalar(&g_beta), FTRAIN_NUMERIC_TYPE_FP32));
    nothing->execute(Resources{nullptr, 0, nullptr});
    CHECK_EQ(fake::state().launches.size(), static_cast<std::size_t>(1));
    g_alpha = 1.5F;
    g_beta  = 0.25F;
    fake::reset();
}

TEST(plan_dispatches_only_the_indexed_primitive) {
    fake::reset();
    std::vector<std::unique_ptr<PrimitiveBase>> primitives;
    for (const int kernel : {FTCUDA_GEMM_TF32X3_SPLITK, FTCUDA_GEMM_TF32X3, FTCUDA_GEMM_SIMT}) {
        auto primitive = std::make_unique<CudaGemm>(kernel);
        primitive->configure(problem(256, 8192, 256));
        primitives.push_back(std::move(primitive));
    }
    Plan plan(std::move(primitives), 0);
    CHECK_EQ(plan.getNumPrimitives(), std::uint64_t{3});
    CHECK_EQ(std::string(plan.getPrimitiveName(0)), std::string("Fp32Gemm3xTf32SplitK"));
    CHECK_EQ(plan.getPrimitiveRequiredWorkspaceBytes(0), std::uint64_t{4096});
    CHECK_EQ(plan.getPrimitiveRequiredWorkspaceBytes(2), std::uint64_t{0});
    CHECK_THROWS_STATUS(plan.getPrimitiveName(3), FTRAIN_STATUS_INVALID_ARGUMENT);
    CHECK_THROWS_STATUS(plan.getPrimitiveRequiredWorkspaceBytes(3), FTRAIN_STATUS_INVALID_ARGUMENT);
    // Short or null workspace and a bad index are refused before anything is dispatched.
    char buffer[8];
    CHECK_THROWS_STATUS(plan.execute(0, buffer, 100, nullptr), FTRAIN_STATUS_INVALID_ARGUMENT);
    CHECK_THROWS_STATUS(plan.execute(0, nullptr, 4096, nullptr), FTRAIN_STATUS_INVALID_ARGUMENT);
    CHECK_THROWS_STATUS(plan.execute(3, nullptr, 0, nullptr), FTRAIN_STATUS_INVALID_ARGUMENT);
    CHECK(fake::state().launches.empty());
    // The workspace pointer and size reach the primitive verbatim.
    plan.execute(0, buffer, 5000, nullptr);
    plan.execute(2, nullptr, 0, nullptr);
    CHECK_EQ(fake::state().launches.size(), static_cast<std::size_t>(2));
    CHECK_EQ(fake::state().launches[0].kernel, static_cast<int>(FTCUDA_GEMM_TF32X3_SPLITK));
    CHECK(fake::state().launches[0].workspace == buffer);
    CHECK_EQ(fake::state().launches[0].workspace_bytes, std::uint64_t{5000});
    CHECK_EQ(fake::state().launches[1].kernel, static_cast<int>(FTCUDA_GEMM_SIMT));
    CHECK_THROWS_STATUS(Plan({}, 0), FTRAIN_STATUS_INVALID_ARGUMENT);
    std::vector<std::unique_ptr<PrimitiveBase>> with_null;
    with_null.push_back(nullptr);
    CHECK_THROWS_STATUS(Plan(std::move(with_null), 0), FTRAIN_STATUS_INVALID_ARGUMENT);
    fake::reset();
}

TEST(finder_regime_map) {
    fake::reset();
    const Constraints device0{0};
    const auto first = [&](std::int64_t m, std::int64_t k, std::int64_t n) {
        return B200Heuristic::findCandidates(problem(m, k, n), device0);
    };
    using Names = std::vector<std::string>;
    CHECK(first(1, 4096, 4096) == (Names{"Fp32GemmSkinny", "Fp32GemmSplitK", "Fp32Gemm"}));
    // From 9 rows on (17 whatever the size of B) B goes through the tensor cores as their 128-row operand.
    CHECK(first(17, 4096, 4096) == (Names{"Fp32Gemm3xTf32FewRows", "Fp32Gemm3xTf32SplitK", "Fp32GemmSkinny", "Fp32Gemm3xTf32",
                                          "Fp32GemmSplitK", "Fp32Gemm"}));
    CHECK(first(12, 4096, 4096).front() == "Fp32Gemm3xTf32FewRows");
    CHECK(first(12, 2048, 2048).front() == "Fp32GemmSkinny");
    CHECK(first(9, 4096, 4096).front() == "Fp32Gemm3xTf32FewRows");
    CHECK(first(8, 4096, 4096).front() == "Fp32GemmSkinny");
    CHECK(first(17, 512, 4096).front() == "Fp32GemmSkinny");
    // 2 x 22 tiles on 148 SMs, K = 4096: the single launch cuts K over clusters of three.
    CHECK(first(255, 4096, 4096) == (Names{"Fp32Gemm3xTf32", "Fp32Gemm3xTf32SplitK", "Fp32GemmSplitK", "Fp32Gemm"}));
    // The same tiles with a deeper K, or under an eighth of a wave of tiles at K = 4096: the two-launch
    // split-K cuts finer. Half as many tiles (22) still go to the single launch, and so does any
    // number of tiles under half a wave when K is at most 2048.
    CHECK(first(255, 16384, 4096).front() == "Fp32Gemm3xTf32SplitK");
    CHECK(first(128, 4096, 4096).front() == "Fp32Gemm3xTf32");
    CHECK(first(128, 4096, 1536).front() == "Fp32Gemm3xTf32SplitK");
    CHECK(first(128, 2048, 768).front() == "Fp32Gemm3xTf32");
    CHECK(first(128, 3072, 1152).front() == "Fp32Gemm3xTf32SplitK");
    CHECK(first(4097, 4096, 4096) == (Names{"Fp32Gemm3xTf32", "Fp32Gemm"}));
    // From 33 rows on the tensor kernel's 128-row tile wins over the SIMT kernel.
    CHECK(first(64, 4096, 4096).front() == "Fp32Gemm3xTf32FewRows");
    CHECK(first(65, 4096, 4096).front() == "Fp32Gemm3xTf32");
    // Narrow and deep: eight K slices per strip are too few CTAs.
    CHECK(first(64, 8192, 1024).front() == "Fp32Gemm3xTf32FewRows");
    CHECK(first(48, 65536, 512)[1] == "Fp32Gemm3xTf32FewRows");
    CHECK(first(48, 65536, 512).front() == "Fp32Gemm3xTf32SplitK");
    CHECK(first(64, 256, 4096).front() == "Fp32Gemm3xTf32FewRows");
    CHECK(first(65, 256, 4096) == (Names{"Fp32Gemm3xTf32", "Fp32Gemm"}));
    // Small outputs with a short K: the exact kernel's 32 x 32 tiling comes first, the tensor kernel behind it.
    CHECK(first(256, 256, 256) == (Names{"Fp32Gemm", "Fp32Gemm3xTf32"}));
    CHECK(first(384, 256, 320) == (Names{"Fp32Gemm", "Fp32Gemm3xTf32"}));
    CHECK(first(384, 512, 384).front() == "Fp32Gemm");  // 72 M multiply-adds, K = 512: still the exact kernel
    CHECK(first(512, 512, 512).front() != "Fp32Gemm");
    CHECK(first(256, 1024, 256).front() != "Fp32Gemm");  // 64 M with K = 1024: the tensor kernel
    CHECK(first(17, 1024, 1024).front() == "Fp32GemmSkinny");
    CHECK(first(17, 2048, 512).front() == "Fp32Gemm3xTf32FewRows");
    CHECK(first(64, 1024, 1024).front() == "Fp32Gemm3xTf32FewRows");
    CHECK(first(96, 1024, 1024) == (Names{"Fp32Gemm3xTf32", "Fp32Gemm3xTf32SplitK", "Fp32GemmSplitK", "Fp32Gemm"}));
    CHECK(first(1024, 1024, 4096) == (Names{"Fp32Gemm3xTf32", "Fp32Gemm"}));
    CHECK(first(1024, 1024, 1024) == (Names{"Fp32Gemm3xTf32", "Fp32Gemm3xTf32SplitK", "Fp32GemmSplitK", "Fp32Gemm"}));
    // Few rows but a narrow B: too few strips for the few-rows kernel.
    CHECK(first(17, 65536, 512).front() == "Fp32Gemm3xTf32SplitK");
    CHECK(first(1, 65536, 512).front() == "Fp32Gemm3xTf32SplitK");
    CHECK(first(17, 16384, 1024).front() == "Fp32Gemm3xTf32FewRows");
    CHECK(first(8, 16384, 1024).front() == "Fp32GemmSkinny");
    CHECK(first(32, 4096, 2048).front() == "Fp32Gemm3xTf32FewRows");
    CHECK(first(16, 4096, 2048).front() == "Fp32Gemm3xTf32FewRows");
    CHECK(first(32, 4096, 4096).front() == "Fp32Gemm3xTf32FewRows");
    CHECK(first(24, 4096, 4096).front() == "Fp32Gemm3xTf32FewRows");
    CHECK(first(64, 1024, 64) == (Names{"Fp32GemmSplitK", "Fp32Gemm"}));
    CHECK(first(16384, 4096, 14336) == (Names{"Fp32Gemm3xTf32", "Fp32Gemm"}));
    CHECK(first(2048, 262144, 2048) == (Names{"Fp32Gemm3xTf32SplitK", "Fp32Gemm3xTf32", "Fp32GemmSplitK", "Fp32Gemm"}));
    CHECK(first(128, 64, 96) == (Names{"Fp32Gemm"}));
    CHECK(first(64, 8192, 64) == (Names{"Fp32GemmSplitK", "Fp32Gemm"}));
    CHECK(first(0, 5, 7) == (Names{"Fp32Gemm"}));
    // Every list ends with the workspace-free, accept-all kernel.
    for (const auto& shape : {std::array<std::int64_t, 3>{3, 3, 3}, {4096, 4096, 4096}, {2048, 9000, 2048}}) {
        CHECK(first(shape[0], shape[1], shape[2]).back() == "Fp32Gemm");
    }
    CHECK_EQ(std::string(B200Heuristic::getName()), std::string("B200Heuristic"));
    CHECK(RegistrationOrderFinder::findCandidates(problem(1, 1, 1), device0).empty());
}

TEST(builtin_gemm_engine_is_registered) {
    Handle& handle = getGlobalHandle();
    CHECK(handle.getNumOpsEngines() >= 1);
    const auto engine = handle.findOpsEngine(GemmFamily::makePattern().getKey());
    CHECK(engine != nullptr);
    // A user pattern built in another order finds the same engine.
    PatternBuilder builder;
    const std::uint64_t d     = builder.addOperand(OperandKind::kTensor);
    const std::uint64_t beta  = builder.addOperand(OperandKind::kTensor);
    const std::uint64_t a     = builder.addOperand(OperandKind::kTensor);
    const std::uint64_t alpha = builder.addOperand(OperandKind::kTensor);
    const std::uint64_t c     = builder.addOperand(OperandKind::kTensor);
    const std::uint64_t b     = builder.addOperand(OperandKind::kTensor);
    builder.addOperation(OperationKind::kGemm, {a, b, c, alpha, beta}, {d});
    CHECK(handle.findOpsEngine(builder.build().getKey()) == engine);
    CHECK(handle.findOpsEngine(PatternBuilder().build().getKey()) == nullptr);
    CHECK_THROWS_STATUS(handle.registerOpsEngine(nullptr), FTRAIN_STATUS_INVALID_ARGUMENT);
    CHECK_THROWS_STATUS(handle.registerOpsEngine(makeBuiltinOpsEngines().front()), FTRAIN_STATUS_INVALID_ARGUMENT);
    CHECK_EQ(GemmFamily::makeRecords().size(), static_cast<std::size_t>(6));
    CHECK_EQ(std::string(GemmFamily::makeRecords().front()->getName()), std::string("Fp32Gemm"));
}
