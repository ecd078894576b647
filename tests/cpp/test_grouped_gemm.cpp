// The GroupedABCDGemm family on the fake platform: decoding and validation of the per-group
// metadata (GroupedTensor contract of the public header: element (i, j) of group g lies at
// offsets[g] + i * strides[0][g] + j * strides[1][g]), the Primitives' support checklist, selection,
// and what reaches the platform's grouped entry points through the public C API.
#include <cstring>
#include <string>
#include <vector>

#include "core/handle.hpp"
#include "fake_platform.hpp"
#include "family/grouped_gemm/family.hpp"
#include "flash_train/flash_train.h"
#include "mini_test.hpp"
#include "primitive/cuda/gemm/cuda_grouped_gemm.hpp"

using namespace ftrain;

namespace {

float g_alpha = 2.0F;
float g_beta  = -0.5F;

void* address(std::uintptr_t value) { return reinterpret_cast<void*>(value); }

// Host arrays behind one grouped operand; must outlive the views made from them.
struct GroupedSpec {
    void* data;
    std::vector<std::int64_t> rows, cols;
    std::vector<std::int64_t> offsets;  // empty: dense packing (GROUPED_CONTINUOUS)
    std::vector<std::int64_t> row_strides, col_strides;  // empty: dense row-major groups
    FTrainNumericType meta_type = FTRAIN_NUMERIC_TYPE_INT64;
    bool meta_on_host           = true;
    FTrainNumericType data_type = FTRAIN_NUMERIC_TYPE_FP32;

    FTrainStorageView vector(const std::vector<std::int64_t>& values, const std::int64_t* length) const {
        return FTrainStorageView{const_cast<std::int64_t*>(values.data()), length, nullptr, 1, meta_type, FTRAIN_INDEX_TYPE_CONTINUOUS,
                                 meta_on_host};
    }
};

GroupedTensor grouped(const GroupedSpec& spec) {
    const std::int64_t count    = static_cast<std::int64_t>(spec.rows.size());
    const std::int64_t whole[2] = {0, 0};  // per-group extents come from dim_sizes, not from data.dims
    StorageView data(FTrainStorageView{spec.data, whole, nullptr, 2, spec.data_type, FTRAIN_INDEX_TYPE_GROUPED_CONTINUOUS, false});
    std::optional<StorageView> offsets;
    if (!spec.offsets.empty()) { offsets.emplace(spec.vector(spec.offsets, &count)); }
    std::vector<StorageView> dims, strides;
    dims.emplace_back(spec.vector(spec.rows, &count));
    dims.emplace_back(spec.vector(spec.cols, &count));
    if (!spec.row_strides.empty()) {
        strides.emplace_back(spec.vector(spec.row_strides, &count));
        strides.emplace_back(spec.vector(spec.col_strides, &count));
    }
    return GroupedTensor(static_cast<std::uint32_t>(count), std::move(data), std::move(offsets), std::move(dims), std::move(strides));
}

Tensor scalar(float* value, bool host = true) {
    return Tensor(StorageView(FTrainStorageView{value, nullptr, nullptr, 0, FTRAIN_NUMERIC_TYPE_FP32, FTRAIN_INDEX_TYPE_CONTINUOUS, host}));
}

// Three groups, the middle one empty: m = {256, 0, 130}, k = {512, 512, 260}, n = {384, 384, 200}.
struct Ragged {
    GroupedSpec a{address(0x100000), {256, 0, 130}, {512, 512, 260}};
    GroupedSpec b{address(0x900000), {512, 512, 260}, {384, 384, 200}};
    GroupedSpec c{address(0x1100000), {256, 0, 130}, {384, 384, 200}};
    GroupedSpec d{address(0x1900000), {256, 0, 130}, {384, 384, 200}};
    GroupedGemmProblem problem(FTrainNumericType compute = FTRAIN_NUMERIC_TYPE_FP32) {
        return GroupedGemmProblem(OperandValue(grouped(a)), OperandValue(grouped(b)), OperandValue(grouped(c)), OperandValue(grouped(d)),
                                  scalar(&g_alpha), scalar(&g_beta), compute);
    }
};

}  // namespace

TEST(grouped_problem_decodes_dense_and_explicit_layouts) {
    Ragged ragged;
    const GroupedGemmProblem dense = ragged.problem();
    CHECK_EQ(dense.getNumGroups(), std::uint32_t{3});
    CHECK(!dense.hasEmptyOutput() && !dense.isInPlace());
    // Dense packing: group 2 of a starts after 256 * 512 + 0 * 512 elements, rows of 260.
    CHECK_EQ(dense.getGroup(GroupedPort::kA, 2).offset, std::int64_t{256 * 512});
    CHECK_EQ(dense.getGroup(GroupedPort::kA, 2).row_stride, std::int64_t{260});
    CHECK_EQ(dense.getGroup(GroupedPort::kA, 2).col_stride, std::int64_t{1});
    CHECK_EQ(dense.getGroup(GroupedPort::kB, 1).offset, std::int64_t{512 * 384});
    // Explicit offsets and strides (here: b's groups stored transposed, with padded pitches) are taken as given.
    ragged.b.offsets     = {0, 400000, 800000};
    ragged.b.row_strides = {1, 1, 1};
    ragged.b.col_strides = {512, 512, 264};
    const GroupedGemmProblem strided = ragged.problem();
    CHECK_EQ(strided.getGroup(GroupedPort::kB, 2).offset, std::int64_t{800000});
    CHECK_EQ(strided.getGroup(GroupedPort::kB, 2).col_stride, std::int64_t{264});
    CHECK(dense.getProblemKey() != strided.getProblemKey());
    // 32-bit metadata decodes the same way.
    std::vector<std::int32_t> rows32 = {256, 0, 130}, cols32 = {512, 512, 260};
    const std::int64_t count = 3, whole[2] = {0, 0};
    std::vector<StorageView> dims32;
    dims32.emplace_back(FTrainStorageView{rows32.data(), &count, nullptr, 1, FTRAIN_NUMERIC_TYPE_INT32, FTRAIN_INDEX_TYPE_CONTINUOUS, true});
    dims32.emplace_back(FTrainStorageView{cols32.data(), &count, nullptr, 1, FTRAIN_NUMERIC_TYPE_INT32, FTRAIN_INDEX_TYPE_CONTINUOUS, true});
    GroupedTensor a32(3, StorageView(FTrainStorageView{address(0x100000), whole, nullptr, 2, FTRAIN_NUMERIC_TYPE_FP32,
                                                       FTRAIN_INDEX_TYPE_GROUPED_CONTINUOUS, false}),
                      std::nullopt, std::move(dims32), {});
    Ragged other;
    const GroupedGemmProblem mixed(OperandValue(std::move(a32)), OperandValue(grouped(other.b)), OperandValue(grouped(other.c)),
                                   OperandValue(grouped(other.d)), scalar(&g_alpha), scalar(&g_beta), FTRAIN_NUMERIC_TYPE_FP32);
    CHECK_EQ(mixed.getGroup(GroupedPort::kA, 2).offset, std::int64_t{256 * 512});
    CHECK(mixed.getProblemKey() == dense.getProblemKey());
    // c and d on the same memory with the same offsets: in place.
    Ragged in_place;
    in_place.c.data = in_place.d.data;
    CHECK(in_place.problem().isInPlace());
}

TEST(grouped_problem_validation_statuses) {
    {
        Ragged r;
        r.b.rows = {512, 512, 261};  // a's columns != b's rows in group 2
        CHECK_THROWS_STATUS(r.problem(), FTRAIN_STATUS_INVALID_ARGUMENT);
    }
    {
        Ragged r;
        r.d.cols = {384, 384, 201};
        CHECK_THROWS_STATUS(r.problem(), FTRAIN_STATUS_INVALID_ARGUMENT);
    }
    {
        Ragged r;
        r.c.rows = {256, 0};  // another number of groups
        r.c.cols = {384, 384};
        CHECK_THROWS_STATUS(r.problem(), FTRAIN_STATUS_INVALID_ARGUMENT);
    }
    {
        Ragged r;
        r.a.rows = {256, -1, 130};
        CHECK_THROWS_STATUS(r.problem(), FTRAIN_STATUS_INVALID_ARGUMENT);
    }
    {
        Ragged r;
        r.a.meta_on_host = false;  // metadata on the device: nothing here can read it
        CHECK_THROWS_STATUS(r.problem(), FTRAIN_STATUS_UNSUPPORTED);
    }
    {
        Ragged r;
        r.a.meta_type = FTRAIN_NUMERIC_TYPE_FP32;
        CHECK_THROWS_STATUS(r.problem(), FTRAIN_STATUS_UNSUPPORTED);
    }
    {
        Ragged r;
        const std::int64_t huge = std::int64_t{1} << 62;
        r.a.rows = {huge, 0, 130};
        r.a.cols = {huge, 512, 260};
        r.b.rows = {huge, 512, 260};
        r.c.rows = r.d.rows = {huge, 0, 130};
        CHECK_THROWS_STATUS(r.problem(), FTRAIN_STATUS_OVERFLOW);
    }
    {
        Ragged r;  // alpha in device memory
        CHECK_THROWS_STATUS(GroupedGemmProblem(OperandValue(grouped(r.a)), OperandValue(grouped(r.b)), OperandValue(grouped(r.c)),
                                               OperandValue(grouped(r.d)), scalar(&g_alpha, false), scalar(&g_beta), FTRAIN_NUMERIC_TYPE_FP32),
                            FTRAIN_STATUS_INVALID_ARGUMENT);
    }
}

TEST(grouped_checklist_and_descriptors) {
    fake::reset();
    Ragged ragged;
    const GroupedGemmProblem problem = ragged.problem();
    const Constraints constraints{0};
    const CudaGroupedGemm exact(FTCUDA_GROUPED_GEMM_EXACT), tensor(FTCUDA_GROUPED_GEMM_TF32X3);
    CHECK_EQ(std::string(exact.getName()), std::string("GroupedFp32Gemm"));
    CHECK_EQ(std::string(tensor.getName()), std::string("GroupedFp32Gemm3xTf32"));
    CHECK(exact.isApplicable(problem, constraints).isSuccess());
    CHECK(tensor.isApplicable(problem, constraints).isSuccess());
    CHECK(!exact.isApplicable(ragged.problem(FTRAIN_NUMERIC_TYPE_FP64), constraints).isSuccess());
    Ragged half;
    half.a.data_type = FTRAIN_NUMERIC_TYPE_FP16;
    CHECK(std::strstr(exact.isApplicable(half.problem(), constraints).getMessage(), "an operand is not fp32") != nullptr);
    Ragged headless;
    headless.a.data = nullptr;
    CHECK(std::strstr(exact.isApplicable(headless.problem(), constraints).getMessage(), "a required operand address is null") != nullptr);
    Ragged no_addend;  // c without memory is fine: no beta * C term
    no_addend.c.data = nullptr;
    CHECK(exact.isApplicable(no_addend.problem(), constraints).isSuccess());
    Ragged shallow;  // one group too shallow for the split-precision kernel: the exact Primitive still applies
    shallow.a.cols = {512, 512, 64};
    shallow.b.rows = {512, 512, 64};
    CHECK(!tensor.isApplicable(shallow.problem(), constraints).isSuccess());
    CHECK(exact.isApplicable(shallow.problem(), constraints).isSuccess());

    const std::vector<FtcudaGemmDesc> descs = makeCudaGroupedDescs(problem, 0, true);
    CHECK_EQ(descs.size(), std::size_t{3});
    CHECK(descs[2].a == static_cast<const float*>(address(0x100000)) + 256 * 512);
    CHECK_EQ(descs[2].m, std::uint64_t{130});
    CHECK_EQ(descs[2].k, std::uint64_t{260});
    CHECK_EQ(descs[2].n, std::uint64_t{200});
    CHECK_EQ(descs[2].d_row_stride, std::int64_t{200});
    CHECK_EQ(descs[1].m, std::uint64_t{0});
    CHECK_EQ(descs[0].alpha, 2.0F);
    CHECK_EQ(descs[0].beta, -0.5F);
}

TEST(grouped_engine_is_registered_and_selects_best_first) {
    fake::reset();
    const auto engine = getGlobalHandle().findOpsEngine(GroupedGemmFamily::getRoles().pattern.getKey());
    CHECK(engine != nullptr);
    CHECK(getGlobalHandle().findOpsEngine(GroupedBcdGemmFamily::getRoles().pattern.getKey()) != nullptr);
    CHECK(getGlobalHandle().findOpsEngine(GroupedAbGemmFamily::getRoles().pattern.getKey()) != nullptr);
    CHECK_EQ(getGlobalHandle().getNumOpsEngines(), std::size_t{4});
}

// Through the public C API: Pattern with the roles in a foreign order -> Ops -> Args -> Plan -> execute.
TEST(grouped_gemm_through_the_c_api) {
    fake::reset();
    FTrainPattern pattern = nullptr;
    CHECK_EQ(static_cast<int>(ftrainPatternCreate(&pattern)), 0);
    FTrainGroupedTensorId d, b, a, c;
    FTrainTensorId beta, alpha;
    ftrainPatternAddGroupedTensor(pattern, &d);
    ftrainPatternAddTensor(pattern, &beta);
    ftrainPatternAddGroupedTensor(pattern, &b);
    ftrainPatternAddGroupedTensor(pattern, &a);
    ftrainPatternAddTensor(pattern, &alpha);
    ftrainPatternAddGroupedTensor(pattern, &c);
    FTrainGroupedABCDGemmOpId op;
    CHECK_EQ(static_cast<int>(ftrainPatternAddGroupedABCDGemm(pattern, &op, a, b, c, d, alpha, beta)), 0);
    FTrainOps ops = nullptr;
    CHECK_EQ(static_cast<int>(ftrainOpsCreate(&ops, pattern)), 0);
    ftrainPatternDestroy(pattern);
    FTrainArgs args = nullptr;
    CHECK_EQ(static_cast<int>(ftrainArgsCreate(&args, ops)), 0);

    Ragged ragged;
    const std::int64_t count = 3, whole[2] = {0, 0};
    const auto set = [&](FTrainGroupedTensorId role, const GroupedSpec& spec) {
        const FTrainStorageView data{spec.data, whole, nullptr, 2, FTRAIN_NUMERIC_TYPE_FP32, FTRAIN_INDEX_TYPE_GROUPED_CONTINUOUS, false};
        const FTrainStorageView dims[2] = {spec.vector(spec.rows, &count), spec.vector(spec.cols, &count)};
        return ftrainArgsSetGroupedTensor(args, role, 3, data, nullptr, dims, nullptr);
    };
    CHECK_EQ(static_cast<int>(set(a, ragged.a)), 0);
    CHECK_EQ(static_cast<int>(set(b, ragged.b)), 0);
    CHECK_EQ(static_cast<int>(set(c, ragged.c)), 0);
    CHECK_EQ(static_cast<int>(set(d, ragged.d)), 0);
    const FTrainStorageView alpha_view{&g_alpha, nullptr, nullptr, 0, FTRAIN_NUMERIC_TYPE_FP32, FTRAIN_INDEX_TYPE_CONTINUOUS, true};
    const FTrainStorageView beta_view{&g_beta, nullptr, nullptr, 0, FTRAIN_NUMERIC_TYPE_FP32, FTRAIN_INDEX_TYPE_CONTINUOUS, true};
    CHECK_EQ(static_cast<int>(ftrainArgsSetTensor(args, alpha, alpha_view)), 0);
    CHECK_EQ(static_cast<int>(ftrainArgsSetTensor(args, beta, beta_view)), 0);
    // Incomplete until the operation's compute type is set.
    FTrainPlan plan = nullptr;
    CHECK_EQ(static_cast<int>(ftrainPlanCreate(&plan, args)), static_cast<int>(FTRAIN_STATUS_INVALID_ARGUMENT));
    CHECK_EQ(static_cast<int>(ftrainArgsSetGroupedABCDGemm(args, op, FTRAIN_NUMERIC_TYPE_FP32)), 0);
    CHECK_EQ(static_cast<int>(ftrainPlanCreate(&plan, args)), 0);

    std::uint64_t primitives = 0;
    CHECK_EQ(static_cast<int>(ftrainPlanGetNumPrimitives(plan, &primitives)), 0);
    CHECK_EQ(primitives, std::uint64_t{2});
    const char* name = nullptr;
    ftrainPlanGetPrimitiveName(plan, 0, &name);
    CHECK_EQ(std::string(name), std::string("GroupedFp32Gemm3xTf32"));
    ftrainPlanGetPrimitiveName(plan, 1, &name);
    CHECK_EQ(std::string(name), std::string("GroupedFp32Gemm"));
    std::uint64_t bytes = 0;
    ftrainPlanGetPrimitiveRequiredWorkspaceBytes(plan, 0, &bytes);
    CHECK_EQ(bytes, std::uint64_t{1024});
    ftrainPlanGetPrimitiveRequiredWorkspaceBytes(plan, 1, &bytes);
    CHECK_EQ(bytes, std::uint64_t{0});

    // Primitive 0 refuses to run without its workspace; with it, one grouped launch reaches the platform.
    CHECK_EQ(static_cast<int>(ftrainPlanExecutePrimitive(plan, 0, nullptr, 0, nullptr)), static_cast<int>(FTRAIN_STATUS_INVALID_ARGUMENT));
    CHECK_EQ(fake::state().grouped_launches.size(), std::size_t{0});
    char workspace[8];
    CHECK_EQ(static_cast<int>(ftrainPlanExecutePrimitive(plan, 0, workspace, 4096, reinterpret_cast<FTrainStream>(address(0x77)))), 0);
    CHECK_EQ(fake::state().grouped_launches.size(), std::size_t{1});
    const fake::GroupedLaunchRecord& launched = fake::state().grouped_launches.back();
    CHECK_EQ(launched.kernel, static_cast<int>(FTCUDA_GROUPED_GEMM_TF32X3));
    CHECK(launched.workspace == workspace && launched.stream == address(0x77));
    CHECK_EQ(launched.groups.size(), std::size_t{3});
    CHECK_EQ(launched.groups[2].m, std::uint64_t{130});
    CHECK_EQ(launched.groups[0].alpha, 2.0F);
    CHECK_EQ(static_cast<int>(ftrainPlanExecutePrimitive(plan, 1, nullptr, 0, nullptr)), 0);
    CHECK_EQ(fake::state().grouped_launches.back().kernel, static_cast<int>(FTCUDA_GROUPED_GEMM_EXACT));

    // An equal description is a cache hit: same order, nothing asked of the platform's support check again.
    const int supports_before = fake::state().supports;
    FTrainPlan again = nullptr;
    CHECK_EQ(static_cast<int>(ftrainPlanCreate(&again, args)), 0);
    CHECK_EQ(fake::state().supports, supports_before);
    CHECK(again != plan);
    // A launch failure is INTERNAL_ERROR with the platform's reason.
    fake::state().fail_next_launch = "too many resources requested for launch (injected)";
    CHECK_EQ(static_cast<int>(ftrainPlanExecutePrimitive(again, 1, nullptr, 0, nullptr)), static_cast<int>(FTRAIN_STATUS_INTERNAL_ERROR));
    CHECK(std::strstr(ftrainGetLastMessage(), "too many resources requested for launch (injected)") != nullptr);

    // Every configured launch is released with its Plan.
    CHECK(fake::state().grouped_live > 0);
    ftrainPlanDestroy(again);
    ftrainPlanDestroy(plan);
    CHECK_EQ(fake::state().grouped_live, 0);
    ftrainArgsDestroy(args);
    ftrainOpsDestroy(ops);
    fake::reset();
}

TEST(grouped_gemm_with_only_empty_groups_plans_and_runs_nothing) {
    fake::reset();
    Ragged ragged;
    ragged.a.rows = ragged.c.rows = ragged.d.rows = {0, 0, 0};
    const GroupedGemmProblem problem = ragged.problem();
    CHECK(problem.hasEmptyOutput());
    CudaGroupedGemm exact(FTCUDA_GROUPED_GEMM_EXACT);
    CHECK(exact.isApplicable(problem, Constraints{0}).isSuccess());
    exact.configure(problem);
    CHECK_EQ(exact.getRequiredWorkspaceBytes(), std::uint64_t{0});
    exact.execute(Resources(nullptr, 0, nullptr));
    CHECK_EQ(fake::state().grouped_launches.size(), std::size_t{0});
    fake::reset();
}

// GroupedBCDGemm (a is a TensorList) and GroupedABGemm (c and d are TensorLists): a list's g-th view is group g,
// an ordinary matrix view with its own address, extents and (optional) strides.
TEST(grouped_problem_takes_tensor_lists) {
    Ragged ragged;
    const std::int64_t dims[3][2]  = {{256, 512}, {0, 512}, {130, 260}};
    const std::int64_t pitch[2]    = {264, 1};  // group 2 of a lives in a wider buffer
    std::vector<StorageView> a_views;
    a_views.emplace_back(FTrainStorageView{address(0x100000), dims[0], nullptr, 2, FTRAIN_NUMERIC_TYPE_FP32, FTRAIN_INDEX_TYPE_CONTINUOUS, false});
    a_views.emplace_back(FTrainStorageView{nullptr, dims[1], nullptr, 2, FTRAIN_NUMERIC_TYPE_FP32, FTRAIN_INDEX_TYPE_CONTINUOUS, false});
    a_views.emplace_back(FTrainStorageView{address(0x300010), dims[2], pitch, 2, FTRAIN_NUMERIC_TYPE_FP32, FTRAIN_INDEX_TYPE_INVALID, false});
    const GroupedGemmProblem bcd(OperandValue(TensorList(std::vector<StorageView>(a_views))), OperandValue(grouped(ragged.b)),
                                 OperandValue(grouped(ragged.c)), OperandValue(grouped(ragged.d)), scalar(&g_alpha), scalar(&g_beta),
                                 FTRAIN_NUMERIC_TYPE_FP32);
    CHECK(bcd.getOperand(GroupedPort::kA).is_list && !bcd.getOperand(GroupedPort::kB).is_list);
    CHECK(bcd.getGroup(GroupedPort::kA, 2).address() == static_cast<const float*>(address(0x300010)));
    CHECK_EQ(bcd.getGroup(GroupedPort::kA, 2).row_stride, std::int64_t{264});
    CHECK_EQ(bcd.getGroup(GroupedPort::kA, 0).row_stride, std::int64_t{512});
    const CudaGroupedGemm exact(FTCUDA_GROUPED_GEMM_EXACT);
    CHECK(exact.isApplicable(bcd, Constraints{0}).isSuccess());  // the empty group's a needs no address
    const std::vector<FtcudaGemmDesc> descs = makeCudaGroupedDescs(bcd, 0, true);
    CHECK(descs[2].a == static_cast<const float*>(address(0x300010)));
    CHECK_EQ(descs[2].a_row_stride, std::int64_t{264});
    // Another list length than the other operands' group count: contradictory.
    a_views.pop_back();
    CHECK_THROWS_STATUS(GroupedGemmProblem(OperandValue(TensorList(std::move(a_views))), OperandValue(grouped(ragged.b)),
                                           OperandValue(grouped(ragged.c)), OperandValue(grouped(ragged.d)), scalar(&g_alpha), scalar(&g_beta),
                                           FTRAIN_NUMERIC_TYPE_FP32),
                        FTRAIN_STATUS_INVALID_ARGUMENT);
    // A list mixing numeric types is not something a Primitive takes.
    const std::int64_t cd_dims[3][2] = {{256, 384}, {0, 384}, {130, 200}};
    std::vector<StorageView> c_views, d_views;
    for (int g = 0; g < 3; ++g) {
        c_views.emplace_back(FTrainStorageView{address(0x1100000 + 0x100000 * g), cd_dims[g], nullptr, 2,
                                               g == 1 ? FTRAIN_NUMERIC_TYPE_FP16 : FTRAIN_NUMERIC_TYPE_FP32, FTRAIN_INDEX_TYPE_CONTINUOUS, false});
        d_views.emplace_back(FTrainStorageView{address(0x1900000 + 0x100000 * g), cd_dims[g], nullptr, 2, FTRAIN_NUMERIC_TYPE_FP32,
                                               FTRAIN_INDEX_TYPE_CONTINUOUS, false});
    }
    const GroupedGemmProblem ab(OperandValue(grouped(ragged.a)), OperandValue(grouped(ragged.b)), OperandValue(TensorList(std::move(c_views))),
                                OperandValue(TensorList(std::move(d_views))), scalar(&g_alpha), scalar(&g_beta), FTRAIN_NUMERIC_TYPE_FP32);
    CHECK(std::strstr(exact.isApplicable(ab, Constraints{0}).getMessage(), "an operand is not fp32") != nullptr);
    // A plain Tensor where a grouped operand belongs.
    CHECK_THROWS_STATUS(GroupedGemmProblem(OperandValue(scalar(&g_alpha)), OperandValue(grouped(ragged.b)), OperandValue(grouped(ragged.c)),
                                           OperandValue(grouped(ragged.d)), scalar(&g_alpha), scalar(&g_beta), FTRAIN_NUMERIC_TYPE_FP32),
                        FTRAIN_STATUS_INVALID_ARGUMENT);
}

TEST(grouped_ab_gemm_through_the_c_api) {
    fake::reset();
    FTrainPattern pattern = nullptr;
    CHECK_EQ(static_cast<int>(ftrainPatternCreate(&pattern)), 0);
    FTrainGroupedTensorId a, b;
    FTrainTensorListId c, d;
    FTrainTensorId alpha, beta;
    ftrainPatternAddTensorList(pattern, &d);
    ftrainPatternAddGroupedTensor(pattern, &a);
    ftrainPatternAddTensor(pattern, &alpha);
    ftrainPatternAddTensorList(pattern, &c);
    ftrainPatternAddGroupedTensor(pattern, &b);
    ftrainPatternAddTensor(pattern, &beta);
    FTrainGroupedABGemmOpId op;
    CHECK_EQ(static_cast<int>(ftrainPatternAddGroupedABGemm(pattern, &op, a, b, c, d, alpha, beta)), 0);
    FTrainOps ops = nullptr;
    CHECK_EQ(static_cast<int>(ftrainOpsCreate(&ops, pattern)), 0);
    ftrainPatternDestroy(pattern);
    FTrainArgs args = nullptr;
    CHECK_EQ(static_cast<int>(ftrainArgsCreate(&args, ops)), 0);
    Ragged ragged;
    const std::int64_t count = 3, whole[2] = {0, 0};
    const auto set = [&](FTrainGroupedTensorId role, const GroupedSpec& spec) {
        const FTrainStorageView data{spec.data, whole, nullptr, 2, FTRAIN_NUMERIC_TYPE_FP32, FTRAIN_INDEX_TYPE_GROUPED_CONTINUOUS, false};
        const FTrainStorageView dims[2] = {spec.vector(spec.rows, &count), spec.vector(spec.cols, &count)};
        return ftrainArgsSetGroupedTensor(args, role, 3, data, nullptr, dims, nullptr);
    };
    CHECK_EQ(static_cast<int>(set(a, ragged.a)), 0);
    CHECK_EQ(static_cast<int>(set(b, ragged.b)), 0);
    const std::int64_t cd_dims[3][2] = {{256, 384}, {0, 384}, {130, 200}};
    FTrainStorageView c_views[3], d_views[3];
    for (int g = 0; g < 3; ++g) {
        c_views[g] = FTrainStorageView{g == 2 ? nullptr : address(0x1100000 + 0x100000 * g), cd_dims[g], nullptr, 2, FTRAIN_NUMERIC_TYPE_FP32,
                                       FTRAIN_INDEX_TYPE_CONTINUOUS, false};  // group 2 has no addend
        d_views[g] = FTrainStorageView{address(0x1900000 + 0x100000 * g), cd_dims[g], nullptr, 2, FTRAIN_NUMERIC_TYPE_FP32,
                                       FTRAIN_INDEX_TYPE_CONTINUOUS, false};
    }
    CHECK_EQ(static_cast<int>(ftrainArgsSetTensorList(args, c, c_views, 3)), 0);
    CHECK_EQ(static_cast<int>(ftrainArgsSetTensorList(args, d, d_views, 3)), 0);
    const FTrainStorageView alpha_view{&g_alpha, nullptr, nullptr, 0, FTRAIN_NUMERIC_TYPE_FP32, FTRAIN_INDEX_TYPE_CONTINUOUS, true};
    const FTrainStorageView beta_view{&g_beta, nullptr, nullptr, 0, FTRAIN_NUMERIC_TYPE_FP32, FTRAIN_INDEX_TYPE_CONTINUOUS, true};
    CHECK_EQ(static_cast<int>(ftrainArgsSetTensor(args, alpha, alpha_view)), 0);
    CHECK_EQ(static_cast<int>(ftrainArgsSetTensor(args, beta, beta_view)), 0);
    // The other operations' setters do not fit this role.
    CHECK_EQ(static_cast<int>(ftrainArgsSetGroupedABCDGemm(args, FTrainGroupedABCDGemmOpId{op.opaque}, FTRAIN_NUMERIC_TYPE_FP32)),
             static_cast<int>(FTRAIN_STATUS_INVALID_ARGUMENT));
    CHECK_EQ(static_cast<int>(ftrainArgsSetGroupedABGemm(args, op, FTRAIN_NUMERIC_TYPE_FP32)), 0);
    FTrainPlan plan = nullptr;
    CHECK_EQ(static_cast<int>(ftrainPlanCreate(&plan, args)), 0);
    const char* name = nullptr;
    ftrainPlanGetPrimitiveName(plan, 0, &name);
    CHECK_EQ(std::string(name), std::string("GroupedFp32Gemm3xTf32"));
    char workspace[8];
    CHECK_EQ(static_cast<int>(ftrainPlanExecutePrimitive(plan, 0, workspace, 4096, nullptr)), 0);
    const fake::GroupedLaunchRecord& launched = fake::state().grouped_launches.back();
    CHECK(launched.groups[0].c == static_cast<const float*>(address(0x1100000)));
    CHECK(launched.groups[2].c == nullptr);
    CHECK(launched.groups[2].d == static_cast<float*>(address(0x1b00000)));
    CHECK_EQ(launched.groups[2].d_row_stride, std::int64_t{200});
    ftrainPlanDestroy(plan);
    ftrainArgsDestroy(args);
    ftrainOpsDestroy(ops);
    fake::reset();
}
