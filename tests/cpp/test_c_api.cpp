// The extern "C" surface, black box, on the fake platform.
// Behaviours pinned by the reference's tests/api/pattern_api_test.cpp:64-228,
// tests/api/common_api_test.cpp:25-150 and tests/api/runtime_api_test.cpp:430-741.
#include <cstring>
#include <string>
#include <thread>

#include "fake_platform.hpp"
#include "flash_train/flash_train.h"
#include "mini_test.hpp"

namespace {

struct GemmGraph {
    FTrainPattern pattern = nullptr;
    FTrainTensorId a, b, c, d, alpha, beta;
    FTrainGemmOpId op;
};

// Roles are added in the order d, beta, a, alpha, c, b (not the library's own).
GemmGraph makeGraph() {
    GemmGraph g;
    CHECK_EQ(static_cast<int>(ftrainPatternCreate(&g.pattern)), 0);
    ftrainPatternAddTensor(g.pattern, &g.d);
    ftrainPatternAddTensor(g.pattern, &g.beta);
    ftrainPatternAddTensor(g.pattern, &g.a);
    ftrainPatternAddTensor(g.pattern, &g.alpha);
    ftrainPatternAddTensor(g.pattern, &g.c);
    ftrainPatternAddTensor(g.pattern, &g.b);
    CHECK_EQ(static_cast<int>(ftrainPatternAddGemm(g.pattern, &g.op, g.a, g.b, g.c, g.d, g.alpha, g.beta)), 0);
    return g;
}

FTrainStorageView matrix(void* memory, const std::int64_t* dims) {
    return FTrainStorageView{memory, dims, nullptr, 2, FTRAIN_NUMERIC_TYPE_FP32, FTRAIN_INDEX_TYPE_CONTINUOUS, false};
}

FTrainStorageView scalar(float* value) {
    return FTrainStorageView{value, nullptr, nullptr, 0, FTRAIN_NUMERIC_TYPE_FP32, FTRAIN_INDEX_TYPE_CONTINUOUS, true};
}

void* address(std::uintptr_t value) { return reinterpret_cast<void*>(value); }

}  // namespace

TEST(role_ids_count_from_zero) {
    GemmGraph g = makeGraph();
    CHECK_EQ(g.d.opaque, std::uint64_t{0});
    CHECK_EQ(g.b.opaque, std::uint64_t{5});
    CHECK_EQ(g.op.opaque, std::uint64_t{0});
    FTrainTensorListId list;
    FTrainGroupedTensorId grouped;
    CHECK_EQ(static_cast<int>(ftrainPatternAddTensorList(g.pattern, &list)), 0);
    CHECK_EQ(static_cast<int>(ftrainPatternAddGroupedTensor(g.pattern, &grouped)), 0);
    CHECK_EQ(list.opaque, std::uint64_t{6});
    CHECK_EQ(grouped.opaque, std::uint64_t{7});
    ftrainPatternDestroy(g.pattern);
}

TEST(null_arguments_are_invalid_and_outputs_stay_untouched) {
    FTrainPattern pattern = reinterpret_cast<FTrainPattern>(0x1);
    CHECK_EQ(static_cast<int>(ftrainPatternCreate(nullptr)), static_cast<int>(FTRAIN_STATUS_INVALID_ARGUMENT));
    CHECK(std::strstr(ftrainGetLastMessage(), "ftrainPatternCreate") != nullptr);
    FTrainTensorId tensor{77};
    CHECK_EQ(static_cast<int>(ftrainPatternAddTensor(nullptr, &tensor)), static_cast<int>(FTRAIN_STATUS_INVALID_ARGUMENT));
    CHECK_EQ(tensor.opaque, std::uint64_t{77});
    CHECK_EQ(static_cast<int>(ftrainPatternDestroy(nullptr)), static_cast<int>(FTRAIN_STATUS_INVALID_ARGUMENT));
    FTrainOps ops = reinterpret_cast<FTrainOps>(0x2);
    CHECK_EQ(static_cast<int>(ftrainOpsCreate(&ops, nullptr)), static_cast<int>(FTRAIN_STATUS_INVALID_ARGUMENT));
    CHECK(ops == reinterpret_cast<FTrainOps>(0x2));
    CHECK_EQ(static_cast<int>(ftrainOpsDestroy(nullptr)), static_cast<int>(FTRAIN_STATUS_INVALID_ARGUMENT));
    FTrainArgs args = reinterpret_cast<FTrainArgs>(0x3);
    CHECK_EQ(static_cast<int>(ftrainArgsCreate(&args, nullptr)), static_cast<int>(FTRAIN_STATUS_INVALID_ARGUMENT));
    CHECK(args == reinterpret_cast<FTrainArgs>(0x3));
    CHECK_EQ(static_cast<int>(ftrainArgsDestroy(nullptr)), static_cast<int>(FTRAIN_STATUS_INVALID_ARGUMENT));
    FTrainPlan plan = reinterpret_cast<FTrainPlan>(0x4);
    CHECK_EQ(static_cast<int>(ftrainPlanCreate(&plan, nullptr)), static_cast<int>(FTRAIN_STATUS_INVALID_ARGUMENT));
    CHECK(plan == reinterpret_cast<FTrainPlan>(0x4));
    CHECK_EQ(static_cast<int>(ftrainPlanDestroy(nullptr)), static_cast<int>(FTRAIN_STATUS_INVALID_ARGUMENT));
    std::uint64_t count = 5;
    CHECK_EQ(static_cast<int>(ftrainPlanGetNumPrimitives(nullptr, &count)), static_cast<int>(FTRAIN_STATUS_INVALID_ARGUMENT));
    CHECK_EQ(count, std::uint64_t{5});
    CHECK_EQ(static_cast<int>(ftrainPlanExecutePrimitive(nullptr, 0, nullptr, 0, nullptr)), static_cast<int>(FTRAIN_STATUS_INVALID_ARGUMENT));
    (void)pattern;
}

TEST(ops_create_validates_and_matches) {
    // Wiring is only checked here, not when nodes are added.
    FTrainPattern bad = nullptr;
    ftrainPatternCreate(&bad);
    FTrainTensorId t[6];
    for (auto& id : t) { ftrainPatternAddTensor(bad, &id); }
    FTrainGemmOpId op;
    CHECK_EQ(static_cast<int>(ftrainPatternAddGemm(bad, &op, t[0], t[0], t[2], t[5], t[3], t[4])), 0);  // duplicate accepted
    FTrainOps ops = nullptr;
    CHECK_EQ(static_cast<int>(ftrainOpsCreate(&ops, bad)), static_cast<int>(FTRAIN_STATUS_INVALID_ARGUMENT));
    CHECK(ops == nullptr);
    ftrainPatternDestroy(bad);
    // A graph no engine supports (two Gemm nodes chained through one matrix): UNSUPPORTED, the caller's
    // variable unchanged.
    FTrainPattern unsupported = nullptr;
    ftrainPatternCreate(&unsupported);
    FTrainTensorId n[10];
    for (auto& id : n) { ftrainPatternAddTensor(unsupported, &id); }
    FTrainGemmOpId first_op, second_op;
    CHECK_EQ(static_cast<int>(ftrainPatternAddGemm(unsupported, &first_op, n[0], n[1], n[2], n[3], n[4], n[5])), 0);
    CHECK_EQ(static_cast<int>(ftrainPatternAddGemm(unsupported, &second_op, n[3], n[6], n[7], n[8], n[4], n[5])), 0);
    CHECK_EQ(static_cast<int>(ftrainOpsCreate(&ops, unsupported)), static_cast<int>(FTRAIN_STATUS_UNSUPPORTED));
    CHECK(ops == nullptr);
    ftrainPatternDestroy(unsupported);
    // The Gemm graph in a foreign insertion order matches; the Pattern can go right away.
    GemmGraph graph = makeGraph();
    CHECK_EQ(static_cast<int>(ftrainOpsCreate(&ops, graph.pattern)), 0);
    CHECK(ops != nullptr);
    ftrainPatternDestroy(graph.pattern);
    ftrainOpsDestroy(ops);
}

TEST(args_setters_validate_copy_and_replace) {
    fake::reset();
    GemmGraph g = makeGraph();
    FTrainOps ops = nullptr;
    ftrainOpsCreate(&ops, g.pattern);
    FTrainArgs args = nullptr;
    CHECK_EQ(static_cast<int>(ftrainArgsCreate(&args, ops)), 0);
    std::int64_t dims[2] = {4, 3};
    CHECK_EQ(static_cast<int>(ftrainArgsSetTensor(args, g.a, matrix(address(0x1000), dims))), 0);
    dims[0] = 777;  // metadata was copied
    // Wrong storage family for the role, out-of-range ids, invalid compute types.
    FTrainTensorListId as_list{g.a.opaque};
    CHECK_EQ(static_cast<int>(ftrainArgsSetTensorList(args, as_list, nullptr, 0)), static_cast<int>(FTRAIN_STATUS_INVALID_ARGUMENT));
    FTrainTensorId out_of_range{42};
    CHECK_EQ(static_cast<int>(ftrainArgsSetTensor(args, out_of_range, matrix(address(0x1000), dims))), static_cast<int>(FTRAIN_STATUS_INVALID_ARGUMENT));
    CHECK_EQ(static_cast<int>(ftrainArgsSetGemm(args, g.op, FTRAIN_NUMERIC_TYPE_INVALID)), static_cast<int>(FTRAIN_STATUS_INVALID_ARGUMENT));
    CHECK_EQ(static_cast<int>(ftrainArgsSetGemm(args, g.op, FTRAIN_NUMERIC_TYPE_COUNT)), static_cast<int>(FTRAIN_STATUS_INVALID_ARGUMENT));
    FTrainGroupedABGemmOpId other_kind{g.op.opaque};
    CHECK_EQ(static_cast<int>(ftrainArgsSetGroupedABGemm(args, other_kind, FTRAIN_NUMERIC_TYPE_FP32)), static_cast<int>(FTRAIN_STATUS_INVALID_ARGUMENT));
    // An invalid view leaves the previous value in place.
    FTrainStorageView broken = matrix(address(0x1000), nullptr);
    CHECK_EQ(static_cast<int>(ftrainArgsSetTensor(args, g.a, broken)), static_cast<int>(FTRAIN_STATUS_INVALID_ARGUMENT));
    // Incomplete Args cannot be planned.
    FTrainPlan plan = nullptr;
    CHECK_EQ(static_cast<int>(ftrainPlanCreate(&plan, args)), static_cast<int>(FTRAIN_STATUS_INVALID_ARGUMENT));
    CHECK(plan == nullptr);
    // Complete them: the copied dims {4, 3} of `a` are what the Plan sees.
    const std::int64_t b_dims[2] = {3, 5}, d_dims[2] = {4, 5};
    float alpha = 2.0F, beta = 0.5F;
    ftrainArgsSetTensor(args, g.b, matrix(address(0x2000), b_dims));
    ftrainArgsSetTensor(args, g.c, matrix(nullptr, d_dims));
    ftrainArgsSetTensor(args, g.d, matrix(address(0x4000), d_dims));
    ftrainArgsSetTensor(args, g.alpha, scalar(&alpha));
    ftrainArgsSetTensor(args, g.beta, scalar(&beta));
    ftrainArgsSetGemm(args, g.op, FTRAIN_NUMERIC_TYPE_FP32);
    CHECK_EQ(static_cast<int>(ftrainPlanCreate(&plan, args)), 0);
    CHECK(plan != nullptr);
    // The Plan outlives Pattern, Ops and Args.
    ftrainArgsDestroy(args);
    ftrainOpsDestroy(ops);
    ftrainPatternDestroy(g.pattern);
    std::uint64_t count = 0;
    CHECK_EQ(static_cast<int>(ftrainPlanGetNumPrimitives(plan, &count)), 0);
    CHECK(count >= 1);
    const char* name = nullptr;
    CHECK_EQ(static_cast<int>(ftrainPlanGetPrimitiveName(plan, count - 1, &name)), 0);
    CHECK_EQ(std::string(name), std::string("Fp32Gemm"));
    CHECK_EQ(static_cast<int>(ftrainPlanGetPrimitiveName(plan, count, &name)), static_cast<int>(FTRAIN_STATUS_INVALID_ARGUMENT));
    std::uint64_t workspace = 99;
    CHECK_EQ(static_cast<int>(ftrainPlanGetPrimitiveRequiredWorkspaceBytes(plan, 0, &workspace)), 0);
    CHECK_EQ(workspace, std::uint64_t{0});
    CHECK_EQ(static_cast<int>(ftrainPlanExecutePrimitive(plan, 0, nullptr, 0, nullptr)), 0);
    CHECK_EQ(fake::state().launches.size(), static_cast<std::size_t>(1));
    CHECK_EQ(fake::state().launches[0].desc.m, std::uint64_t{4});
    CHECK_EQ(fake::state().launches[0].desc.alpha, 2.0F);
    CHECK(fake::state().launches[0].desc.c == nullptr);
    // A Plan runs only on the device it was created on.
    fake::state().device = 1;
    CHECK_EQ(static_cast<int>(ftrainPlanExecutePrimitive(plan, 0, nullptr, 0, nullptr)), static_cast<int>(FTRAIN_STATUS_INVALID_ARGUMENT));
    CHECK(std::strstr(ftrainGetLastMessage(), "calling thread uses device") != nullptr);
    fake::state().device = 0;
    ftrainPlanDestroy(plan);
    fake::reset();
}

TEST(tensor_list_and_grouped_tensor_setters) {
    // No engine consumes these operand kinds; the setters still have to behave.
    // They are reachable only through an Ops, and no supported graph has such a
    // role, so the family mismatch path is what a caller can observe here.
    GemmGraph g = makeGraph();
    FTrainOps ops = nullptr;
    ftrainOpsCreate(&ops, g.pattern);
    FTrainArgs args = nullptr;
    ftrainArgsCreate(&args, ops);
    float cell = 0;
    const std::int64_t dims[2] = {2, 2};
    FTrainStorageView views[2] = {matrix(&cell, dims), matrix(&cell, dims)};
    FTrainTensorListId list{g.c.opaque};
    CHECK_EQ(static_cast<int>(ftrainArgsSetTensorList(args, list, views, 2)), static_cast<int>(FTRAIN_STATUS_INVALID_ARGUMENT));
    CHECK_EQ(static_cast<int>(ftrainArgsSetTensorList(args, list, nullptr, 2)), static_cast<int>(FTRAIN_STATUS_INVALID_ARGUMENT));
    FTrainGroupedTensorId grouped{g.c.opaque};
    CHECK_EQ(static_cast<int>(ftrainArgsSetGroupedTensor(args, grouped, 1, matrix(&cell, dims), nullptr, nullptr, nullptr)),
             static_cast<int>(FTRAIN_STATUS_INVALID_ARGUMENT));
    ftrainArgsDestroy(args);
    ftrainOpsDestroy(ops);
    ftrainPatternDestroy(g.pattern);
}

TEST(last_status_is_per_thread_and_survives_queries) {
    CHECK_EQ(static_cast<int>(ftrainPatternCreate(nullptr)), static_cast<int>(FTRAIN_STATUS_INVALID_ARGUMENT));
    const char* message = ftrainGetLastMessage();
    CHECK(std::strlen(message) > 0);
    CHECK_EQ(static_cast<int>(ftrainGetLastStatus()), static_cast<int>(FTRAIN_STATUS_INVALID_ARGUMENT));
    CHECK(ftrainGetLastMessage() == message);  // queries neither reset nor move it
    std::thread([] {
        CHECK_EQ(static_cast<int>(ftrainGetLastStatus()), 0);  // a fresh thread starts clean
        CHECK_EQ(std::string(ftrainGetLastMessage()), std::string(""));
    }).join();
    CHECK_EQ(static_cast<int>(ftrainGetLastStatus()), static_cast<int>(FTRAIN_STATUS_INVALID_ARGUMENT));
    FTrainPattern pattern = nullptr;
    CHECK_EQ(static_cast<int>(ftrainPatternCreate(&pattern)), 0);
    CHECK_EQ(static_cast<int>(ftrainGetLastStatus()), 0);  // a success clears it
    CHECK_EQ(std::string(ftrainGetLastMessage()), std::string(""));
    ftrainPatternDestroy(pattern);
}

TEST(one_shot_gemm_walks_the_workspace_budget) {
    fake::reset();
    const std::int64_t a_dims[2] = {256, 16384}, b_dims[2] = {16384, 256}, d_dims[2] = {256, 256};
    float alpha = 1.0F, beta = 0.0F;
    const auto call = [&](void* workspace, std::uint64_t bytes) {
        return ftrainGemm(matrix(address(0x10000), a_dims), matrix(address(0x20000), b_dims), matrix(nullptr, d_dims),
                          matrix(address(0x40000), d_dims), scalar(&alpha), scalar(&beta), FTRAIN_NUMERIC_TYPE_FP32, workspace,
                          bytes, nullptr);
    };
    // No workspace: the first workspace-free primitive of the Plan runs.
    CHECK_EQ(static_cast<int>(call(nullptr, 0)), 0);
    CHECK_EQ(fake::state().launches.back().kernel, static_cast<int>(FTCUDA_GEMM_TF32X3));
    // Enough workspace: primitive 0 (split-K here) runs.
    char buffer[8];
    CHECK_EQ(static_cast<int>(call(buffer, 1 << 20)), 0);
    CHECK_EQ(fake::state().launches.back().kernel, static_cast<int>(FTCUDA_GEMM_TF32X3_SPLITK));
    // A workspace smaller than primitive 0 asks for (the fake's split-K kernels want 4096 bytes) is
    // walked past like no workspace at all; one of exactly the required size selects primitive 0.
    CHECK_EQ(static_cast<int>(call(buffer, 4095)), 0);
    CHECK_EQ(fake::state().launches.back().kernel, static_cast<int>(FTCUDA_GEMM_TF32X3));
    CHECK_EQ(fake::state().launches.back().workspace_bytes, std::uint64_t{4095});
    CHECK_EQ(static_cast<int>(call(buffer, 4096)), 0);
    CHECK_EQ(fake::state().launches.back().kernel, static_cast<int>(FTCUDA_GEMM_TF32X3_SPLITK));
    // A failing call leaves its own diagnostic as the thread's last message.
    const std::int64_t wrong[2] = {5, 5};
    CHECK_EQ(static_cast<int>(ftrainGemm(matrix(address(0x10000), a_dims), matrix(address(0x20000), wrong), matrix(nullptr, d_dims),
                                         matrix(address(0x40000), d_dims), scalar(&alpha), scalar(&beta), FTRAIN_NUMERIC_TYPE_FP32,
                                         nullptr, 0, nullptr)),
             static_cast<int>(FTRAIN_STATUS_INVALID_ARGUMENT));
    CHECK(std::strstr(ftrainGetLastMessage(), "columns but b has") != nullptr);
    fake::reset();
}

// A failed kernel launch or a failed launch configuration surfaces as INTERNAL_ERROR with the platform's
// reason in the message (the reference maps hipGetLastError the same way,
// src/primitive/hygon/gemm/fp32_gemm.hip:47-50, through the catch-all of src/include/flash_train/api.hpp:36-62);
// the Plan stays valid and destroyable, and the next call is clean.
TEST(one_shot_and_staged_calls_report_injected_platform_failures) {
    fake::reset();
    GemmGraph g = makeGraph();
    FTrainOps ops = nullptr;
    CHECK_EQ(static_cast<int>(ftrainOpsCreate(&ops, g.pattern)), 0);
    FTrainArgs args = nullptr;
    CHECK_EQ(static_cast<int>(ftrainArgsCreate(&args, ops)), 0);
    const std::int64_t a_dims[2] = {512, 1024}, b_dims[2] = {1024, 768}, d_dims[2] = {512, 768};
    float alpha = 1.0F, beta = 0.0F;
    ftrainArgsSetTensor(args, g.a, matrix(address(0x10000), a_dims));
    ftrainArgsSetTensor(args, g.b, matrix(address(0x20000), b_dims));
    ftrainArgsSetTensor(args, g.c, matrix(nullptr, d_dims));
    ftrainArgsSetTensor(args, g.d, matrix(address(0x40000), d_dims));
    ftrainArgsSetTensor(args, g.alpha, scalar(&alpha));
    ftrainArgsSetTensor(args, g.beta, scalar(&beta));
    CHECK_EQ(static_cast<int>(ftrainArgsSetGemm(args, g.op, FTRAIN_NUMERIC_TYPE_FP32)), 0);

    // Configure fails: no Plan, the caller's variable untouched, the reason in the message.
    FTrainPlan plan = reinterpret_cast<FTrainPlan>(0x5);
    fake::state().fail_next_configure = "cudaFuncSetAttribute failed: injected";
    CHECK_EQ(static_cast<int>(ftrainPlanCreate(&plan, args)), static_cast<int>(FTRAIN_STATUS_INTERNAL_ERROR));
    CHECK(plan == reinterpret_cast<FTrainPlan>(0x5));
    CHECK(std::strstr(ftrainGetLastMessage(), "configuring the launch failed: cudaFuncSetAttribute failed: injected") != nullptr);
    CHECK_EQ(static_cast<int>(ftrainGetLastStatus()), static_cast<int>(FTRAIN_STATUS_INTERNAL_ERROR));

    // The same Args make a Plan once the platform answers again.
    plan = nullptr;
    CHECK_EQ(static_cast<int>(ftrainPlanCreate(&plan, args)), 0);
    CHECK(plan != nullptr);
    std::uint64_t bytes = 0;
    CHECK_EQ(static_cast<int>(ftrainPlanGetPrimitiveRequiredWorkspaceBytes(plan, 0, &bytes)), 0);
    char workspace[8];
    void* const pointer = bytes != 0 ? workspace : nullptr;

    // Launch fails: INTERNAL_ERROR, nothing recorded as launched, the Plan still answers queries.
    const std::size_t launched = fake::state().launches.size();
    fake::state().fail_next_launch = "an illegal memory access was encountered (injected)";
    CHECK_EQ(static_cast<int>(ftrainPlanExecutePrimitive(plan, 0, pointer, bytes, nullptr)),
             static_cast<int>(FTRAIN_STATUS_INTERNAL_ERROR));
    CHECK(std::strstr(ftrainGetLastMessage(), "kernel launch failed: an illegal memory access was encountered (injected)") != nullptr);
    CHECK_EQ(fake::state().launches.size(), launched);
    CHECK_EQ(static_cast<int>(ftrainGetLastStatus()), static_cast<int>(FTRAIN_STATUS_INTERNAL_ERROR));
    std::uint64_t count = 0;
    CHECK_EQ(static_cast<int>(ftrainPlanGetNumPrimitives(plan, &count)), 0);
    CHECK(count >= 1);

    // The next execute of the same Plan is clean and reaches the platform.
    CHECK_EQ(static_cast<int>(ftrainPlanExecutePrimitive(plan, 0, pointer, bytes, nullptr)), 0);
    CHECK_EQ(fake::state().launches.size(), launched + 1);
    CHECK_EQ(static_cast<int>(ftrainGetLastStatus()), 0);
    CHECK_EQ(std::strlen(ftrainGetLastMessage()), std::size_t{0});

    // The one-shot call carries the launch failure through its own clean-up.
    fake::state().fail_next_launch = "unspecified launch failure (injected)";
    CHECK_EQ(static_cast<int>(ftrainGemm(matrix(address(0x10000), a_dims), matrix(address(0x20000), b_dims), matrix(nullptr, d_dims),
                                         matrix(address(0x40000), d_dims), scalar(&alpha), scalar(&beta), FTRAIN_NUMERIC_TYPE_FP32,
                                         nullptr, 0, nullptr)),
             static_cast<int>(FTRAIN_STATUS_INTERNAL_ERROR));
    CHECK(std::strstr(ftrainGetLastMessage(), "unspecified launch failure (injected)") != nullptr);

    CHECK_EQ(static_cast<int>(ftrainPlanDestroy(plan)), 0);
    CHECK_EQ(static_cast<int>(ftrainArgsDestroy(args)), 0);
    CHECK_EQ(static_cast<int>(ftrainOpsDestroy(ops)), 0);
    CHECK_EQ(static_cast<int>(ftrainPatternDestroy(g.pattern)), 0);
    fake::reset();
}

// The one-shot call keeps the Plans of its recent calls per thread: equal arguments (addresses, shapes,
// the VALUES of alpha and beta, device) execute the kept Plan again without configuring anything; any
// difference makes a new Plan, as the reference's per-call Plan would be (src/api/gemm_api.cpp:54-83 there).
TEST(one_shot_gemm_reuses_the_plan_of_an_equal_call) {
    fake::reset();
    const std::int64_t a_dims[2] = {640, 512}, b_dims[2] = {512, 384}, d_dims[2] = {640, 384};
    float alpha = 1.0F, beta = 0.0F;
    const auto call = [&](std::uintptr_t a_address) {
        return ftrainGemm(matrix(address(a_address), a_dims), matrix(address(0x200000), b_dims), matrix(nullptr, d_dims),
                          matrix(address(0x400000), d_dims), scalar(&alpha), scalar(&beta), FTRAIN_NUMERIC_TYPE_FP32, nullptr, 0,
                          nullptr);
    };
    CHECK_EQ(static_cast<int>(call(0x100000)), 0);
    const int configured = fake::state().configures;
    const std::size_t launched = fake::state().launches.size();
    CHECK(configured >= 1);
    CHECK_EQ(static_cast<int>(call(0x100000)), 0);
    CHECK_EQ(fake::state().configures, configured);            // nothing configured again
    CHECK_EQ(fake::state().launches.size(), launched + 1);     // but launched again, with the same description
    CHECK(fake::state().launches.back().desc.a == address(0x100000));
    CHECK_EQ(static_cast<int>(ftrainGetLastStatus()), 0);
    // The scalars are compared by value, as a Plan reads them when it is made: a changed alpha is another Plan...
    alpha = 2.5F;
    CHECK_EQ(static_cast<int>(call(0x100000)), 0);
    CHECK(fake::state().configures > configured);
    CHECK_EQ(fake::state().launches.back().desc.alpha, 2.5F);
    // ...and so is another address.
    const int after_alpha = fake::state().configures;
    CHECK_EQ(static_cast<int>(call(0x180000)), 0);
    CHECK(fake::state().configures > after_alpha);
    CHECK(fake::state().launches.back().desc.a == address(0x180000));
    // The first pair of values is still remembered.
    alpha = 1.0F;
    const int before = fake::state().configures;
    CHECK_EQ(static_cast<int>(call(0x100000)), 0);
    CHECK_EQ(fake::state().configures, before);
    CHECK_EQ(fake::state().launches.back().desc.alpha, 1.0F);
    // Another current device: a Plan of its own (Plans are bound to their device).
    fake::state().device = 3;
    CHECK_EQ(static_cast<int>(call(0x100000)), 0);
    CHECK(fake::state().configures > before);
    // More distinct calls than the memo holds: still correct, the oldest simply are planned again.
    fake::state().device = 0;
    for (std::uintptr_t i = 0; i < 80; ++i) { CHECK_EQ(static_cast<int>(call(0x1000000 + i * 0x10000)), 0); }
    CHECK(fake::state().launches.back().desc.a == address(0x1000000 + 79 * 0x10000));
    fake::reset();
}
