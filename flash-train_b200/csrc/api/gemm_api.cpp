// ftrainGemm: the one-shot call, built strictly on the staged C API.
// Reference: src/api/gemm_api.cpp:28-83.
#include "api/api_support.hpp"
#include "core/trace.hpp"
#include "flash_train/flash_train.h"

namespace {

// Pattern -> Ops for the plain Gemm graph, made once per process.
struct GemmEntry {
    FTrainOps ops{nullptr};
    FTrainTensorId a{}, b{}, c{}, d{}, alpha{}, beta{};
    FTrainGemmOpId gemm{};
    FTrainStatus status{FTRAIN_STATUS_SUCCESS};
};

const GemmEntry& gemmEntry() {
    static const GemmEntry entry = [] {
        GemmEntry made;
        FTrainPattern pattern = nullptr;
        FTrainStatus status   = ftrainPatternCreate(&pattern);
        FTrainTensorId* const roles[] = {&made.a, &made.b, &made.c, &made.alpha, &made.beta, &made.d};
        for (FTrainTensorId* role : roles) {
            if (status == FTRAIN_STATUS_SUCCESS) { status = ftrainPatternAddTensor(pattern, role); }
        }
        if (status == FTRAIN_STATUS_SUCCESS) {
            status = ftrainPatternAddGemm(pattern, &made.gemm, made.a, made.b, made.c, made.d, made.alpha, made.beta);
        }
        if (status == FTRAIN_STATUS_SUCCESS) { status = ftrainOpsCreate(&made.ops, pattern); }
        if (pattern != nullptr) { ftrainPatternDestroy(pattern); }
        made.status = status;
        return made;
    }();
    return entry;
}

// The reference's one-shot call always runs primitive 0 and fails when the
// caller's workspace is smaller than that primitive needs (src/api/gemm_api.cpp:73
// there, where the only primitive needs none). Here primitive 0 can be a
// split-K kernel that wants a workspace, so the one-shot call follows the
// documented budget walk instead: the first primitive, in the Plan's best-first
// order, whose requirement the supplied workspace covers. With a sufficient
// workspace that is primitive 0, as in the reference; if nothing fits,
// primitive 0 is run so that its diagnostic reaches the caller.
std::uint64_t pickPrimitive(FTrainPlan plan, const void* workspace, std::uint64_t workspace_bytes) {
    std::uint64_t count = 0;
    if (ftrainPlanGetNumPrimitives(plan, &count) != FTRAIN_STATUS_SUCCESS) { return 0; }
    for (std::uint64_t index = 0; index < count; ++index) {
        std::uint64_t needed = 0;
        if (ftrainPlanGetPrimitiveRequiredWorkspaceBytes(plan, index, &needed) != FTRAIN_STATUS_SUCCESS) { return 0; }
        if (needed == 0 || (workspace != nullptr && needed <= workspace_bytes)) { return index; }
    }
    return 0;
}

}  // namespace

extern "C" FTrainStatus ftrainGemm(FTrainStorageView a, FTrainStorageView b, FTrainStorageView c, FTrainStorageView d,
                                   FTrainStorageView alpha, FTrainStorageView beta, FTrainNumericType compute_type,
                                   void* workspace, uint64_t workspace_bytes, FTrainStream stream) {
    ftrain::ScopedTraceRange trace("ftrainGemm");
    const GemmEntry& entry = gemmEntry();
    if (entry.status != FTRAIN_STATUS_SUCCESS) { return entry.status; }

    FTrainArgs args     = nullptr;
    FTrainPlan plan     = nullptr;
    FTrainStatus status = ftrainArgsCreate(&args, entry.ops);
    const struct {
        FTrainTensorId role;
        const FTrainStorageView* view;
    } bindings[] = {{entry.a, &a}, {entry.b, &b}, {entry.c, &c}, {entry.d, &d}, {entry.alpha, &alpha}, {entry.beta, &beta}};
    for (const auto& binding : bindings) {
        if (status == FTRAIN_STATUS_SUCCESS) { status = ftrainArgsSetTensor(args, binding.role, *binding.view); }
    }
    if (status == FTRAIN_STATUS_SUCCESS) { status = ftrainArgsSetGemm(args, entry.gemm, compute_type); }
    if (status == FTRAIN_STATUS_SUCCESS) { status = ftrainPlanCreate(&plan, args); }
    if (status == FTRAIN_STATUS_SUCCESS) {
        status = ftrainPlanExecutePrimitive(plan, pickPrimitive(plan, workspace, workspace_bytes), workspace,
                                            workspace_bytes, stream);
    }

    // The clean-up calls below overwrite the thread's last result; the failing
    // call's diagnostic is what the caller must see.
    if (status == FTRAIN_STATUS_SUCCESS) {
        if (plan != nullptr) { ftrainPlanDestroy(plan); }
        if (args != nullptr) { ftrainArgsDestroy(args); }
        return status;
    }
    const ftrain::Result failure = ftrain::getLastResult();
    if (plan != nullptr) { ftrainPlanDestroy(plan); }
    if (args != nullptr) { ftrainArgsDestroy(args); }
    ftrain::setLastResult(failure.getStatus(), failure.getMessage());
    return status;
}
