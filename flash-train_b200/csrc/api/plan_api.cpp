// extern "C" Plan creation, queries and execution. Reference: src/api/plan_api.cpp:12-95.
#include <memory>

#include "api/api_support.hpp"
#include "core/handle.hpp"
#include "core/trace.hpp"

using ftrain::Exception;
using ftrain::invokeApi;
using ftrain::requireNonNull;

extern "C" FTrainStatus ftrainPlanCreate(FTrainPlan* plan, FTrainArgs args) {
    ftrain::ScopedTraceRange trace("ftrainPlanCreate");
    return invokeApi([&] {
        requireNonNull(plan, "ftrainPlanCreate", "plan output");
        requireNonNull(args, "ftrainPlanCreate", "args handle");
        const auto engine = ftrain::getGlobalHandle().findOpsEngine(args->args.getPatternKey());
        if (engine == nullptr) {
            throw Exception(FTRAIN_STATUS_INTERNAL_ERROR, "OpsEngine registered for Args is unavailable");
        }
        *plan = new FTrainPlanStruct(engine->createPlan(args->args));
    });
}

extern "C" FTrainStatus ftrainPlanDestroy(FTrainPlan plan) {
    return invokeApi([&] {
        requireNonNull(plan, "ftrainPlanDestroy", "plan handle");
        delete plan;
    });
}

extern "C" FTrainStatus ftrainPlanGetNumPrimitives(FTrainPlan plan, std::uint64_t* num_primitives) {
    return invokeApi([&] {
        requireNonNull(plan, "ftrainPlanGetNumPrimitives", "plan handle");
        requireNonNull(num_primitives, "ftrainPlanGetNumPrimitives", "num_primitives output");
        *num_primitives = plan->plan.getNumPrimitives();
    });
}

extern "C" FTrainStatus ftrainPlanGetPrimitiveName(FTrainPlan plan, std::uint64_t primitive_index, const char** name) {
    return invokeApi([&] {
        requireNonNull(plan, "ftrainPlanGetPrimitiveName", "plan handle");
        requireNonNull(name, "ftrainPlanGetPrimitiveName", "name output");
        *name = plan->plan.getPrimitiveName(primitive_index);
    });
}

extern "C" FTrainStatus ftrainPlanGetPrimitiveRequiredWorkspaceBytes(FTrainPlan plan, std::uint64_t primitive_index,
                                                                     std::uint64_t* workspace_bytes) {
    return invokeApi([&] {
        requireNonNull(plan, "ftrainPlanGetPrimitiveRequiredWorkspaceBytes", "plan handle");
        requireNonNull(workspace_bytes, "ftrainPlanGetPrimitiveRequiredWorkspaceBytes", "workspace_bytes output");
        *workspace_bytes = plan->plan.getPrimitiveRequiredWorkspaceBytes(primitive_index);
    });
}

extern "C" FTrainStatus ftrainPlanExecutePrimitive(FTrainPlan plan, std::uint64_t primitive_index, void* workspace,
                                                   std::uint64_t workspace_bytes, FTrainStream stream) {
    ftrain::ScopedTraceRange trace("ftrainPlanExecutePrimitive");
    return invokeApi([&] {
        requireNonNull(plan, "ftrainPlanExecutePrimitive", "plan handle");
        plan->plan.execute(primitive_index, workspace, workspace_bytes, stream);
    });
}
