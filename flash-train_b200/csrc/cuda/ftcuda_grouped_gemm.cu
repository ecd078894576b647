// The grouped-GEMM entry points of ftcuda/ftcuda.h: many independent FP32 GEMMs
// D_g = alpha * A_g * B_g + beta * C_g behind one configure / launch pair.
//
//   FTCUDA_GROUPED_GEMM_EXACT   every non-empty group is one launch of the exact-FP32 family
//                               (FTCUDA_GEMM_SIMT: TMA-staged where the group's layout allows it, the
//                               predicated kernel otherwise, K = 0 included). Any layout, no workspace.
//   FTCUDA_GROUPED_GEMM_TF32X3  ONE persistent launch of the 3xTF32 tensor-core kernel over the
//                               output tiles of all groups (gemm_tf32x3.cu, grouped form). The
//                               per-group table (TMA descriptors, output views) travels in the
//                               workspace.
#include <cuda_runtime_api.h>

#include <new>

#include "gemm_kernels.hpp"

using ftcuda::fail;
using ftcuda::GroupedLaunchState;

struct FtcudaGroupedGemmLaunch {
    GroupedLaunchState state;
};

namespace {

const char* supportsGrouped(int kernel, const FtcudaGemmDesc* groups, std::uint32_t count) {
    switch (kernel) {
        case FTCUDA_GROUPED_GEMM_EXACT:
            for (std::uint32_t g = 0; g < count; ++g) {
                if (groups[g].m * groups[g].n == 0) { continue; }
                if (const char* reason = ftcuda::supportsSimt(groups[g], false)) { return reason; }
            }
            return nullptr;
        case FTCUDA_GROUPED_GEMM_TF32X3: return ftcuda::supportsTensorGrouped(groups, count);
        default: return "unknown grouped kernel family";
    }
}

}  // namespace

extern "C" int ftcuda_grouped_gemm_supports(int kernel, const FtcudaGemmDesc* groups, uint32_t num_groups, char* message,
                                            size_t message_capacity) {
    if (groups == nullptr && num_groups != 0) { return fail(message, message_capacity, 1, "null descriptors"); }
    const char* reason = supportsGrouped(kernel, groups, num_groups);
    if (reason != nullptr) { return fail(message, message_capacity, 1, "%s", reason); }
    return 0;
}

extern "C" int ftcuda_grouped_gemm_configure(int kernel, const FtcudaGemmDesc* groups, uint32_t num_groups,
                                             FtcudaGroupedGemmLaunch** launch, char* message, size_t message_capacity) {
    if (launch == nullptr || (groups == nullptr && num_groups != 0)) { return fail(message, message_capacity, 1, "null argument"); }
    const char* reason = supportsGrouped(kernel, groups, num_groups);
    if (reason != nullptr) { return fail(message, message_capacity, 1, "%s", reason); }
    FtcudaGroupedGemmLaunch* made = new (std::nothrow) FtcudaGroupedGemmLaunch();
    if (made == nullptr) { return fail(message, message_capacity, 1, "out of host memory"); }
    GroupedLaunchState& state = made->state;
    state.kernel              = kernel;
    state.device              = num_groups != 0 ? groups[0].device : 0;
    int status                = 0;
    try {
        if (kernel == FTCUDA_GROUPED_GEMM_EXACT) {
            for (std::uint32_t g = 0; g < num_groups && status == 0; ++g) {
                if (groups[g].m * groups[g].n == 0) { continue; }
                ftcuda::LaunchState one{};
                one.desc   = groups[g];
                one.kernel = FTCUDA_GEMM_SIMT;
                status     = ftcuda::configureSimt(one, false, message, message_capacity);
                if (status == 0) {
                    state.per_group.push_back(one);
                    state.host_status = one.host_status;
                }
            }
        } else {
            status = ftcuda::configureTensorGrouped(state, groups, num_groups, message, message_capacity);
        }
    } catch (const std::bad_alloc&) { status = fail(message, message_capacity, 1, "out of host memory"); }
    if (status != 0) {
        delete made;
        return status;
    }
    *launch = made;
    return 0;
}

extern "C" uint64_t ftcuda_grouped_gemm_workspace_bytes(const FtcudaGroupedGemmLaunch* launch) {
    return launch == nullptr ? 0 : launch->state.workspace_bytes;
}

extern "C" int ftcuda_grouped_gemm_launch(const FtcudaGroupedGemmLaunch* launch, void* workspace, uint64_t workspace_bytes,
                                          void* stream, char* message, size_t message_capacity) {
    if (launch == nullptr) { return fail(message, message_capacity, 1, "null launch"); }
    const GroupedLaunchState& state = launch->state;
    if (workspace_bytes < state.workspace_bytes || (state.workspace_bytes != 0 && workspace == nullptr)) {
        return fail(message, message_capacity, 1, "workspace of %llu bytes needed", static_cast<unsigned long long>(state.workspace_bytes));
    }
    if (const int code = ftcuda::takeDeviceStatus(state.host_status)) {
        return fail(message, message_capacity, 1, "an earlier kernel reported a timed-out wait (code %d)", code);
    }
    const cudaStream_t cuda_stream = static_cast<cudaStream_t>(stream);
    cudaError_t error              = cudaSuccess;
    if (state.kernel == FTCUDA_GROUPED_GEMM_EXACT) {
        for (const ftcuda::LaunchState& one : state.per_group) {
            error = ftcuda::launchSimt(one, nullptr, cuda_stream);
            if (error != cudaSuccess) { break; }
        }
    } else {
        error = ftcuda::launchTensorGrouped(state, workspace, cuda_stream);
    }
    if (error != cudaSuccess) { return fail(message, message_capacity, 1, "%s", cudaGetErrorString(error)); }
    return 0;
}

extern "C" void ftcuda_grouped_gemm_destroy(FtcudaGroupedGemmLaunch* launch) { delete launch; }
