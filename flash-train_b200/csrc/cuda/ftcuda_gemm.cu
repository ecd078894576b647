// The GEMM entry points of ftcuda/ftcuda.h: dispatch on the kernel family.
#include <cuda_runtime_api.h>

#include <cstring>
#include <type_traits>

#include "gemm_kernels.hpp"

namespace {

using ftcuda::LaunchState;

static_assert(std::is_trivially_copyable<LaunchState>::value, "a launch must be copyable with the Primitive");

bool stagesOperands(int kernel) {
    return kernel == FTCUDA_GEMM_TF32X3 || kernel == FTCUDA_GEMM_TF32X3_SPLITK || kernel == FTCUDA_GEMM_TF32X3_ROWS;
}

const char* supportsAsGiven(int kernel, const FtcudaGemmDesc& desc);

// The tensor-core families take operands TMA cannot describe through a copy in the workspace: their
// own rules are asked about the problem with those operands replaced by the copies' description.
const char* supports(int kernel, const FtcudaGemmDesc& desc) {
    if (!stagesOperands(kernel)) { return supportsAsGiven(kernel, desc); }
    LaunchState probe{};
    probe.desc = desc;
    if (const char* reason = ftcuda::planStaging(kernel, desc, probe)) { return reason; }
    return supportsAsGiven(kernel, probe.desc);
}

const char* supportsAsGiven(int kernel, const FtcudaGemmDesc& desc) {
    switch (kernel) {
        case FTCUDA_GEMM_SIMT: return ftcuda::supportsSimt(desc, false);
        case FTCUDA_GEMM_SIMT_SPLITK: return ftcuda::supportsSimt(desc, true);
        case FTCUDA_GEMM_TF32X3: return ftcuda::supportsTensor(desc, false);
        case FTCUDA_GEMM_TF32X3_SPLITK: return ftcuda::supportsTensor(desc, true);
        case FTCUDA_GEMM_SKINNY: return ftcuda::supportsSkinny(desc);
        case FTCUDA_GEMM_TF32X3_ROWS: return ftcuda::supportsTensorRows(desc);
        default: return "unknown kernel family";
    }
}

}  // namespace

extern "C" int ftcuda_gemm_supports(int kernel, const FtcudaGemmDesc* desc, char* message, size_t message_capacity) {
    if (desc == nullptr) { return ftcuda::fail(message, message_capacity, 1, "null descriptor"); }
    const char* reason = supports(kernel, *desc);
    if (reason != nullptr) { return ftcuda::fail(message, message_capacity, 1, "%s", reason); }
    return 0;
}

extern "C" int ftcuda_gemm_configure(int kernel, const FtcudaGemmDesc* desc, FtcudaGemmLaunch* launch, char* message,
                                     size_t message_capacity) {
    if (desc == nullptr || launch == nullptr) { return ftcuda::fail(message, message_capacity, 1, "null argument"); }
    const char* reason = supports(kernel, *desc);
    if (reason != nullptr) { return ftcuda::fail(message, message_capacity, 1, "%s", reason); }
    std::memset(launch, 0, sizeof *launch);
    LaunchState& state = *reinterpret_cast<LaunchState*>(launch);
    state.desc         = *desc;
    state.kernel       = kernel;
    if (stagesOperands(kernel)) {
        // state.desc now describes the copies; the family configures itself for them.
        if (const char* staging = ftcuda::planStaging(kernel, *desc, state)) { return ftcuda::fail(message, message_capacity, 1, "%s", staging); }
    }
    int status = 0;
    switch (kernel) {
        case FTCUDA_GEMM_SIMT: status = ftcuda::configureSimt(state, false, message, message_capacity); break;
        case FTCUDA_GEMM_SIMT_SPLITK: status = ftcuda::configureSimt(state, true, message, message_capacity); break;
        case FTCUDA_GEMM_TF32X3: status = ftcuda::configureTensor(state, false, message, message_capacity); break;
        case FTCUDA_GEMM_TF32X3_SPLITK: status = ftcuda::configureTensor(state, true, message, message_capacity); break;
        case FTCUDA_GEMM_TF32X3_ROWS: status = ftcuda::configureTensorRows(state, message, message_capacity); break;
        default: status = ftcuda::configureSkinny(state, message, message_capacity); break;
    }
    if (status == 0 && state.staged != 0) {
        // The copies take the head of the workspace (plus room to align them), the family's own needs follow.
        state.stage_bytes += 256;
        state.workspace_bytes += state.stage_bytes;
    }
    return status;
}

extern "C" uint64_t ftcuda_gemm_workspace_bytes(const FtcudaGemmLaunch* launch) {
    return launch == nullptr ? 0 : reinterpret_cast<const LaunchState*>(launch)->workspace_bytes;
}

extern "C" int ftcuda_gemm_launch(const FtcudaGemmLaunch* launch, void* workspace, uint64_t workspace_bytes,
                                  void* stream, char* message, size_t message_capacity) {
    if (launch == nullptr) { return ftcuda::fail(message, message_capacity, 1, "null launch"); }
    const LaunchState& state = *reinterpret_cast<const LaunchState*>(launch);
    if (workspace_bytes < state.workspace_bytes || (state.workspace_bytes != 0 && workspace == nullptr)) {
        return ftcuda::fail(message, message_capacity, 1, "workspace of %llu bytes needed",
                            static_cast<unsigned long long>(state.workspace_bytes));
    }
    // A kernel of an earlier launch on this device gave up on a wait (its results are not valid):
    // reported once, here, and cleared -- the kernel left in order, so later launches may proceed.
    if (const int code = ftcuda::takeDeviceStatus(state.host_status)) {
        return ftcuda::fail(message, message_capacity, 1, "an earlier kernel reported a timed-out wait (code %d)", code);
    }
    const cudaStream_t cuda_stream = static_cast<cudaStream_t>(stream);
    cudaError_t error              = cudaSuccess;
    if (state.staged != 0) {
        // Copy the operands TMA cannot fetch into the head of the workspace, point a copy of the launch's
        // descriptors at them, and hand the rest of the workspace to the kernel family.
        LaunchState local = state;
        if (message != nullptr && message_capacity != 0) { message[0] = '\0'; }
        error = ftcuda::runStaging(local, workspace, cuda_stream, message, message_capacity);
        if (error != cudaSuccess) {
            if (message != nullptr && message_capacity != 0 && message[0] != '\0') { return 1; }
            return ftcuda::fail(message, message_capacity, 1, "%s", cudaGetErrorString(error));
        }
        void* const rest = static_cast<unsigned char*>(workspace) + local.stage_bytes;
        local.workspace_bytes -= local.stage_bytes;
        if (local.kernel == FTCUDA_GEMM_TF32X3_ROWS) {
            error = ftcuda::launchTensorRows(local, cuda_stream);
        } else {
            error = ftcuda::launchTensor(local, rest, cuda_stream);
        }
        if (error != cudaSuccess) { return ftcuda::fail(message, message_capacity, 1, "%s", cudaGetErrorString(error)); }
        return 0;
    }
    switch (state.kernel) {
        case FTCUDA_GEMM_SIMT:
        case FTCUDA_GEMM_SIMT_SPLITK: error = ftcuda::launchSimt(state, workspace, cuda_stream); break;
        case FTCUDA_GEMM_TF32X3:
        case FTCUDA_GEMM_TF32X3_SPLITK: error = ftcuda::launchTensor(state, workspace, cuda_stream); break;
        case FTCUDA_GEMM_SKINNY: error = ftcuda::launchSkinny(state, cuda_stream); break;
        case FTCUDA_GEMM_TF32X3_ROWS: error = ftcuda::launchTensorRows(state, cuda_stream); break;
        default: return ftcuda::fail(message, message_capacity, 1, "unknown kernel family %d", state.kernel);
    }
    if (error != cudaSuccess) { return ftcuda::fail(message, message_capacity, 1, "%s", cudaGetErrorString(error)); }
    return 0;
}

extern "C" int ftcuda_gemm_launch_scatter(const FtcudaGemmLaunch* launch, void* workspace, uint64_t workspace_bytes,
                                          float* const* owner_rows, int32_t owners, uint64_t rows_per_owner, void* stream,
                                          char* message, size_t message_capacity) {
    if (launch == nullptr || owner_rows == nullptr) { return ftcuda::fail(message, message_capacity, 1, "null argument"); }
    const LaunchState& state = *reinterpret_cast<const LaunchState*>(launch);
    if (state.kernel != FTCUDA_GEMM_TF32X3 && state.kernel != FTCUDA_GEMM_TF32X3_SPLITK) {
        return ftcuda::fail(message, message_capacity, 1, "scatter launches exist for the tensor-core kernels only");
    }
    if (state.staged != 0) {
        return ftcuda::fail(message, message_capacity, 1, "scatter launches take operands TMA can fetch as they are (no staging)");
    }
    if (owners < 1 || owners > 8) { return ftcuda::fail(message, message_capacity, 1, "1 to 8 owners, got %d", owners); }
    if (rows_per_owner == 0 || rows_per_owner >= (1ULL << 31) || rows_per_owner * static_cast<uint64_t>(owners) < state.desc.m) {
        return ftcuda::fail(message, message_capacity, 1, "%d owners of %llu rows do not cover m = %llu", owners,
                            static_cast<unsigned long long>(rows_per_owner), static_cast<unsigned long long>(state.desc.m));
    }
    for (int32_t i = 0; i < owners; ++i) {
        if (owner_rows[i] == nullptr) { return ftcuda::fail(message, message_capacity, 1, "owner %d has no buffer", i); }
    }
    if (const int code = ftcuda::takeDeviceStatus(state.host_status)) {
        return ftcuda::fail(message, message_capacity, 1, "an earlier kernel reported a timed-out wait (code %d)", code);
    }
    // A workspace is optional here; one that is too small is ignored (direct adds).
    if (workspace_bytes < state.workspace_bytes) { workspace = nullptr; }
    const cudaError_t error = ftcuda::launchTensorScatter(state, workspace, owner_rows, static_cast<std::uint32_t>(owners),
                                                          static_cast<std::uint32_t>(rows_per_owner), static_cast<cudaStream_t>(stream));
    if (error != cudaSuccess) { return ftcuda::fail(message, message_capacity, 1, "%s", cudaGetErrorString(error)); }
    return 0;
}
