#include "fake_platform.hpp"

#include <cstdio>
#include <cstring>
#include <vector>

namespace fake {

State& state() {
    static thread_local State current;
    return current;
}

void reset() { state() = State{}; }

namespace {

struct Blob {
    int kernel;
    std::uint64_t workspace;
    FtcudaGemmDesc desc;
};

int fail(char* message, size_t capacity, const char* text) {
    if (message != nullptr && capacity != 0) { std::snprintf(message, capacity, "%s", text); }
    return 1;
}

}  // namespace
}  // namespace fake

extern "C" int ftcuda_current_device(int32_t* device, char* message, size_t capacity) {
    if (fake::state().device_query_fails) { return fake::fail(message, capacity, "no CUDA-capable device is detected"); }
    *device = fake::state().device;
    return 0;
}

extern "C" int ftcuda_device_sm_count(int32_t, int32_t* sm_count, char*, size_t) {
    *sm_count = fake::state().sm_count;
    return 0;
}

// Mirrors the real layer's documented rules closely enough for selection tests.
extern "C" int ftcuda_gemm_supports(int kernel, const FtcudaGemmDesc* desc, char* message, size_t capacity) {
    ++fake::state().supports;
    const bool row_major_a = desc->a_col_stride == 1 && desc->a_row_stride % 4 == 0 &&
                             reinterpret_cast<std::uintptr_t>(desc->a) % 16 == 0 && desc->a != nullptr;
    const bool row_major_b = desc->b_col_stride == 1 && desc->b_row_stride % 4 == 0 &&
                             reinterpret_cast<std::uintptr_t>(desc->b) % 16 == 0 && desc->b != nullptr;
    switch (kernel) {
        case FTCUDA_GEMM_SIMT: return 0;
        case FTCUDA_GEMM_SIMT_SPLITK:
            return desc->m * desc->n != 0 && desc->k >= 512 ? 0 : fake::fail(message, capacity, "K is too short to split");
        case FTCUDA_GEMM_TF32X3:
        case FTCUDA_GEMM_TF32X3_SPLITK:
            if (desc->m * desc->n == 0 || desc->k < 32) { return fake::fail(message, capacity, "K is shorter than one K block"); }
            if (!row_major_a) { return fake::fail(message, capacity, "A is not row-major with a 16-byte aligned base and row pitch"); }
            if (!row_major_b) { return fake::fail(message, capacity, "B is not row-major with a 16-byte aligned base and row pitch"); }
            if (kernel == FTCUDA_GEMM_TF32X3_SPLITK && desc->k < 512) { return fake::fail(message, capacity, "K is too short to split"); }
            return 0;
        case FTCUDA_GEMM_SKINNY:
            if (desc->m == 0 || desc->m > 32) { return fake::fail(message, capacity, "more than 32 rows (or none) in A"); }
            if (desc->n % 4 != 0 || !row_major_b) { return fake::fail(message, capacity, "B is not row-major with a 16-byte row pitch"); }
            return 0;
        case FTCUDA_GEMM_TF32X3_ROWS:
            if (desc->m == 0 || desc->m > 64) { return fake::fail(message, capacity, "more than 64 rows (or none) in A"); }
            if (desc->k < 128 || !row_major_a || !row_major_b) { return fake::fail(message, capacity, "layout or K unsuitable"); }
            return 0;
        default: return fake::fail(message, capacity, "unknown kernel family");
    }
}

extern "C" int ftcuda_gemm_configure(int kernel, const FtcudaGemmDesc* desc, FtcudaGemmLaunch* launch, char* message,
                                     size_t capacity) {
    ++fake::state().configures;
    if (const char* reason = fake::state().fail_next_configure) {
        fake::state().fail_next_configure = nullptr;
        return fake::fail(message, capacity, reason);
    }
    std::memset(launch, 0, sizeof *launch);
    auto* blob      = reinterpret_cast<fake::Blob*>(launch);
    blob->kernel    = kernel;
    blob->desc      = *desc;
    blob->workspace = (kernel == FTCUDA_GEMM_TF32X3_SPLITK || kernel == FTCUDA_GEMM_SIMT_SPLITK)
                          ? fake::state().split_k_workspace
                          : 0;
    return 0;
}

extern "C" uint64_t ftcuda_gemm_workspace_bytes(const FtcudaGemmLaunch* launch) {
    return reinterpret_cast<const fake::Blob*>(launch)->workspace;
}

extern "C" int ftcuda_gemm_launch(const FtcudaGemmLaunch* launch, void* workspace, uint64_t workspace_bytes,
                                  void* stream, char* message, size_t capacity) {
    if (const char* reason = fake::state().fail_next_launch) {
        fake::state().fail_next_launch = nullptr;
        return fake::fail(message, capacity, reason);
    }
    const auto* blob = reinterpret_cast<const fake::Blob*>(launch);
    fake::state().launches.push_back(fake::LaunchRecord{blob->kernel, workspace, workspace_bytes, stream, blob->desc});
    return 0;
}

// ---- grouped entry points: the same rules as the real layer, nothing launched ----
struct FtcudaGroupedGemmLaunch {
    int kernel;
    std::uint64_t workspace;
    std::vector<FtcudaGemmDesc> groups;
};

extern "C" int ftcuda_grouped_gemm_supports(int kernel, const FtcudaGemmDesc* groups, uint32_t num_groups, char* message,
                                            size_t capacity) {
    ++fake::state().supports;
    if (kernel == FTCUDA_GROUPED_GEMM_EXACT) { return 0; }
    if (kernel != FTCUDA_GROUPED_GEMM_TF32X3) { return fake::fail(message, capacity, "unknown grouped kernel family"); }
    bool any = false;
    for (uint32_t g = 0; g < num_groups; ++g) {
        if (groups[g].m * groups[g].n == 0) { continue; }
        any = true;
        if (ftcuda_gemm_supports(FTCUDA_GEMM_TF32X3, &groups[g], message, capacity) != 0) { return 1; }
        if (groups[g].k < 128) { return fake::fail(message, capacity, "K is too short for the split-precision kernel (under 128)"); }
    }
    return any ? 0 : fake::fail(message, capacity, "every group is empty");
}

extern "C" int ftcuda_grouped_gemm_configure(int kernel, const FtcudaGemmDesc* groups, uint32_t num_groups,
                                             FtcudaGroupedGemmLaunch** launch, char* message, size_t capacity) {
    ++fake::state().configures;
    if (const char* reason = fake::state().fail_next_configure) {
        fake::state().fail_next_configure = nullptr;
        return fake::fail(message, capacity, reason);
    }
    auto* made      = new FtcudaGroupedGemmLaunch{};
    made->kernel    = kernel;
    made->workspace = kernel == FTCUDA_GROUPED_GEMM_TF32X3 ? fake::state().grouped_tensor_workspace : 0;
    made->groups.assign(groups, groups + num_groups);
    ++fake::state().grouped_live;
    *launch = made;
    return 0;
}

extern "C" uint64_t ftcuda_grouped_gemm_workspace_bytes(const FtcudaGroupedGemmLaunch* launch) { return launch->workspace; }

extern "C" int ftcuda_grouped_gemm_launch(const FtcudaGroupedGemmLaunch* launch, void* workspace, uint64_t workspace_bytes,
                                          void* stream, char* message, size_t capacity) {
    if (const char* reason = fake::state().fail_next_launch) {
        fake::state().fail_next_launch = nullptr;
        return fake::fail(message, capacity, reason);
    }
    fake::state().grouped_launches.push_back(fake::GroupedLaunchRecord{launch->kernel, workspace, workspace_bytes, stream, launch->groups});
    return 0;
}

extern "C" void ftcuda_grouped_gemm_destroy(FtcudaGroupedGemmLaunch* launch) {
    if (launch != nullptr) { --fake::state().grouped_live; }
    delete launch;
}

extern "C" uint64_t ftcuda_launch_count(void) { return fake::state().launches.size(); }
extern "C" int ftcuda_trace_push(const char*) { return 1; }
extern "C" void ftcuda_trace_pop(void) {}
extern "C" void ftcuda_trace_mark(const char*) {}
