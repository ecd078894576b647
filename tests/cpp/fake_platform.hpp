// A fake of the platform layer's C ABI (ftcuda/ftcuda.h) for host-only tests:
// a settable "current device", and configure/launch calls that are recorded
// instead of touching a GPU. The host pipeline is linked against this fake in
// the C++ test binary, the way the reference's engine tests inject mock
// policies instead of faking a device (tests/engine/engine_test.cpp:59-201 there).
#ifndef FTRAIN_TESTS_FAKE_PLATFORM_HPP_
#define FTRAIN_TESTS_FAKE_PLATFORM_HPP_

#include <cstdint>
#include <vector>

#include "ftcuda/ftcuda.h"

namespace fake {

struct LaunchRecord {
    int kernel;
    void* workspace;
    std::uint64_t workspace_bytes;
    void* stream;
    FtcudaGemmDesc desc;
};

struct GroupedLaunchRecord {
    int kernel;
    void* workspace;
    std::uint64_t workspace_bytes;
    void* stream;
    std::vector<FtcudaGemmDesc> groups;
};

struct State {
    int device               = 0;
    bool device_query_fails  = false;
    int sm_count             = 148;
    std::uint64_t split_k_workspace = 4096;  // what the fake split-K kernels ask for
    std::vector<LaunchRecord> launches;
    std::vector<GroupedLaunchRecord> grouped_launches;
    std::uint64_t grouped_tensor_workspace = 1024;  // what the fake grouped tensor-core kernel asks for
    int grouped_live = 0;                           // configured grouped launches not yet destroyed
    int configures = 0;
    int supports   = 0;
    // Host-side failure injection: the next configure / launch call answers with this reason (and
    // clears it), the way the real layer reports a failed cudaFuncSetAttribute or kernel launch.
    const char* fail_next_configure = nullptr;
    const char* fail_next_launch    = nullptr;
};

State& state();
void reset();

}  // namespace fake

#endif
