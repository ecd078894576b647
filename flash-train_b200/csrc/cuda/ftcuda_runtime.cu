// Device queries, TMA descriptor encoding, NVTX ranges and the launch counter
// behind ftcuda/ftcuda.h.
#include <cuda.h>
#include <cuda_runtime_api.h>
#include <cudaTypedefs.h>
#include <nvtx3/nvToolsExt.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <mutex>

#include "gemm_kernels.hpp"
#include "ptx.cuh"

namespace ftcuda {
namespace {

constexpr int kMaxDevices = 64;

struct DeviceInfo {
    std::once_flag sm_once;
    cudaError_t sm_error = cudaSuccess;
    int sm_count         = 0;
    std::once_flag status_once;
    cudaError_t status_error = cudaSuccess;
    int* status_host         = nullptr;
    int* status_device       = nullptr;
};

DeviceInfo& deviceInfo(int device) {
    static DeviceInfo table[kMaxDevices];
    return table[device];
}

std::atomic<std::uint64_t> g_launches{0};

// FP32 FFMA throughput probe: eight independent accumulator chains per thread, 32 FFMAs per loop trip.
__global__ void __launch_bounds__(1024) ffmaRateProbe(float* sink, float x, float y, int trips) {
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) { acc[i] = 1e-3F * static_cast<float>(threadIdx.x) + static_cast<float>(i); }
    for (int trip = 0; trip < trips; ++trip) {
#pragma unroll
        for (int round = 0; round < 4; ++round) {
#pragma unroll
            for (int i = 0; i < 8; ++i) { acc[i] = fmaf(acc[i], x, y); }
        }
    }
    float total = 0.0F;
#pragma unroll
    for (int i = 0; i < 8; ++i) { total += acc[i]; }
    if (total == 12345.678F && sink != nullptr) { *sink = total; }  // keeps the chains alive; never true in practice
}

// One warp waiting on a barrier nobody arrives on: the give-up path of every bounded wait.
__global__ void boundedWaitProbe(int* status, unsigned long long budget_ns) {
    __shared__ std::uint64_t barrier;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbarrierInit(&barrier, 1);
        abort_flag = 0;
        fenceBarrierInit();
    }
    __syncthreads();
    const bool completed = mbarrierWaitFor(&barrier, 0, &abort_flag, budget_ns);
    if (!completed && threadIdx.x == 0 && status != nullptr) { *status = 2; }
}

PFN_cuTensorMapEncodeTiled_v12000 tensorMapEncoder() {
    // Resolved through the runtime so the library needs no link-time libcuda.
    static const PFN_cuTensorMapEncodeTiled_v12000 encoder = [] {
        void* entry                            = nullptr;
        cudaDriverEntryPointQueryResult result = cudaDriverEntryPointSymbolNotFound;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &result) != cudaSuccess ||
            result != cudaDriverEntryPointSuccess) {
            entry = nullptr;
        }
        return reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(entry);
    }();
    return encoder;
}

}  // namespace

int fail(char* message, std::size_t capacity, int code, const char* format, ...) {
    if (message != nullptr && capacity != 0) {
        std::va_list arguments;
        va_start(arguments, format);
        std::vsnprintf(message, capacity, format, arguments);
        va_end(arguments);
    }
    return code;
}

bool deviceSmCount(int device, int* sm_count, char* message, std::size_t capacity) {
    if (device < 0 || device >= kMaxDevices) {
        fail(message, capacity, 1, "device %d is out of range", device);
        return false;
    }
    DeviceInfo& info = deviceInfo(device);
    std::call_once(info.sm_once, [&] {
        info.sm_error = cudaDeviceGetAttribute(&info.sm_count, cudaDevAttrMultiProcessorCount, device);
    });
    if (info.sm_error != cudaSuccess) {
        fail(message, capacity, 1, "cudaDeviceGetAttribute failed: %s", cudaGetErrorString(info.sm_error));
        return false;
    }
    *sm_count = info.sm_count;
    return true;
}

bool deviceStatusWord(int device, int** device_pointer, volatile int** host_pointer, char* message,
                      std::size_t capacity) {
    if (device < 0 || device >= kMaxDevices) {
        fail(message, capacity, 1, "device %d is out of range", device);
        return false;
    }
    DeviceInfo& info = deviceInfo(device);
    std::call_once(info.status_once, [&] {
        // Mapped pinned memory: the kernels can write it, the host can read it
        // without synchronising any stream. Allocated once per device; the
        // device that is current when a Plan is configured is `device`.
        void* host        = nullptr;
        info.status_error = cudaHostAlloc(&host, 64, cudaHostAllocMapped | cudaHostAllocPortable);
        if (info.status_error != cudaSuccess) { return; }
        info.status_host    = static_cast<int*>(host);
        info.status_host[0] = 0;
        void* device_side   = nullptr;
        info.status_error   = cudaHostGetDevicePointer(&device_side, host, 0);
        info.status_device  = static_cast<int*>(device_side);
    });
    if (info.status_error != cudaSuccess) {
        fail(message, capacity, 1, "allocating the device status word failed: %s",
             cudaGetErrorString(info.status_error));
        return false;
    }
    *device_pointer = info.status_device;
    *host_pointer   = info.status_host;
    return true;
}

bool tmaEligible(const void* base, std::int64_t contiguous_stride, std::int64_t other_stride,
                 std::uint64_t contiguous_extent, std::uint64_t other_extent) {
    if (base == nullptr || contiguous_stride != 1 || other_stride <= 0) { return false; }
    if (reinterpret_cast<std::uintptr_t>(base) % 16 != 0) { return false; }
    if (contiguous_extent == 0 || other_extent == 0) { return false; }
    if (contiguous_extent >= (1ULL << 32) || other_extent >= (1ULL << 32)) { return false; }
    const std::uint64_t pitch = static_cast<std::uint64_t>(other_stride) * sizeof(float);
    if (pitch % 16 != 0 || pitch >= (1ULL << 40)) { return false; }
    // Rows must not overlap: the descriptor describes a plain 2-D array.
    return static_cast<std::uint64_t>(other_stride) >= contiguous_extent;
}

bool encodeTensorMap2d(CUtensorMap* map, const void* base, std::uint64_t inner, std::uint64_t outer,
                       std::uint64_t row_pitch_bytes, std::uint32_t box_inner, std::uint32_t box_outer,
                       int swizzle, char* message, std::size_t capacity) {
    const PFN_cuTensorMapEncodeTiled_v12000 encode = tensorMapEncoder();
    if (encode == nullptr) {
        fail(message, capacity, 1, "the CUDA driver does not provide cuTensorMapEncodeTiled");
        return false;
    }
    const cuuint64_t dims[2]     = {inner, outer};
    const cuuint64_t strides[1]  = {row_pitch_bytes};
    const cuuint32_t box[2]      = {box_inner, box_outer};
    const cuuint32_t elements[2] = {1, 1};
    const CUresult result        = encode(
        map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box, elements,
        CU_TENSOR_MAP_INTERLEAVE_NONE,
        swizzle == kSwizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B
                               : swizzle == kSwizzle128Atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_NONE,
        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (result != CUDA_SUCCESS) {
        fail(message, capacity, 1, "cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(result));
        return false;
    }
    return true;
}

void countLaunches(std::uint64_t launches) { g_launches.fetch_add(launches, std::memory_order_relaxed); }

}  // namespace ftcuda

extern "C" int ftcuda_current_device(int32_t* device, char* message, size_t message_capacity) {
    int current             = 0;
    const cudaError_t error = cudaGetDevice(&current);
    if (error != cudaSuccess) { return ftcuda::fail(message, message_capacity, 1, "%s", cudaGetErrorString(error)); }
    *device = current;
    return 0;
}

extern "C" int ftcuda_device_sm_count(int32_t device, int32_t* sm_count, char* message, size_t message_capacity) {
    int count = 0;
    if (!ftcuda::deviceSmCount(device, &count, message, message_capacity)) { return 1; }
    *sm_count = count;
    return 0;
}

extern "C" int ftcuda_device_status(int32_t device, int32_t* code, char* message, size_t message_capacity) {
    if (code == nullptr) { return ftcuda::fail(message, message_capacity, 1, "null argument"); }
    int* device_side          = nullptr;
    volatile int* host_side   = nullptr;
    if (!ftcuda::deviceStatusWord(device, &device_side, &host_side, message, message_capacity)) { return 1; }
    *code = *host_side;
    return 0;
}

extern "C" int ftcuda_device_status_reset(int32_t device, char* message, size_t message_capacity) {
    int* device_side        = nullptr;
    volatile int* host_side = nullptr;
    if (!ftcuda::deviceStatusWord(device, &device_side, &host_side, message, message_capacity)) { return 1; }
    *host_side = 0;
    return 0;
}

extern "C" int ftcuda_selftest_bounded_wait(int32_t device, uint64_t budget_ns, void* stream, char* message,
                                            size_t message_capacity) {
    if (budget_ns > 1000000000ULL) { return ftcuda::fail(message, message_capacity, 1, "the budget is at most one second"); }
    int current       = -1;
    cudaError_t error = cudaGetDevice(&current);
    if (error != cudaSuccess) { return ftcuda::fail(message, message_capacity, 1, "%s", cudaGetErrorString(error)); }
    if (current != device) { return ftcuda::fail(message, message_capacity, 1, "device %d must be current", device); }
    int* device_side        = nullptr;
    volatile int* host_side = nullptr;
    if (!ftcuda::deviceStatusWord(device, &device_side, &host_side, message, message_capacity)) { return 1; }
    ftcuda::boundedWaitProbe<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(device_side, budget_ns);
    error = cudaGetLastError();
    if (error != cudaSuccess) { return ftcuda::fail(message, message_capacity, 1, "%s", cudaGetErrorString(error)); }
    return 0;
}

extern "C" int ftcuda_measure_ffma_tflops(int32_t device, double* tflops, char* message, size_t message_capacity) {
    if (tflops == nullptr) { return ftcuda::fail(message, message_capacity, 1, "null argument"); }
    int current       = -1;
    cudaError_t error = cudaGetDevice(&current);
    if (error != cudaSuccess) { return ftcuda::fail(message, message_capacity, 1, "%s", cudaGetErrorString(error)); }
    if (current != device) { return ftcuda::fail(message, message_capacity, 1, "device %d must be current", device); }
    int sms = 0;
    if (!ftcuda::deviceSmCount(device, &sms, message, message_capacity)) { return 1; }
    cudaEvent_t begin = nullptr, end = nullptr;
    if ((error = cudaEventCreate(&begin)) != cudaSuccess || (error = cudaEventCreate(&end)) != cudaSuccess) {
        if (begin != nullptr) { cudaEventDestroy(begin); }
        return ftcuda::fail(message, message_capacity, 1, "%s", cudaGetErrorString(error));
    }
    constexpr int kTrips = 4096;                 // x 32 FFMAs per thread
    const int blocks     = 2 * sms;              // 2048 threads per SM
    double best_ms       = 0.0;
    for (int attempt = 0; attempt < 4 && error == cudaSuccess; ++attempt) {  // the first launch warms up
        cudaEventRecord(begin, nullptr);
        ftcuda::ffmaRateProbe<<<blocks, 1024>>>(nullptr, 0.999F, 1e-3F, kTrips);
        cudaEventRecord(end, nullptr);
        error = cudaEventSynchronize(end);
        float ms = 0.0F;
        if (error == cudaSuccess) { error = cudaEventElapsedTime(&ms, begin, end); }
        if (attempt > 0 && (best_ms == 0.0 || ms < best_ms)) { best_ms = ms; }
    }
    cudaEventDestroy(begin);
    cudaEventDestroy(end);
    if (error != cudaSuccess || best_ms <= 0.0) {
        return ftcuda::fail(message, message_capacity, 1, "FFMA probe failed: %s", cudaGetErrorString(error));
    }
    const double flops = 2.0 * 32.0 * kTrips * 1024.0 * blocks;
    *tflops            = flops / (best_ms * 1e-3) / 1e12;
    return 0;
}

extern "C" uint64_t ftcuda_launch_count(void) { return ftcuda::g_launches.load(std::memory_order_relaxed); }

extern "C" int ftcuda_trace_push(const char* name) { return nvtxRangePushA(name) >= 0 ? 1 : 0; }

extern "C" void ftcuda_trace_pop(void) { nvtxRangePop(); }

extern "C" void ftcuda_trace_mark(const char* name) { nvtxMarkA(name); }
