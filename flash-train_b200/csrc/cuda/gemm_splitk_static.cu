// ftcuda_gemm_splitk_static: the exact-FP32 split-K GEMM for callers that have
// no workspace to hand over and are not allowed to allocate one.
//
// Who that is. The library's normal contract is "the caller brings the
// workspace" (ftrainPlanGetPrimitiveRequiredWorkspaceBytes, then a buffer of
// that size). Some callers cannot honour it: code that runs after a framework
// has reserved all device memory for its own pool, so that cudaMalloc would
// fail; code on a latency-critical path where the implicit device-wide
// synchronisation of cudaMalloc / cudaFree is not acceptable; and thin bindings
// that were written against the reference's single workspace-free kernel and
// always pass a null workspace. For them this entry point keeps the split-K
// partial sums in memory that belongs to the library image itself.
//
// The scratch is the file-scope array g_scratch below: 16 MiB per GPU, resident
// on every GPU that loads the library until the process exits. Requests whose
// partial sums (slices x m x n floats) do not fit are refused with a message;
// nothing here calls cudaMalloc, cudaFree, cudaHostAlloc or any other
// allocating routine.
//
// Sharing rules. All calls on one GPU use the same array. The array keeps
// whatever the previous call left in it, which is harmless: the first pass
// writes every partial element that the second pass reads, so nothing has to
// start at zero and nothing is cleared. Two calls whose kernels can overlap on
// the GPU (different streams, or different host threads on different streams)
// would overwrite each other's partial sums: callers must order them, for
// instance by using one stream.
//
// Set-up. The first call on a device looks up the device address of the array
// with cudaGetSymbolAddress while that device is current, and remembers it; a
// name like g_scratch is a device symbol, and in host code it is only a
// stand-in, not an address a kernel could use. Make that first call outside of
// any stream capture.
#include <cuda_runtime.h>

#include <cstdint>
#include <mutex>

#include "gemm_kernels.hpp"

namespace {

constexpr std::uint64_t kScratchBytes  = 16ULL << 20;
constexpr std::uint64_t kScratchFloats = kScratchBytes / sizeof(float);
constexpr int kMaxDevices              = 64;

static __device__ __align__(256) float g_scratch[kScratchFloats];

struct DeviceScratch {
    std::mutex mutex;
    bool resolved  = false;
    float* address = nullptr;
};

DeviceScratch g_device_scratch[kMaxDevices];

// The device address of g_scratch on `device`, which must be current. Only a successful lookup is
// remembered: one that failed (for instance because the first call came during a stream capture)
// is tried again by the next call, and the error it left in the runtime is cleared.
cudaError_t scratchAddress(int device, float** address) {
    DeviceScratch& slot = g_device_scratch[device];
    std::lock_guard<std::mutex> guard(slot.mutex);
    if (!slot.resolved) {
        void* pointer           = nullptr;
        const cudaError_t error = cudaGetSymbolAddress(&pointer, g_scratch);
        if (error != cudaSuccess || pointer == nullptr) {
            (void)cudaGetLastError();
            *address = nullptr;
            return error != cudaSuccess ? error : cudaErrorInvalidSymbol;
        }
        slot.address  = static_cast<float*>(pointer);
        slot.resolved = true;
    }
    *address = slot.address;
    return cudaSuccess;
}

// True once the array's address on `device` is known (no lookup is needed any more).
bool scratchResolved(int device) {
    DeviceScratch& slot = g_device_scratch[device];
    std::lock_guard<std::mutex> guard(slot.mutex);
    return slot.resolved;
}

}  // namespace

extern "C" uint64_t ftcuda_gemm_splitk_static_capacity(void) { return kScratchBytes; }

extern "C" int ftcuda_gemm_splitk_static(const FtcudaGemmDesc* desc, void* stream, char* message,
                                         size_t message_capacity) {
    using ftcuda::fail;
    if (desc == nullptr) { return fail(message, message_capacity, 1, "null descriptor"); }
    if (desc->m * desc->n == 0) { return 0; }
    const char* reason = ftcuda::supportsSimt(*desc, true);
    if (reason != nullptr) { return fail(message, message_capacity, 1, "%s", reason); }
    if (desc->d == nullptr || desc->a == nullptr || desc->b == nullptr) {
        return fail(message, message_capacity, 1, "a required operand address is null");
    }
    if (desc->device < 0 || desc->device >= kMaxDevices) {
        return fail(message, message_capacity, 1, "device %d is out of range", desc->device);
    }
    int current       = -1;
    cudaError_t error = cudaGetDevice(&current);
    if (error != cudaSuccess) { return fail(message, message_capacity, 1, "%s", cudaGetErrorString(error)); }
    if (current != desc->device) {
        return fail(message, message_capacity, 1, "device %d must be current, but device %d is", desc->device, current);
    }

    // As many K slices as give every SM two CTAs, each at least 256 deep, and
    // no more than the static scratch can hold.
    const std::uint64_t slab   = desc->m * desc->n;
    const std::uint64_t fit    = kScratchFloats / slab;
    if (fit < 2) {
        return fail(message, message_capacity, 1,
                    "m * n = %llu partial sums per K slice do not fit the %llu-byte static scratch twice "
                    "(limit: m * n <= %llu)",
                    static_cast<unsigned long long>(slab), static_cast<unsigned long long>(kScratchBytes),
                    static_cast<unsigned long long>(kScratchFloats / 2));
    }
    int sms = 0;
    if (!ftcuda::deviceSmCount(desc->device, &sms, message, message_capacity)) { return 1; }
    const std::uint64_t tiles = ftcuda::ceilDiv(desc->m, 64) * ftcuda::ceilDiv(desc->n, 64);
    std::uint64_t splits      = ftcuda::ceilDiv(2ULL * static_cast<std::uint64_t>(sms), tiles);
    if (splits > desc->k / 256) { splits = desc->k / 256; }
    if (splits > 64) { splits = 64; }
    if (splits > fit) { splits = fit; }
    if (splits < 2) { splits = 2; }

    ftcuda::LaunchState state{};
    state.desc   = *desc;
    state.kernel = FTCUDA_GEMM_SIMT_SPLITK;
    ftcuda::planSimtGenericSplitK(state, static_cast<std::uint32_t>(splits));
    if (state.workspace_bytes > kScratchBytes) {
        return fail(message, message_capacity, 1, "internal: %llu bytes of partial sums exceed the static scratch",
                    static_cast<unsigned long long>(state.workspace_bytes));
    }

    // The first call on a device looks the array up, which is not allowed while the stream is being
    // captured: say so instead of invalidating the capture.
    if (!scratchResolved(desc->device)) {
        cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(static_cast<cudaStream_t>(stream), &capture) != cudaSuccess) { (void)cudaGetLastError(); }
        if (capture != cudaStreamCaptureStatusNone) {
            return fail(message, message_capacity, 1,
                        "the first call on a device resolves the static scratch and must come before stream capture");
        }
    }
    float* scratch = nullptr;
    error          = scratchAddress(desc->device, &scratch);
    if (error != cudaSuccess || scratch == nullptr) {
        return fail(message, message_capacity, 1, "cudaGetSymbolAddress failed: %s", cudaGetErrorString(error));
    }
    error = ftcuda::launchSimt(state, scratch, static_cast<cudaStream_t>(stream));
    if (error != cudaSuccess) { return fail(message, message_capacity, 1, "%s", cudaGetErrorString(error)); }
    return 0;
}
