// ORACLE -- TEST INFRASTRUCTURE ONLY.
// A stand-in for the HIP runtime API, just large enough to compile the
// reference's host sources for the CPU (oracle/build_ref.py). "Device" memory
// is host memory and there is one device, number 0 (or $FTREF_DEVICE).
#ifndef FTREF_HIP_RUNTIME_API_H_
#define FTREF_HIP_RUNTIME_API_H_

#include <cstdlib>

typedef struct ftrefStream* hipStream_t;
typedef int hipError_t;
constexpr hipError_t hipSuccess = 0;

inline hipError_t hipGetDevice(int* device) {
    const char* chosen = std::getenv("FTREF_DEVICE");
    *device            = chosen != nullptr ? std::atoi(chosen) : 0;
    return hipSuccess;
}

inline hipError_t hipGetLastError() { return hipSuccess; }

inline const char* hipGetErrorString(hipError_t) { return "no error"; }

#endif
