/*
 * flash_train/control.h -- build-time switches of the B200 build.
 *
 * Mirrors the role of the reference's generated control.h
 * (include/flash_train/control.h.in:7-28): it defines the FTRAIN_API export
 * macro and names the platform the library was built for. The reference
 * generates the file with CMake for FTRAIN_PLATFORM_HYGON_HIP; this build has
 * exactly one platform, NVIDIA CUDA on sm_100a, so the file is static.
 */
#ifndef FTRAIN_CONTROL_H_
#define FTRAIN_CONTROL_H_

#if defined(FTRAIN_STATIC)
#    define FTRAIN_API
#elif defined(_WIN32)
#    if defined(FTRAIN_BUILDING)
#        define FTRAIN_API __declspec(dllexport)
#    else
#        define FTRAIN_API __declspec(dllimport)
#    endif
#elif defined(__GNUC__) || defined(__clang__)
#    define FTRAIN_API __attribute__((visibility("default")))
#else
#    error "flash_train needs GCC or Clang on non-Windows targets"
#endif

/* The reference's only platform macro stays defined (as 0) so that code written
 * against the reference header keeps preprocessing. */
#define FTRAIN_PLATFORM_HYGON_HIP 0
#define FTRAIN_HYGON_HIP_ARCHS ""

/* The platform of this build. */
#define FTRAIN_PLATFORM_NVIDIA_CUDA 1
#define FTRAIN_NVIDIA_CUDA_ARCHS "sm_100a"

#endif
