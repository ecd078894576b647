// ORACLE -- TEST INFRASTRUCTURE ONLY.
// Lets the reference's kernel source (a .hip file that is plain C++ inside the
// kernel body) run on the CPU: a launch walks the grid, block by block and
// thread by thread, setting the built-in index variables before each call of
// the kernel function. Blocks are spread over the host's cores.
#ifndef FTREF_HIP_RUNTIME_H_
#define FTREF_HIP_RUNTIME_H_

#include <algorithm>
#include <thread>
#include <vector>

#include "hip/hip_runtime_api.h"

struct dim3 {
    unsigned x, y, z;
    constexpr dim3(unsigned x_ = 1, unsigned y_ = 1, unsigned z_ = 1) : x(x_), y(y_), z(z_) {}
};

inline thread_local dim3 blockIdx, threadIdx, blockDim, gridDim;

#define __global__

template<typename Body>
void ftrefLaunch(dim3 grid, dim3 block, Body body) {
    const unsigned workers = std::max(1U, std::min(std::thread::hardware_concurrency(), grid.x));
    std::vector<std::thread> pool;
    for (unsigned worker = 0; worker < workers; ++worker) {
        pool.emplace_back([=] {
            gridDim  = grid;
            blockDim = block;
            for (unsigned b = worker; b < grid.x; b += workers) {
                blockIdx = dim3(b);
                for (unsigned t = 0; t < block.x; ++t) {
                    threadIdx = dim3(t);
                    body();
                }
            }
        });
    }
    for (std::thread& thread : pool) { thread.join(); }
}

#define hipLaunchKernelGGL(kernel, grid, block, shared_bytes, stream, ...) \
    ftrefLaunch((grid), (block), [=] { kernel(__VA_ARGS__); })

#endif
