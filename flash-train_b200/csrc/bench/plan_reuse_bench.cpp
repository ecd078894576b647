// Host-overhead benchmark of the Plan-reuse path, in C++ so that no binding
// cost is included: one Plan for an m x k x n FP32 GEMM, then `calls`
// back-to-back ftrainPlanExecutePrimitive(plan, index, ...) enqueues with no
// synchronisation inside the loop and one after it (the method of the
// reference's C harness, benchmarks/csrc/ftrain_bench.cpp:26-80 there, tier L3).
// Prints one JSON object: host microseconds per call (wall clock of the
// enqueue loop / calls) and device microseconds per call (CUDA events).
//
//   plan_reuse_bench [m k n calls primitive_index]
#include <cuda_runtime_api.h>

#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>

#include <flash_train/flash_train.h>

namespace {

#define CUDA_OK(call)                                                                     \
    do {                                                                                  \
        const cudaError_t error_ = (call);                                                \
        if (error_ != cudaSuccess) {                                                      \
            std::fprintf(stderr, "%s failed: %s\n", #call, cudaGetErrorString(error_));   \
            return 2;                                                                     \
        }                                                                                 \
    } while (0)

#define FT_OK(call)                                                                                   \
    do {                                                                                              \
        const FTrainStatus status_ = (call);                                                          \
        if (status_ != FTRAIN_STATUS_SUCCESS) {                                                       \
            std::fprintf(stderr, "%s failed with status %u: %s\n", #call, static_cast<unsigned>(status_), \
                         ftrainGetLastMessage());                                                     \
            return 3;                                                                                 \
        }                                                                                             \
    } while (0)

FTrainStorageView matrix(void* memory, const std::int64_t* dims) {
    return FTrainStorageView{memory, dims, nullptr, 2, FTRAIN_NUMERIC_TYPE_FP32, FTRAIN_INDEX_TYPE_CONTINUOUS, false};
}

FTrainStorageView scalar(float* value) {
    return FTrainStorageView{value, nullptr, nullptr, 0, FTRAIN_NUMERIC_TYPE_FP32, FTRAIN_INDEX_TYPE_CONTINUOUS, true};
}

}  // namespace

int main(int argc, char** argv) {
    const std::int64_t m     = argc > 1 ? std::atoll(argv[1]) : 1024;
    const std::int64_t k     = argc > 2 ? std::atoll(argv[2]) : 1024;
    const std::int64_t n     = argc > 3 ? std::atoll(argv[3]) : 1024;
    const int calls          = argc > 4 ? std::atoi(argv[4]) : 1000;
    const std::uint64_t index = argc > 5 ? std::strtoull(argv[5], nullptr, 10) : 0;

    float *a = nullptr, *b = nullptr, *d = nullptr;
    CUDA_OK(cudaMalloc(reinterpret_cast<void**>(&a), sizeof(float) * m * k));
    CUDA_OK(cudaMalloc(reinterpret_cast<void**>(&b), sizeof(float) * k * n));
    CUDA_OK(cudaMalloc(reinterpret_cast<void**>(&d), sizeof(float) * m * n));
    CUDA_OK(cudaMemset(a, 0, sizeof(float) * m * k));
    CUDA_OK(cudaMemset(b, 0, sizeof(float) * k * n));
    cudaStream_t stream = nullptr;
    CUDA_OK(cudaStreamCreate(&stream));

    FTrainPattern pattern = nullptr;
    FTrainTensorId ra, rb, rc, rd, ralpha, rbeta;
    FTrainGemmOpId gemm;
    FT_OK(ftrainPatternCreate(&pattern));
    FT_OK(ftrainPatternAddTensor(pattern, &ra));
    FT_OK(ftrainPatternAddTensor(pattern, &rb));
    FT_OK(ftrainPatternAddTensor(pattern, &rc));
    FT_OK(ftrainPatternAddTensor(pattern, &rd));
    FT_OK(ftrainPatternAddTensor(pattern, &ralpha));
    FT_OK(ftrainPatternAddTensor(pattern, &rbeta));
    FT_OK(ftrainPatternAddGemm(pattern, &gemm, ra, rb, rc, rd, ralpha, rbeta));
    FTrainOps ops = nullptr;
    FT_OK(ftrainOpsCreate(&ops, pattern));
    FTrainArgs args = nullptr;
    FT_OK(ftrainArgsCreate(&args, ops));
    const std::int64_t a_dims[2] = {m, k}, b_dims[2] = {k, n}, d_dims[2] = {m, n};
    float alpha = 1.0F, beta = 0.0F;
    FT_OK(ftrainArgsSetTensor(args, ra, matrix(a, a_dims)));
    FT_OK(ftrainArgsSetTensor(args, rb, matrix(b, b_dims)));
    FT_OK(ftrainArgsSetTensor(args, rc, matrix(nullptr, d_dims)));
    FT_OK(ftrainArgsSetTensor(args, rd, matrix(d, d_dims)));
    FT_OK(ftrainArgsSetTensor(args, ralpha, scalar(&alpha)));
    FT_OK(ftrainArgsSetTensor(args, rbeta, scalar(&beta)));
    FT_OK(ftrainArgsSetGemm(args, gemm, FTRAIN_NUMERIC_TYPE_FP32));

    // Plan creation cost, first (selection) and second (cache hit).
    FTrainPlan plan = nullptr;
    auto tick       = std::chrono::steady_clock::now();
    FT_OK(ftrainPlanCreate(&plan, args));
    const double first_create_us = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - tick).count();
    FT_OK(ftrainPlanDestroy(plan));
    tick = std::chrono::steady_clock::now();
    for (int i = 0; i < 100; ++i) {
        FT_OK(ftrainPlanCreate(&plan, args));
        if (i != 99) { FT_OK(ftrainPlanDestroy(plan)); }
    }
    const double cached_create_us =
        std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - tick).count() / 100.0;

    const char* name = nullptr;
    FT_OK(ftrainPlanGetPrimitiveName(plan, index, &name));
    std::uint64_t workspace_bytes = 0;
    FT_OK(ftrainPlanGetPrimitiveRequiredWorkspaceBytes(plan, index, &workspace_bytes));
    void* workspace = nullptr;
    if (workspace_bytes != 0) { CUDA_OK(cudaMalloc(&workspace, workspace_bytes)); }

    for (int i = 0; i < 50; ++i) { FT_OK(ftrainPlanExecutePrimitive(plan, index, workspace, workspace_bytes, stream)); }
    CUDA_OK(cudaStreamSynchronize(stream));
    cudaEvent_t begin, end;
    CUDA_OK(cudaEventCreate(&begin));
    CUDA_OK(cudaEventCreate(&end));
    CUDA_OK(cudaEventRecord(begin, stream));
    tick = std::chrono::steady_clock::now();
    for (int i = 0; i < calls; ++i) {
        if (ftrainPlanExecutePrimitive(plan, index, workspace, workspace_bytes, stream) != FTRAIN_STATUS_SUCCESS) {
            std::fprintf(stderr, "execute failed: %s\n", ftrainGetLastMessage());
            return 3;
        }
    }
    const double host_us = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - tick).count();
    CUDA_OK(cudaEventRecord(end, stream));
    CUDA_OK(cudaStreamSynchronize(stream));
    float device_ms = 0.0F;
    CUDA_OK(cudaEventElapsedTime(&device_ms, begin, end));

    // The one-shot call, for the per-call cost of Args + Plan on top (tier L2).
    tick = std::chrono::steady_clock::now();
    for (int i = 0; i < calls; ++i) {
        if (ftrainGemm(matrix(a, a_dims), matrix(b, b_dims), matrix(nullptr, d_dims), matrix(d, d_dims), scalar(&alpha),
                       scalar(&beta), FTRAIN_NUMERIC_TYPE_FP32, workspace, workspace_bytes, stream) != FTRAIN_STATUS_SUCCESS) {
            std::fprintf(stderr, "ftrainGemm failed: %s\n", ftrainGetLastMessage());
            return 3;
        }
    }
    const double one_shot_us = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - tick).count();
    CUDA_OK(cudaStreamSynchronize(stream));

    std::printf(
        "{\"m\": %lld, \"k\": %lld, \"n\": %lld, \"calls\": %d, \"primitive\": \"%s\", \"workspace_bytes\": %llu, "
        "\"plan_reuse_host_us_per_call\": %.3f, \"device_us_per_call\": %.3f, \"one_shot_host_us_per_call\": %.3f, "
        "\"plan_create_first_us\": %.1f, \"plan_create_cached_us\": %.2f}\n",
        static_cast<long long>(m), static_cast<long long>(k), static_cast<long long>(n), calls, name,
        static_cast<unsigned long long>(workspace_bytes), host_us / calls, device_ms * 1000.0 / calls, one_shot_us / calls,
        first_create_us, cached_create_us);
    ftrainPlanDestroy(plan);
    ftrainArgsDestroy(args);
    ftrainOpsDestroy(ops);
    ftrainPatternDestroy(pattern);
    return 0;
}
