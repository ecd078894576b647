// Host-overhead benchmark of the Plan-reuse path, in C++ so that no binding
// cost is included: one Plan for an m x k x n FP32 GEMM, then `calls`
// back-to-back ftrainPlanExecutePrimitive(plan, index, ...) enqueues with no
// synchronisation inside the loop and one after it (the method of the
// reference's C harness, benchmarks/csrc/ftrain_bench.cpp:26-80 there, tier L3).
// Prints one JSON object: host microseconds per call (wall clock of the
// enqueue loop / calls) and device microseconds per call (CUDA events), and, under "tiers", the
// reference suite's tiers timed with the reference suite's policy (warm-up 10, about 200 ms of calls
// clamped to [10, 200], every call between its own pair of events with a synchronise after it,
// median first; benchmarks/ftrain_bench/timing.py:21-44 and benchmarks/README.md:7-14 there):
// L2 the one-shot ftrainGemm, L3 Plan reuse of primitive 0, L4 every primitive of the Plan.
//
//   plan_reuse_bench [m k n calls primitive_index]
#include <cuda_runtime_api.h>

#include <algorithm>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

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

struct Timing {
    double median_us = 0.0, mean_us = 0.0, min_us = 0.0, p10_us = 0.0, p90_us = 0.0;
    int iters        = 0;
    bool ok          = true;
};

// `call` enqueues one unit of work on `stream` and returns false on failure.
template<typename Call>
Timing measureCalls(Call&& call, cudaStream_t stream, cudaEvent_t begin, cudaEvent_t end) {
    Timing timing;
    const auto one = [&](double* microseconds) {
        float ms = 0.0F;
        if (cudaEventRecord(begin, stream) != cudaSuccess || !call() || cudaEventRecord(end, stream) != cudaSuccess ||
            cudaEventSynchronize(end) != cudaSuccess || cudaEventElapsedTime(&ms, begin, end) != cudaSuccess) {
            return false;
        }
        *microseconds = static_cast<double>(ms) * 1e3;
        return true;
    };
    for (int i = 0; i < 10 && timing.ok; ++i) { timing.ok = call(); }
    if (!timing.ok || cudaStreamSynchronize(stream) != cudaSuccess) { return Timing{0, 0, 0, 0, 0, 0, false}; }
    double probe = 0.0;
    if (!one(&probe)) { return Timing{0, 0, 0, 0, 0, 0, false}; }
    const int count = static_cast<int>(std::min(200.0, std::max(10.0, 200e3 / std::max(probe, 1.0) + 1.0)));
    std::vector<double> samples(static_cast<std::size_t>(count));
    for (double& sample : samples) {
        if (!one(&sample)) { return Timing{0, 0, 0, 0, 0, 0, false}; }
    }
    std::sort(samples.begin(), samples.end());
    const auto pick = [&](double fraction) { return samples[static_cast<std::size_t>(fraction * (count - 1) + 0.5)]; };
    double sum = 0.0;
    for (const double sample : samples) { sum += sample; }
    timing.median_us = count % 2 == 1 ? samples[count / 2] : 0.5 * (samples[count / 2 - 1] + samples[count / 2]);
    timing.mean_us   = sum / count;
    timing.min_us    = samples.front();
    timing.p10_us    = pick(0.10);
    timing.p90_us    = pick(0.90);
    timing.iters     = count;
    return timing;
}

std::string timingJson(const Timing& t) {
    char text[256];
    std::snprintf(text, sizeof text, "{\"median_us\": %.3f, \"mean_us\": %.3f, \"min_us\": %.3f, \"p10_us\": %.3f, \"p90_us\": %.3f, \"iters\": %d}",
                  t.median_us, t.mean_us, t.min_us, t.p10_us, t.p90_us, t.iters);
    return text;
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

    // The reference suite's tiers with its timing policy. Every primitive gets the workspace it asks for.
    std::uint64_t primitives = 0;
    FT_OK(ftrainPlanGetNumPrimitives(plan, &primitives));
    std::uint64_t most_bytes = workspace_bytes;
    for (std::uint64_t i = 0; i < primitives; ++i) {
        std::uint64_t bytes = 0;
        FT_OK(ftrainPlanGetPrimitiveRequiredWorkspaceBytes(plan, i, &bytes));
        most_bytes = std::max(most_bytes, bytes);
    }
    void* tier_workspace = nullptr;
    if (most_bytes != 0) { CUDA_OK(cudaMalloc(&tier_workspace, most_bytes)); }
    const Timing one_shot_tier = measureCalls(
        [&] {
            return ftrainGemm(matrix(a, a_dims), matrix(b, b_dims), matrix(nullptr, d_dims), matrix(d, d_dims), scalar(&alpha), scalar(&beta),
                              FTRAIN_NUMERIC_TYPE_FP32, tier_workspace, most_bytes, stream) == FTRAIN_STATUS_SUCCESS;
        },
        stream, begin, end);
    const Timing reuse_tier = measureCalls(
        [&] { return ftrainPlanExecutePrimitive(plan, 0, tier_workspace, most_bytes, stream) == FTRAIN_STATUS_SUCCESS; }, stream, begin, end);
    std::string per_primitive = "{";
    for (std::uint64_t i = 0; i < primitives; ++i) {
        const char* primitive_name = nullptr;
        FT_OK(ftrainPlanGetPrimitiveName(plan, i, &primitive_name));
        const Timing timing = measureCalls(
            [&] { return ftrainPlanExecutePrimitive(plan, i, tier_workspace, most_bytes, stream) == FTRAIN_STATUS_SUCCESS; }, stream, begin, end);
        if (!timing.ok) {
            std::fprintf(stderr, "timing primitive %s failed: %s\n", primitive_name, ftrainGetLastMessage());
            return 3;
        }
        per_primitive += std::string(i != 0 ? ", " : "") + "\"" + primitive_name + "\": " + timingJson(timing);
    }
    per_primitive += "}";
    if (!one_shot_tier.ok || !reuse_tier.ok) {
        std::fprintf(stderr, "timing a tier failed: %s\n", ftrainGetLastMessage());
        return 3;
    }

    std::printf(
        "{\"m\": %lld, \"k\": %lld, \"n\": %lld, \"calls\": %d, \"primitive\": \"%s\", \"workspace_bytes\": %llu, "
        "\"plan_reuse_host_us_per_call\": %.3f, \"device_us_per_call\": %.3f, \"one_shot_host_us_per_call\": %.3f, "
        "\"plan_create_first_us\": %.1f, \"plan_create_cached_us\": %.2f, "
        "\"tiers\": {\"L2_one_shot\": %s, \"L3_plan_reuse\": %s, \"L4_per_primitive\": %s}}\n",
        static_cast<long long>(m), static_cast<long long>(k), static_cast<long long>(n), calls, name,
        static_cast<unsigned long long>(workspace_bytes), host_us / calls, device_ms * 1000.0 / calls, one_shot_us / calls,
        first_create_us, cached_create_us, timingJson(one_shot_tier).c_str(), timingJson(reuse_tier).c_str(), per_primitive.c_str());
    ftrainPlanDestroy(plan);
    ftrainArgsDestroy(args);
    ftrainOpsDestroy(ops);
    ftrainPatternDestroy(pattern);
    return 0;
}
