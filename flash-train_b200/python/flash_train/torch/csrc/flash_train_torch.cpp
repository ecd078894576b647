// flash_train.torch.gemm: D = alpha * (A @ B) + beta * C on torch's current
// CUDA stream.
//
// Same Python signature and checks as the reference binding
// (python/flash_train/torch/csrc/flash_train_torch.cpp:34-75 and
// flash_train_torch_capi.cpp:11-33 there). Three things are done differently:
//   * the current stream is asked of c10 directly instead of through a Python
//     call (the reference needs that detour because HIP and torch headers
//     clash; the public header of this build includes no GPU header);
//   * the reference calls ftrainGemm with no workspace, which is enough for its
//     one workspace-free kernel. Here the recommended Primitive can be a
//     split-K kernel that needs one, so the binding makes the same staged calls
//     ftrainGemm makes (Args, Plan, execute primitive 0) and, in between, asks
//     the Plan how much workspace primitive 0 wants and takes it from torch's
//     caching allocator;
//   * a failure carries the library's diagnostic message, not only the status;
//   * the Plans of recent calls are kept per thread (64, least recently used out first), keyed by
//     the four addresses, the shape, alpha, beta and the device: a training loop that calls with
//     the same tensors again executes the kept Plan and skips Args and Plan creation. The output
//     tensor comes from torch's caching allocator, which hands a loop the same blocks again and
//     again. FTRAIN_DISABLE_CACHE switches this off together with the library's selection cache.
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>

#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <optional>
#include <string>

#include <flash_train/env.h>
#include <flash_train/flash_train.h>

namespace {

void checkMatrix(const at::Tensor& tensor, const char* name) {
    TORCH_CHECK(tensor.is_cuda(), name, " must be a device tensor");
    TORCH_CHECK(tensor.scalar_type() == at::kFloat, name, " must be FP32");
    TORCH_CHECK(tensor.dim() == 2, name, " must be rank two");
    TORCH_CHECK(tensor.is_contiguous(), name, " must be contiguous");
}

FTrainStorageView matrixView(const void* memory, const std::int64_t* dims) {
    return FTrainStorageView{const_cast<void*>(memory), dims, nullptr, 2, FTRAIN_NUMERIC_TYPE_FP32,
                             FTRAIN_INDEX_TYPE_CONTINUOUS, false};
}

FTrainStorageView hostScalarView(const float* value) {
    return FTrainStorageView{const_cast<float*>(value), nullptr, nullptr, 0, FTRAIN_NUMERIC_TYPE_FP32,
                             FTRAIN_INDEX_TYPE_CONTINUOUS, true};
}

// Pattern -> Ops for the Gemm graph, made once per process (what ftrainGemm
// keeps internally, src/api/gemm_api.cpp:28-49 of the reference).
struct GemmRoles {
    FTrainOps ops{nullptr};
    FTrainTensorId a{}, b{}, c{}, d{}, alpha{}, beta{};
    FTrainGemmOpId gemm{};
    FTrainStatus status{FTRAIN_STATUS_SUCCESS};
};

const GemmRoles& gemmRoles() {
    static const GemmRoles roles = [] {
        GemmRoles made;
        FTrainPattern pattern         = nullptr;
        FTrainStatus status           = ftrainPatternCreate(&pattern);
        FTrainTensorId* const order[] = {&made.a, &made.b, &made.c, &made.alpha, &made.beta, &made.d};
        for (FTrainTensorId* role : order) {
            if (status == FTRAIN_STATUS_SUCCESS) { status = ftrainPatternAddTensor(pattern, role); }
        }
        if (status == FTRAIN_STATUS_SUCCESS) {
            status = ftrainPatternAddGemm(pattern, &made.gemm, made.a, made.b, made.c, made.d, made.alpha, made.beta);
        }
        if (status == FTRAIN_STATUS_SUCCESS) { status = ftrainOpsCreate(&made.ops, pattern); }
        if (pattern != nullptr) { ftrainPatternDestroy(pattern); }
        made.status = status;
        return made;
    }();
    return roles;
}

// Plans of this thread's recent calls. Everything a Plan depends on is in the key.
struct CallKey {
    const void* a;
    const void* b;
    const void* c;
    const void* d;
    std::int64_t m, k, n;
    float alpha, beta;
    std::int32_t device;
    std::int32_t zero;  // explicit padding: keys are compared bytewise
};

class RecentPlans final {
  public:
    struct Entry {
        CallKey key{};
        FTrainPlan plan               = nullptr;
        std::uint64_t workspace_bytes = 0;
        std::uint64_t last_use        = 0;
    };

    ~RecentPlans() {
        for (Entry& entry : entries_) {
            if (entry.plan != nullptr) { ftrainPlanDestroy(entry.plan); }
        }
    }

    Entry* find(const CallKey& key) noexcept {
        for (Entry& entry : entries_) {
            if (entry.plan != nullptr && std::memcmp(&entry.key, &key, sizeof key) == 0) {
                entry.last_use = ++clock_;
                return &entry;
            }
        }
        return nullptr;
    }

    void insert(const CallKey& key, FTrainPlan plan, std::uint64_t workspace_bytes) noexcept {
        Entry* victim = &entries_[0];
        for (Entry& entry : entries_) {
            if (entry.plan == nullptr) {
                victim = &entry;
                break;
            }
            if (entry.last_use < victim->last_use) { victim = &entry; }
        }
        if (victim->plan != nullptr) { ftrainPlanDestroy(victim->plan); }
        *victim = Entry{key, plan, workspace_bytes, ++clock_};
    }

  private:
    Entry entries_[64];
    std::uint64_t clock_ = 0;
};

bool planReuseDisabled() {
    static const bool disabled = [] {
        const char* text = std::getenv(FTRAIN_DISABLE_CACHE);
        if (text == nullptr) { return false; }
        std::string value(text);
        const auto first = value.find_first_not_of(" \t");
        const auto last  = value.find_last_not_of(" \t");
        value            = first == std::string::npos ? std::string() : value.substr(first, last - first + 1);
        return !value.empty() && value != "0";
    }();
    return disabled;
}

at::Tensor gemm(const at::Tensor& a, const at::Tensor& b, const std::optional<at::Tensor>& c, double alpha,
                double beta) {
    checkMatrix(a, "a");
    checkMatrix(b, "b");
    TORCH_CHECK(a.size(1) == b.size(0), "a's reduction depth must equal b's rows");
    TORCH_CHECK(a.device() == b.device(), "a and b must be on the same device");
    if (c.has_value()) {
        checkMatrix(*c, "c");
        TORCH_CHECK(c->size(0) == a.size(0) && c->size(1) == b.size(1), "c must be shaped m-by-n");
        TORCH_CHECK(c->device() == a.device(), "c must be on a's device");
    }

    // ftrainGemm plans for the calling thread's current device.
    const c10::cuda::CUDAGuard guard(a.device());
    at::Tensor d = torch::empty({a.size(0), b.size(1)}, a.options());

    const std::int64_t a_dims[2]  = {a.size(0), a.size(1)};
    const std::int64_t b_dims[2]  = {b.size(0), b.size(1)};
    const std::int64_t cd_dims[2] = {a.size(0), b.size(1)};
    const float alpha_value       = static_cast<float>(alpha);
    const float beta_value        = static_cast<float>(beta);
    const auto stream = reinterpret_cast<FTrainStream>(c10::cuda::getCurrentCUDAStream(a.device().index()).stream());

    static thread_local RecentPlans recent;
    const bool reuse = !planReuseDisabled();
    CallKey key;
    std::memset(&key, 0, sizeof key);
    key.a      = a.data_ptr();
    key.b      = b.data_ptr();
    key.c      = c.has_value() ? c->data_ptr() : nullptr;
    key.d      = d.data_ptr();
    key.m      = a.size(0);
    key.k      = a.size(1);
    key.n      = b.size(1);
    key.alpha  = alpha_value;
    key.beta   = beta_value;
    key.device = a.device().index();
    if (reuse) {
        if (RecentPlans::Entry* known = recent.find(key)) {
            at::Tensor scratch;
            if (known->workspace_bytes != 0) {
                scratch = torch::empty({static_cast<std::int64_t>(known->workspace_bytes)}, a.options().dtype(at::kByte));
            }
            const FTrainStatus again = ftrainPlanExecutePrimitive(
                known->plan, 0, known->workspace_bytes != 0 ? scratch.data_ptr() : nullptr, known->workspace_bytes, stream);
            TORCH_CHECK(again == FTRAIN_STATUS_SUCCESS, "flash_train gemm failed with status ", static_cast<unsigned>(again), ": ",
                        ftrainGetLastMessage());
            return d;
        }
    }

    const GemmRoles& roles = gemmRoles();
    TORCH_CHECK(roles.status == FTRAIN_STATUS_SUCCESS, "flash_train could not set up its Gemm Ops, status ",
                static_cast<unsigned>(roles.status));
    FTrainArgs args     = nullptr;
    FTrainPlan plan     = nullptr;
    FTrainStatus status = ftrainArgsCreate(&args, roles.ops);
    const struct {
        FTrainTensorId role;
        FTrainStorageView view;
    } bindings[] = {{roles.a, matrixView(a.data_ptr(), a_dims)},
                    {roles.b, matrixView(b.data_ptr(), b_dims)},
                    {roles.c, matrixView(c.has_value() ? c->data_ptr() : nullptr, cd_dims)},
                    {roles.d, matrixView(d.data_ptr(), cd_dims)},
                    {roles.alpha, hostScalarView(&alpha_value)},
                    {roles.beta, hostScalarView(&beta_value)}};
    for (const auto& binding : bindings) {
        if (status == FTRAIN_STATUS_SUCCESS) { status = ftrainArgsSetTensor(args, binding.role, binding.view); }
    }
    if (status == FTRAIN_STATUS_SUCCESS) { status = ftrainArgsSetGemm(args, roles.gemm, FTRAIN_NUMERIC_TYPE_FP32); }
    if (status == FTRAIN_STATUS_SUCCESS) { status = ftrainPlanCreate(&plan, args); }
    std::uint64_t workspace_bytes = 0;
    if (status == FTRAIN_STATUS_SUCCESS) { status = ftrainPlanGetPrimitiveRequiredWorkspaceBytes(plan, 0, &workspace_bytes); }
    at::Tensor workspace;
    if (status == FTRAIN_STATUS_SUCCESS) {
        if (workspace_bytes != 0) {
            workspace = torch::empty({static_cast<std::int64_t>(workspace_bytes)}, a.options().dtype(at::kByte));
        }
        // The caching allocator keeps the block reserved for this stream until
        // the enqueued work is done, so `workspace` may go out of scope below.
        status = ftrainPlanExecutePrimitive(plan, 0, workspace_bytes != 0 ? workspace.data_ptr() : nullptr,
                                            workspace_bytes, stream);
    }
    const std::string failure = status == FTRAIN_STATUS_SUCCESS ? std::string() : std::string(ftrainGetLastMessage());
    if (status == FTRAIN_STATUS_SUCCESS && reuse) {
        recent.insert(key, plan, workspace_bytes);  // kept for the next call with these tensors
        plan = nullptr;
    }
    if (plan != nullptr) { ftrainPlanDestroy(plan); }
    if (args != nullptr) { ftrainArgsDestroy(args); }
    TORCH_CHECK(status == FTRAIN_STATUS_SUCCESS, "flash_train gemm failed with status ", static_cast<unsigned>(status),
                ": ", failure);
    return d;
}

std::string lastMessage() { return ftrainGetLastMessage(); }

}  // namespace

PYBIND11_MODULE(_flash_train_torch, m) {
    m.doc() = "flash-train PyTorch bindings";
    m.def("gemm", &gemm, "d = alpha * (a @ b) + beta * c on the current stream", py::arg("a"), py::arg("b"),
          py::arg("c") = std::nullopt, py::arg("alpha") = 1.0, py::arg("beta") = 0.0);
    m.def("last_message", &lastMessage, "diagnostic message of the calling thread's last failed library call");
}
