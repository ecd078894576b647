// flash_train.torch.gemm: D = alpha * (A @ B) + beta * C on torch's current
// CUDA stream, through the one-shot C entry point ftrainGemm.
//
// Same Python signature and checks as the reference binding
// (python/flash_train/torch/csrc/flash_train_torch.cpp:34-75 and
// flash_train_torch_capi.cpp:11-33 there). Two things are done differently:
// the current stream is asked of c10 directly instead of through a Python call
// (the reference needs that detour because HIP and torch headers clash; the
// public header of this build includes no GPU header), and a failure carries
// the library's diagnostic message, not only the status number.
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>

#include <cstdint>
#include <optional>
#include <string>

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

    const FTrainStatus status =
        ftrainGemm(matrixView(a.data_ptr(), a_dims), matrixView(b.data_ptr(), b_dims),
                   matrixView(c.has_value() ? c->data_ptr() : nullptr, cd_dims), matrixView(d.data_ptr(), cd_dims),
                   hostScalarView(&alpha_value), hostScalarView(&beta_value), FTRAIN_NUMERIC_TYPE_FP32, nullptr, 0,
                   stream);
    TORCH_CHECK(status == FTRAIN_STATUS_SUCCESS, "ftrainGemm failed with status ", static_cast<unsigned>(status), ": ",
                ftrainGetLastMessage());
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
