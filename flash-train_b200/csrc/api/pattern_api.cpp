// extern "C" Pattern construction. Reference: src/api/pattern_api.cpp:9-133.
// Role ids are the builder's 0-based insertion indices; nothing is validated
// until ftrainOpsCreate.
#include <memory>

#include "api/api_support.hpp"

using ftrain::invokeApi;
using ftrain::OperandKind;
using ftrain::OperationKind;
using ftrain::requireNonNull;

namespace {

template<typename Id>
FTrainStatus addOperand(FTrainPattern pattern, Id* out, OperandKind kind, const char* function, const char* out_name) {
    return invokeApi([&] {
        requireNonNull(pattern, function, "pattern");
        requireNonNull(out, function, out_name);
        out->opaque = pattern->builder.addOperand(kind);
    });
}

// Every GEMM node kind has inputs (a, b, c, alpha, beta) and output (d).
template<typename Id>
FTrainStatus addGemmLike(FTrainPattern pattern, Id* out, OperationKind kind, const char* function, std::uint64_t a,
                         std::uint64_t b, std::uint64_t c, std::uint64_t d, std::uint64_t alpha, std::uint64_t beta) {
    return invokeApi([&] {
        requireNonNull(pattern, function, "pattern");
        requireNonNull(out, function, "op output");
        out->opaque = pattern->builder.addOperation(kind, {a, b, c, alpha, beta}, {d});
    });
}

}  // namespace

extern "C" FTrainStatus ftrainPatternCreate(FTrainPattern* pattern) {
    return invokeApi([&] {
        requireNonNull(pattern, "ftrainPatternCreate", "pattern output");
        *pattern = new FTrainPatternStruct();
    });
}

extern "C" FTrainStatus ftrainPatternDestroy(FTrainPattern pattern) {
    return invokeApi([&] {
        requireNonNull(pattern, "ftrainPatternDestroy", "pattern");
        delete pattern;
    });
}

extern "C" FTrainStatus ftrainPatternAddTensor(FTrainPattern pattern, FTrainTensorId* tensor) {
    return addOperand(pattern, tensor, OperandKind::kTensor, "ftrainPatternAddTensor", "tensor output");
}

extern "C" FTrainStatus ftrainPatternAddTensorList(FTrainPattern pattern, FTrainTensorListId* tensor_list) {
    return addOperand(pattern, tensor_list, OperandKind::kTensorList, "ftrainPatternAddTensorList",
                      "tensor_list output");
}

extern "C" FTrainStatus ftrainPatternAddGroupedTensor(FTrainPattern pattern, FTrainGroupedTensorId* grouped_tensor) {
    return addOperand(pattern, grouped_tensor, OperandKind::kGroupedTensor, "ftrainPatternAddGroupedTensor",
                      "grouped_tensor output");
}

extern "C" FTrainStatus ftrainPatternAddGemm(FTrainPattern pattern, FTrainGemmOpId* op, FTrainTensorId a,
                                             FTrainTensorId b, FTrainTensorId c, FTrainTensorId d, FTrainTensorId alpha,
                                             FTrainTensorId beta) {
    return addGemmLike(pattern, op, OperationKind::kGemm, "ftrainPatternAddGemm", a.opaque, b.opaque, c.opaque,
                       d.opaque, alpha.opaque, beta.opaque);
}

extern "C" FTrainStatus ftrainPatternAddGroupedABCDGemm(FTrainPattern pattern, FTrainGroupedABCDGemmOpId* op,
                                                        FTrainGroupedTensorId a, FTrainGroupedTensorId b,
                                                        FTrainGroupedTensorId c, FTrainGroupedTensorId d,
                                                        FTrainTensorId alpha, FTrainTensorId beta) {
    return addGemmLike(pattern, op, OperationKind::kGroupedABCDGemm, "ftrainPatternAddGroupedABCDGemm", a.opaque,
                       b.opaque, c.opaque, d.opaque, alpha.opaque, beta.opaque);
}

extern "C" FTrainStatus ftrainPatternAddGroupedBCDGemm(FTrainPattern pattern, FTrainGroupedBCDGemmOpId* op,
                                                       FTrainTensorListId a, FTrainGroupedTensorId b,
                                                       FTrainGroupedTensorId c, FTrainGroupedTensorId d,
                                                       FTrainTensorId alpha, FTrainTensorId beta) {
    return addGemmLike(pattern, op, OperationKind::kGroupedBCDGemm, "ftrainPatternAddGroupedBCDGemm", a.opaque,
                       b.opaque, c.opaque, d.opaque, alpha.opaque, beta.opaque);
}

extern "C" FTrainStatus ftrainPatternAddGroupedABGemm(FTrainPattern pattern, FTrainGroupedABGemmOpId* op,
                                                      FTrainGroupedTensorId a, FTrainGroupedTensorId b,
                                                      FTrainTensorListId c, FTrainTensorListId d, FTrainTensorId alpha,
                                                      FTrainTensorId beta) {
    return addGemmLike(pattern, op, OperationKind::kGroupedABGemm, "ftrainPatternAddGroupedABGemm", a.opaque, b.opaque,
                       c.opaque, d.opaque, alpha.opaque, beta.opaque);
}
