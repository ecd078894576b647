// extern "C" Ops matching and Args binding. Reference: src/api/ops_args_api.cpp:16-203.
#include <memory>
#include <optional>
#include <vector>

#include "api/api_support.hpp"
#include "core/handle.hpp"
#include "core/trace.hpp"

using ftrain::Exception;
using ftrain::invokeApi;
using ftrain::OperandKind;
using ftrain::OperationKind;
using ftrain::requireNonNull;
using ftrain::StorageView;

namespace {

FTrainStatus setComputeType(FTrainArgs args, std::uint64_t op, OperationKind kind, FTrainNumericType compute_type,
                            const char* function) {
    return invokeApi([&] {
        requireNonNull(args, function, "args handle");
        if (compute_type == FTRAIN_NUMERIC_TYPE_INVALID || compute_type >= FTRAIN_NUMERIC_TYPE_COUNT) {
            throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT, "%s: compute_type %u is invalid", function,
                            static_cast<unsigned>(compute_type));
        }
        args->args.setOperation(op, ftrain::OperationValue{kind, compute_type});
    });
}

std::vector<StorageView> copyViews(const FTrainStorageView* views, std::size_t count) {
    std::vector<StorageView> copies;
    if (views == nullptr) { return copies; }
    copies.reserve(count);
    for (std::size_t i = 0; i < count; ++i) { copies.emplace_back(views[i]); }
    return copies;
}

}  // namespace

extern "C" FTrainStatus ftrainOpsCreate(FTrainOps* ops, FTrainPattern pattern) {
    ftrain::ScopedTraceRange trace("ftrainOpsCreate");
    return invokeApi([&] {
        requireNonNull(ops, "ftrainOpsCreate", "ops output");
        requireNonNull(pattern, "ftrainOpsCreate", "pattern");
        const ftrain::Pattern built = pattern->builder.build();
        const auto engine           = ftrain::getGlobalHandle().findOpsEngine(built.getKey());
        if (engine == nullptr) {
            throw Exception(FTRAIN_STATUS_UNSUPPORTED,
                            "ftrainOpsCreate: PatternBuilder does not match any registered OpsEngine");
        }
        *ops = new FTrainOpsStruct(ftrain::Ops(built, engine->getPattern()));
    });
}

extern "C" FTrainStatus ftrainOpsDestroy(FTrainOps ops) {
    return invokeApi([&] {
        requireNonNull(ops, "ftrainOpsDestroy", "ops handle");
        delete ops;
    });
}

extern "C" FTrainStatus ftrainArgsCreate(FTrainArgs* args, FTrainOps ops) {
    ftrain::ScopedTraceRange trace("ftrainArgsCreate");
    return invokeApi([&] {
        requireNonNull(args, "ftrainArgsCreate", "args output");
        requireNonNull(ops, "ftrainArgsCreate", "ops handle");
        *args = new FTrainArgsStruct(ops->ops.makeArgs());
    });
}

extern "C" FTrainStatus ftrainArgsDestroy(FTrainArgs args) {
    return invokeApi([&] {
        requireNonNull(args, "ftrainArgsDestroy", "args handle");
        delete args;
    });
}

extern "C" FTrainStatus ftrainArgsSetTensor(FTrainArgs args, FTrainTensorId tensor, FTrainStorageView storage_view) {
    return invokeApi([&] {
        requireNonNull(args, "ftrainArgsSetTensor", "args handle");
        args->args.setOperand(tensor.opaque, OperandKind::kTensor, ftrain::Tensor(StorageView(storage_view)));
    });
}

extern "C" FTrainStatus ftrainArgsSetTensorList(FTrainArgs args, FTrainTensorListId tensor_list,
                                                const FTrainStorageView storage_views[],
                                                std::uint32_t num_storage_views) {
    return invokeApi([&] {
        requireNonNull(args, "ftrainArgsSetTensorList", "args handle");
        if (storage_views == nullptr && num_storage_views != 0) {
            throw Exception(FTRAIN_STATUS_INVALID_ARGUMENT,
                            "ftrainArgsSetTensorList: storage_views must not be null when num_storage_views is %u",
                            num_storage_views);
        }
        args->args.setOperand(tensor_list.opaque, OperandKind::kTensorList,
                              ftrain::TensorList(copyViews(storage_views, num_storage_views)));
    });
}

extern "C" FTrainStatus ftrainArgsSetGroupedTensor(FTrainArgs args, FTrainGroupedTensorId grouped_tensor,
                                                   std::uint32_t num_groups, FTrainStorageView data,
                                                   const FTrainStorageView* offsets,
                                                   const FTrainStorageView dim_sizes[],
                                                   const FTrainStorageView strides[]) {
    return invokeApi([&] {
        requireNonNull(args, "ftrainArgsSetGroupedTensor", "args handle");
        StorageView data_copy(data);
        std::optional<StorageView> offsets_copy;
        if (offsets != nullptr) { offsets_copy.emplace(*offsets); }
        const std::size_t rank = data.num_dims;
        args->args.setOperand(grouped_tensor.opaque, OperandKind::kGroupedTensor,
                              ftrain::GroupedTensor(num_groups, std::move(data_copy), std::move(offsets_copy),
                                                    copyViews(dim_sizes, rank), copyViews(strides, rank)));
    });
}

extern "C" FTrainStatus ftrainArgsSetGemm(FTrainArgs args, FTrainGemmOpId op, FTrainNumericType compute_type) {
    return setComputeType(args, op.opaque, OperationKind::kGemm, compute_type, "ftrainArgsSetGemm");
}

extern "C" FTrainStatus ftrainArgsSetGroupedABCDGemm(FTrainArgs args, FTrainGroupedABCDGemmOpId op,
                                                     FTrainNumericType compute_type) {
    return setComputeType(args, op.opaque, OperationKind::kGroupedABCDGemm, compute_type,
                          "ftrainArgsSetGroupedABCDGemm");
}

extern "C" FTrainStatus ftrainArgsSetGroupedBCDGemm(FTrainArgs args, FTrainGroupedBCDGemmOpId op,
                                                    FTrainNumericType compute_type) {
    return setComputeType(args, op.opaque, OperationKind::kGroupedBCDGemm, compute_type,
                          "ftrainArgsSetGroupedBCDGemm");
}

extern "C" FTrainStatus ftrainArgsSetGroupedABGemm(FTrainArgs args, FTrainGroupedABGemmOpId op,
                                                   FTrainNumericType compute_type) {
    return setComputeType(args, op.opaque, OperationKind::kGroupedABGemm, compute_type, "ftrainArgsSetGroupedABGemm");
}
