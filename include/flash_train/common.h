/*
 * flash_train/common.h -- the staged C API: Pattern -> Ops -> Args -> Plan.
 *
 * ABI-compatible with the reference header include/flash_train/common.h
 * (enums :28-74, FTrainStorageView :87-118, role ids :131-137, opaque handles
 * :145-148, functions :162-589). The one platform change: FTrainStream is a
 * CUDA stream (the reference typedefs hipStream_t at :21-24). Both are plain
 * pointers, so every signature keeps its size and calling convention.
 *
 * Life cycle
 *   1. Describe a compute graph with ftrainPatternCreate / ftrainPatternAdd*.
 *   2. ftrainOpsCreate matches it against the supported graphs (the FP32 GEMM
 *      D = alpha*A*B + beta*C is the one supported family).
 *   3. ftrainArgsCreate + ftrainArgsSet* bind concrete storage and attributes.
 *   4. ftrainPlanCreate selects Primitives (kernels) for the current device,
 *      best first; ftrainPlanExecutePrimitive enqueues one of them.
 *
 * Error model: no function throws. Each returns an FTrainStatus and mirrors it,
 * with a message, in thread-local state readable through ftrainGetLastStatus /
 * ftrainGetLastMessage. Output parameters are written only on success.
 */
#ifndef FTRAIN_COMMON_H_
#define FTRAIN_COMMON_H_

#include <stdbool.h>
#include <stdint.h>

#include <flash_train/control.h>
#include <flash_train/version.h>

#ifdef __cplusplus
extern "C" {
#endif

/* A CUDA stream (cudaStream_t / CUstream); declared here without pulling in a
 * CUDA header so C and torch callers need no CUDA include path. */
typedef struct CUstream_st* FTrainStream;
typedef int32_t FTrainDeviceId;

/* ---- enumerations (values fixed by the reference, common.h:28-74) ---- */

typedef uint8_t FTrainStatus;
enum {
    FTRAIN_STATUS_SUCCESS          = 0,
    FTRAIN_STATUS_INVALID_ARGUMENT = 1,
    FTRAIN_STATUS_OUT_OF_MEMORY    = 2,
    FTRAIN_STATUS_OVERFLOW         = 3,
    FTRAIN_STATUS_UNSUPPORTED      = 4,
    FTRAIN_STATUS_INTERNAL_ERROR   = 50,
};

typedef uint8_t FTrainNumericType;
enum {
    FTRAIN_NUMERIC_TYPE_INVALID    = 0,
    FTRAIN_NUMERIC_TYPE_FP64       = 1,
    FTRAIN_NUMERIC_TYPE_INT64      = 2,
    FTRAIN_NUMERIC_TYPE_UINT64     = 3,
    FTRAIN_NUMERIC_TYPE_FP32       = 4,
    FTRAIN_NUMERIC_TYPE_INT32      = 5,
    FTRAIN_NUMERIC_TYPE_UINT32     = 6,
    FTRAIN_NUMERIC_TYPE_FP16       = 7,
    FTRAIN_NUMERIC_TYPE_BF16       = 8,
    FTRAIN_NUMERIC_TYPE_INT16      = 9,
    FTRAIN_NUMERIC_TYPE_UINT16     = 10,
    FTRAIN_NUMERIC_TYPE_FP8_E4M3FN = 11,
    FTRAIN_NUMERIC_TYPE_FP8_E5M2   = 12,
    FTRAIN_NUMERIC_TYPE_UFP8_E8M0  = 13,
    FTRAIN_NUMERIC_TYPE_UFP8_E5M3  = 14,
    FTRAIN_NUMERIC_TYPE_UFP8_E6M2  = 15,
    FTRAIN_NUMERIC_TYPE_INT8       = 16,
    FTRAIN_NUMERIC_TYPE_UINT8      = 17,
    FTRAIN_NUMERIC_TYPE_FP4_E2M1   = 18,
    FTRAIN_NUMERIC_TYPE_FP4_S1P2   = 19,
    FTRAIN_NUMERIC_TYPE_INT4       = 20,
    FTRAIN_NUMERIC_TYPE_UINT4      = 21,
    FTRAIN_NUMERIC_TYPE_UFP1_E1M0  = 22,
    FTRAIN_NUMERIC_TYPE_UINT1      = 23,
    FTRAIN_NUMERIC_TYPE_COUNT,
};

typedef uint8_t FTrainIndexType;
enum {
    /* "No predefined layout": the view's strides array gives the layout. */
    FTRAIN_INDEX_TYPE_INVALID                  = 0,
    /* Dense row-major. */
    FTRAIN_INDEX_TYPE_CONTINUOUS               = 1,
    FTRAIN_INDEX_TYPE_NVIDIA_SF_128X4_SWIZZLED = 2,
    FTRAIN_INDEX_TYPE_GROUPED_CONTINUOUS       = 3,
    FTRAIN_INDEX_TYPE_COUNT,
};

/* ---- storage description (32 bytes on LP64; reference common.h:87-118) ---- */

/*
 * One tensor's address, shape, layout and element type. The library copies the
 * dims/strides arrays during the call that receives the view; it never owns or
 * copies the memory itself.
 *   - num_dims == 0 describes a scalar and needs a non-null memory address.
 *   - A non-scalar view may carry a null address (e.g. an absent C matrix).
 *   - Exactly one layout source: strides != NULL with index_type == INVALID, or
 *     strides == NULL with a predefined index_type. Strides are in elements.
 */
typedef struct {
    void* memory;
    const int64_t* dims;
    const int64_t* strides;
    uint8_t num_dims;
    FTrainNumericType numeric_type;
    FTrainIndexType index_type;
    bool is_host_memory;
} FTrainStorageView;

/* ---- role identifiers: opaque, copyable, own nothing (common.h:131-137) ---- */

// clang-format off
typedef struct { uint64_t opaque; } FTrainTensorId;
typedef struct { uint64_t opaque; } FTrainTensorListId;
typedef struct { uint64_t opaque; } FTrainGroupedTensorId;
typedef struct { uint64_t opaque; } FTrainGemmOpId;
typedef struct { uint64_t opaque; } FTrainGroupedABCDGemmOpId;
typedef struct { uint64_t opaque; } FTrainGroupedBCDGemmOpId;
typedef struct { uint64_t opaque; } FTrainGroupedABGemmOpId;
// clang-format on

/* ---- resource handles (common.h:145-148) ---- */

typedef struct FTrainPatternStruct* FTrainPattern;
typedef struct FTrainOpsStruct* FTrainOps;
typedef struct FTrainArgsStruct* FTrainArgs;
typedef struct FTrainPlanStruct* FTrainPlan;

/* ---- per-thread error state (reference common.h:162-175) ---- */

/* Status of the calling thread's most recent non-query call; SUCCESS on a
 * fresh thread. The two query functions never change it. */
FTRAIN_API FTrainStatus ftrainGetLastStatus(void);

/* Message of the calling thread's most recent non-query call; never NULL, ""
 * after a success. Valid until that thread's next non-query call. */
FTRAIN_API const char* ftrainGetLastMessage(void);

/* ---- Pattern construction (reference common.h:177-306) ----
 * The Add functions only append; wiring is validated by ftrainOpsCreate. Role
 * ids count up from 0 in insertion order, operands and operations separately. */

FTRAIN_API FTrainStatus ftrainPatternCreate(FTrainPattern* pattern);

/* Ops objects created from the Pattern stay valid. */
FTRAIN_API FTrainStatus ftrainPatternDestroy(FTrainPattern pattern);

FTRAIN_API FTrainStatus ftrainPatternAddTensor(FTrainPattern pattern, FTrainTensorId* tensor);

FTRAIN_API FTrainStatus ftrainPatternAddTensorList(FTrainPattern pattern, FTrainTensorListId* tensor_list);

FTRAIN_API FTrainStatus ftrainPatternAddGroupedTensor(FTrainPattern pattern, FTrainGroupedTensorId* grouped_tensor);

/* Gemm node: inputs (a, b, c, alpha, beta), output d; D = alpha*A*B + beta*C. */
FTRAIN_API FTrainStatus ftrainPatternAddGemm(FTrainPattern pattern, FTrainGemmOpId* op, FTrainTensorId a,
                                             FTrainTensorId b, FTrainTensorId c, FTrainTensorId d, FTrainTensorId alpha,
                                             FTrainTensorId beta);

/* The three grouped GEMM node kinds are part of the API surface; no engine is
 * registered for them (as in the reference, src/engine.cpp:25-27), so a Pattern
 * that uses one is answered with FTRAIN_STATUS_UNSUPPORTED by ftrainOpsCreate. */
FTRAIN_API FTrainStatus ftrainPatternAddGroupedABCDGemm(FTrainPattern pattern, FTrainGroupedABCDGemmOpId* op,
                                                        FTrainGroupedTensorId a, FTrainGroupedTensorId b,
                                                        FTrainGroupedTensorId c, FTrainGroupedTensorId d,
                                                        FTrainTensorId alpha, FTrainTensorId beta);

FTRAIN_API FTrainStatus ftrainPatternAddGroupedBCDGemm(FTrainPattern pattern, FTrainGroupedBCDGemmOpId* op,
                                                       FTrainTensorListId a, FTrainGroupedTensorId b,
                                                       FTrainGroupedTensorId c, FTrainGroupedTensorId d,
                                                       FTrainTensorId alpha, FTrainTensorId beta);

FTRAIN_API FTrainStatus ftrainPatternAddGroupedABGemm(FTrainPattern pattern, FTrainGroupedABGemmOpId* op,
                                                      FTrainGroupedTensorId a, FTrainGroupedTensorId b,
                                                      FTrainTensorListId c, FTrainTensorListId d, FTrainTensorId alpha,
                                                      FTrainTensorId beta);

/* ---- Ops matching (reference common.h:308-332) ---- */

/* Validates the Pattern (INVALID_ARGUMENT on bad wiring) and matches it, up to
 * insertion order, against a supported graph (UNSUPPORTED when none matches).
 * The Ops object keeps nothing of the Pattern. */
FTRAIN_API FTrainStatus ftrainOpsCreate(FTrainOps* ops, FTrainPattern pattern);

/* Plans created through the Ops object stay valid. */
FTRAIN_API FTrainStatus ftrainOpsDestroy(FTrainOps ops);

/* ---- Args binding (reference common.h:334-474) ---- */

/* All roles start unset; setters may come in any order and may repeat. */
FTRAIN_API FTrainStatus ftrainArgsCreate(FTrainArgs* args, FTrainOps ops);

/* Plans created from the Args stay valid. */
FTRAIN_API FTrainStatus ftrainArgsDestroy(FTrainArgs args);

FTRAIN_API FTrainStatus ftrainArgsSetTensor(FTrainArgs args, FTrainTensorId tensor, FTrainStorageView storage_view);

/* storage_views may be NULL only when num_storage_views is 0. */
FTRAIN_API FTrainStatus ftrainArgsSetTensorList(FTrainArgs args, FTrainTensorListId tensor_list,
                                                const FTrainStorageView storage_views[], uint32_t num_storage_views);

/* data.num_dims is the rank. offsets (optional) is a rank-1 array of num_groups
 * element offsets; dim_sizes / strides (each optional) are arrays of rank
 * views, each a rank-1 array of num_groups values. */
FTRAIN_API FTrainStatus ftrainArgsSetGroupedTensor(FTrainArgs args, FTrainGroupedTensorId grouped_tensor,
                                                   uint32_t num_groups, FTrainStorageView data,
                                                   const FTrainStorageView* offsets,
                                                   const FTrainStorageView dim_sizes[],
                                                   const FTrainStorageView strides[]);

/* compute_type must be a real numeric type (not INVALID, not COUNT). */
FTRAIN_API FTrainStatus ftrainArgsSetGemm(FTrainArgs args, FTrainGemmOpId op, FTrainNumericType compute_type);

FTRAIN_API FTrainStatus ftrainArgsSetGroupedABCDGemm(FTrainArgs args, FTrainGroupedABCDGemmOpId op,
                                                     FTrainNumericType compute_type);

FTRAIN_API FTrainStatus ftrainArgsSetGroupedBCDGemm(FTrainArgs args, FTrainGroupedBCDGemmOpId op,
                                                    FTrainNumericType compute_type);

FTRAIN_API FTrainStatus ftrainArgsSetGroupedABGemm(FTrainArgs args, FTrainGroupedABGemmOpId op,
                                                   FTrainNumericType compute_type);

/* ---- Plan selection and execution (reference common.h:476-589) ---- */

/*
 * Selects Primitives for the Args on the calling thread's current CUDA device
 * and binds the Args' addresses and scalar values (alpha and beta are read
 * here) into the returned Plan. The Plan holds >= 1 Primitive, best first.
 * Selection results are memoised per device and problem description; raw
 * addresses are not part of that description.
 * INVALID_ARGUMENT: incomplete or inconsistent Args. OVERFLOW: a byte count
 * does not fit 64 bits. UNSUPPORTED: no Primitive applies (the message lists
 * each Primitive's reason).
 */
FTRAIN_API FTrainStatus ftrainPlanCreate(FTrainPlan* plan, FTrainArgs args);

FTRAIN_API FTrainStatus ftrainPlanDestroy(FTrainPlan plan);

FTRAIN_API FTrainStatus ftrainPlanGetNumPrimitives(FTrainPlan plan, uint64_t* num_primitives);

/* The name is the identity the FTRAIN_*_PRIMITIVES variables filter by; the
 * pointer lives as long as the Plan. */
FTRAIN_API FTrainStatus ftrainPlanGetPrimitiveName(FTrainPlan plan, uint64_t primitive_index, const char** name);

FTRAIN_API FTrainStatus ftrainPlanGetPrimitiveRequiredWorkspaceBytes(FTrainPlan plan, uint64_t primitive_index,
                                                                     uint64_t* workspace_bytes);

/*
 * Enqueues one Primitive on stream and returns without synchronising. The
 * calling thread's current device must be the Plan's device; workspace_bytes
 * must cover the Primitive's requirement (non-null workspace when that is
 * nonzero). The Plan, the tensors and the workspace must outlive the enqueued
 * work; concurrent executions of one Plan need external synchronisation.
 */
FTRAIN_API FTrainStatus ftrainPlanExecutePrimitive(FTrainPlan plan, uint64_t primitive_index, void* workspace,
                                                   uint64_t workspace_bytes, FTrainStream stream);

#ifdef __cplusplus
}
#endif

#endif
