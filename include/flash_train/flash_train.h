/*
 * flash_train/flash_train.h -- one-shot convenience call over the staged API.
 * ABI-compatible with the reference's include/flash_train/flash_train.h:46-48.
 */
#ifndef FTRAIN_FLASH_TRAIN_H_
#define FTRAIN_FLASH_TRAIN_H_

#include <flash_train/common.h>

#ifdef __cplusplus
extern "C" {
#endif

/*
 * D = alpha * A * B + beta * C with the best Primitive the supplied workspace allows.
 *
 * Equivalent to: one Gemm Pattern -> Ops (both built once per process), then
 * per call Args, Plan (through the selection cache) and execution of one
 * primitive on stream. The Plan lists its primitives best first; the call
 * walks that list and runs the first one whose required workspace the
 * caller's (workspace, workspace_bytes) covers -- the budget walk a user of
 * the staged API would do. A workspace that covers primitive 0 therefore
 * selects primitive 0 (the recommended one, as in the reference, whose only
 * primitive needs none); NULL/0 selects the first primitive that needs no
 * workspace, which every Plan has (the exact-FP32 kernel, at the latest).
 * Timing and the last bits of the result can differ between the two: index 0
 * may be a split-K kernel. ftrainPlanGetPrimitiveRequiredWorkspaceBytes on a
 * Plan of the same Args tells how much index 0 wants.
 *
 * a: m-by-k, b: k-by-n, c and d: m-by-n, all rank-two device views; c.memory
 * may be NULL (no beta*C term). alpha and beta are host scalar views.
 * Asynchronous on stream.
 *
 * Numerics: the Primitives whose names start with Fp32Gemm3xTf32 multiply on the
 * tensor cores in split precision (three TF32 products per FP32 product, FP32
 * accumulation); their results meet the accuracy of an FP32 FFMA GEMM, and
 * infinities, NaNs and +-FLT_MAX in the inputs propagate as in IEEE FP32
 * arithmetic. FTRAIN_DISABLED_PRIMITIVES=Fp32Gemm3xTf32,Fp32Gemm3xTf32SplitK,Fp32Gemm3xTf32FewRows
 * restricts selection to the exact-FP32 FFMA kernels.
 */
FTRAIN_API FTrainStatus ftrainGemm(FTrainStorageView a, FTrainStorageView b, FTrainStorageView c, FTrainStorageView d,
                                   FTrainStorageView alpha, FTrainStorageView beta, FTrainNumericType compute_type,
                                   void* workspace, uint64_t workspace_bytes, FTrainStream stream);

#ifdef __cplusplus
}
#endif

#endif
