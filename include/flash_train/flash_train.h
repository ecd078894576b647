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
 * D = alpha * A * B + beta * C with the recommended Primitive (index 0).
 *
 * Equivalent to: one Gemm Pattern -> Ops (both built once per process), then
 * per call Args, Plan (through the selection cache) and execution of
 * primitive 0 on stream. a: m-by-k, b: k-by-n, c and d: m-by-n, all rank-two
 * device views; c.memory may be NULL (no beta*C term). alpha and beta are host
 * scalar views. Asynchronous on stream. workspace may be NULL/0 when the
 * recommended Primitive needs none.
 */
FTRAIN_API FTrainStatus ftrainGemm(FTrainStorageView a, FTrainStorageView b, FTrainStorageView c, FTrainStorageView d,
                                   FTrainStorageView alpha, FTrainStorageView beta, FTrainNumericType compute_type,
                                   void* workspace, uint64_t workspace_bytes, FTrainStream stream);

#ifdef __cplusplus
}
#endif

#endif
