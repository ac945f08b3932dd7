/*
 * legion_b200_compat.h -- the five operator entry points under the reference's own symbol
 * names and calling convention (sampling_server/src/engine/operator_impl.cuh:11-69): void
 * return, `bool is_presc`, and print + exit(EXIT_FAILURE) on error like the reference's
 * cudaCheckError (engine/operator_impl.cu:17-25).  A GPURunner built against the reference's
 * header links against these unchanged; the opaque class pointers become this library's handles.
 */
#ifndef LEGION_B200_COMPAT_H
#define LEGION_B200_COMPAT_H

#include <stdbool.h>

#include "legion_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

void BatchGenerate(void *strm_hdl, LegionFeatures *feature, LegionCache *cache, LegionPool *memorypool,
                   int32_t batch_size, int32_t counter, int32_t part_id, int32_t dev_id, int32_t mode,
                   bool is_presc, int32_t hop_num, int dyn_cache);
void RandomSample(void *strm_hdl, LegionGraph *graph, LegionCache *cache, LegionPool *memorypool, int32_t count,
                  int32_t dev_id, int32_t op_id, bool is_presc, int dyn_cache);
void FeatureCacheLookup(void *strm_hdl, LegionCache *cache, LegionPool *memorypool, int32_t op_id, int32_t dev_id,
                        int dyn_cache);
void IOSubmit(void *strm_hdl, LegionFeatures *feature, LegionPool *memorypool, int32_t op_id, int32_t dev_id);
void IOComplete(void *strm_hdl, LegionCache *cache, LegionPool *memorypool, int32_t dev_id, int32_t mode);

#ifdef __cplusplus
}
#endif
#endif
