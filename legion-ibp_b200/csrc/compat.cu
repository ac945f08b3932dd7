// The operator entry points under the reference's symbol names (engine/operator_impl.cuh:11-69).
#include <stdio.h>
#include <stdlib.h>

#include "../../include/legion_b200_compat.h"

static void die_on(int rc, const char *op)
{
    if (rc != LEGION_OK) {
        printf("%s failed: %s\n", op, legion_last_error());
        exit(EXIT_FAILURE);
    }
}

extern "C" void BatchGenerate(void *strm_hdl, LegionFeatures *feature, LegionCache *cache, LegionPool *memorypool,
                              int32_t batch_size, int32_t counter, int32_t part_id, int32_t dev_id, int32_t mode,
                              bool is_presc, int32_t hop_num, int dyn_cache)
{
    die_on(legion_batch_generate(strm_hdl, feature, cache, memorypool, batch_size, counter, part_id, dev_id, mode,
                                 is_presc ? 1 : 0, hop_num, dyn_cache),
           "BatchGenerate");
}

extern "C" void RandomSample(void *strm_hdl, LegionGraph *graph, LegionCache *cache, LegionPool *memorypool,
                             int32_t count, int32_t dev_id, int32_t op_id, bool is_presc, int dyn_cache)
{
    die_on(legion_random_sample(strm_hdl, graph, cache, memorypool, count, dev_id, op_id, is_presc ? 1 : 0, dyn_cache),
           "RandomSample");
}

extern "C" void FeatureCacheLookup(void *strm_hdl, LegionCache *cache, LegionPool *memorypool, int32_t op_id,
                                   int32_t dev_id, int dyn_cache)
{
    die_on(legion_feature_cache_lookup(strm_hdl, cache, memorypool, op_id, dev_id, dyn_cache), "FeatureCacheLookup");
}

extern "C" void IOSubmit(void *strm_hdl, LegionFeatures *feature, LegionPool *memorypool, int32_t op_id, int32_t dev_id)
{
    die_on(legion_io_submit(strm_hdl, feature, memorypool, op_id, dev_id), "IOSubmit");
}

extern "C" void IOComplete(void *strm_hdl, LegionCache *cache, LegionPool *memorypool, int32_t dev_id, int32_t mode)
{
    die_on(legion_io_complete(strm_hdl, cache, memorypool, dev_id, mode), "IOComplete");
}
