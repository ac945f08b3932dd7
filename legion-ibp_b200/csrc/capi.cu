// C ABI: storage handles, the memory pool, the five operators and the whole-batch calls.
#include "common.cuh"

#include <stdarg.h>
#include <string.h>

namespace legion {

static thread_local char g_error[512] = "";

void set_error(const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

static int64_t round_up(int64_t v, int64_t m) { return (v + m - 1) / m * m; }

template <typename T>
static cudaError_t dmalloc(T **p, int64_t count)
{
    return cudaMalloc(reinterpret_cast<void **>(p), sizeof(T) * (size_t)(count > 0 ? count : 1));
}

}  // namespace legion

using namespace legion;

extern "C" const char *legion_last_error(void) { return g_error; }
extern "C" int legion_abi_version(void) { return 1; }

// ---- storage ---------------------------------------------------------------------------------------

extern "C" int legion_graph_create(LegionGraph **out, int32_t dev_id, int64_t n_nodes, int64_t n_edges,
                                   const int64_t *indptr, const int32_t *indices)
{
    LG_ARG(out != nullptr && indptr != nullptr, "NULL pointer");
    LG_ARG(indices != nullptr || n_edges == 0, "indices is NULL");
    LG_ARG(n_nodes > 0 && n_nodes < (1ll << 31), "n_nodes must fit int32");
    LegionGraph *g = new LegionGraph();
    g->dev_id = dev_id;
    g->n_nodes = n_nodes;
    g->n_edges = n_edges;
    g->indptr = indptr;
    g->indices = indices;
    *out = g;
    return LEGION_OK;
}

extern "C" int legion_graph_destroy(LegionGraph *g)
{
    delete g;
    return LEGION_OK;
}

extern "C" int legion_features_create(LegionFeatures **out, int32_t dev_id, int64_t n_nodes, int32_t row_bytes,
                                      const void *host_table)
{
    LG_ARG(out != nullptr, "out is NULL");
    LG_ARG(n_nodes > 0 && n_nodes < (1ll << 31), "n_nodes must fit int32");
    LG_ARG(row_bytes > 0 && row_bytes % 4 == 0, "row_bytes must be a positive multiple of 4");
    LegionFeatures *f = new LegionFeatures();
    memset(f, 0, sizeof(*f));
    f->dev_id = dev_id;
    f->n_nodes = n_nodes;
    f->row_bytes = row_bytes;
    f->host_table = host_table;
    *out = f;
    return LEGION_OK;
}

extern "C" int legion_features_set_split(LegionFeatures *f, int32_t mode, const int32_t *ids_dev,
                                         const int32_t *labels_dev, int32_t count)
{
    LG_ARG(f != nullptr, "features is NULL");
    LG_ARG(mode >= 0 && mode <= 2, "mode must be 0 (train), 1 (valid) or 2 (test)");
    LG_ARG(count >= 0 && (count == 0 || (ids_dev != nullptr && labels_dev != nullptr)), "NULL seed list");
    f->ids[mode] = ids_dev;
    f->labels[mode] = labels_dev;
    f->count[mode] = count;
    return LEGION_OK;
}

extern "C" int legion_features_destroy(LegionFeatures *f)
{
    delete f;
    return LEGION_OK;
}

// ---- memory pool -----------------------------------------------------------------------------------

extern "C" int legion_pool_destroy(LegionPool *p)
{
    if (p == nullptr) return LEGION_OK;
    cudaSetDevice(p->dev_id);
    for (int i = 0; i < LEGION_MAX_PIPES; ++i) {
        if (p->slots < p->pipes) {  // separate hand-off buffers; feature buffers exist once per slot
            cudaFree(p->pub_ids[i]); cudaFree(p->pub_labels[i]); cudaFree(p->pub_agg_src[i]); cudaFree(p->pub_agg_dst[i]);
            cudaFree(p->pub_nc[i]); cudaFree(p->pub_ec[i]);
            if (i >= p->slots) p->features[i] = nullptr;
        }
        cudaFree(p->ids[i]); cudaFree(p->features[i]); cudaFree(p->labels[i]); cudaFree(p->agg_src[i]);
        cudaFree(p->agg_dst[i]); cudaFree(p->node_counter[i]); cudaFree(p->edge_counter[i]);
        cudaFree(p->miss_rows[i]); cudaFree(p->miss_count[i]);
        cudaFree(p->cache_index[i]); cudaFree(p->src_global[i]); cudaFree(p->map[i]); cudaFree(p->node_rec[i]);
        cudaFree(p->tile_sum[i]); cudaFree(p->tile_off[i]); cudaFree(p->eslot[i]); cudaFree(p->erank[i]);
        cudaFree(p->edge_cnt[i]);
        cudaFree(p->lru_victim[i]); cudaFree(p->ctl[i]); cudaFree(p->bctl[i]);
        cudaFree(p->seed_stage[i]);
        if (p->h_stage[i]) cudaFreeHost(p->h_stage[i]);
    }
    delete p;
    return LEGION_OK;
}

extern "C" int legion_pool_create(LegionPool **out, int32_t dev_id, int32_t batch_size, int32_t hop_num,
                                  const int32_t *fanout, int32_t row_bytes_out, int32_t pipes)
{
    return legion_pool_create_ahead(out, dev_id, batch_size, hop_num, fanout, row_bytes_out, pipes, pipes);
}

extern "C" int legion_pool_create_ahead(LegionPool **out, int32_t dev_id, int32_t batch_size, int32_t hop_num,
                                        const int32_t *fanout, int32_t row_bytes_out, int32_t slots, int32_t pipes)
{
    LG_ARG(out != nullptr, "out is NULL");
    LG_ARG(slots >= 1 && slots <= pipes && pipes % slots == 0, "pipes must be a multiple of slots");
    LG_ARG(batch_size > 0, "batch_size must be positive");
    LG_ARG(hop_num >= 0 && hop_num <= LEGION_MAX_HOPS, "hop_num must be 0..3");
    LG_ARG(hop_num == 0 || fanout != nullptr, "fanout is NULL");
    LG_ARG(row_bytes_out > 0 && row_bytes_out % 4 == 0, "row_bytes_out must be a positive multiple of 4");
    LG_ARG(pipes >= 1 && pipes <= LEGION_MAX_PIPES, "pipes must be 1..4");
    for (int h = 0; h < hop_num; ++h)
        LG_ARG(fanout[h] >= 1 && fanout[h] <= LEGION_MAX_FANOUT, "fanout must be 1..32");
    LG_CUDA(cudaSetDevice(dev_id));

    LegionPool *p = new LegionPool();
    memset(p, 0, sizeof(*p));
    p->dev_id = dev_id;
    p->batch_size = batch_size;
    p->hop_num = hop_num;
    p->row_bytes_out = row_bytes_out;
    p->pipes = pipes;
    p->slots = slots;
    // True worst case: every hop samples all nodes found so far (the reference sizes its buffers
    // as B*(1+f1+f1*f2), engine/server.cu:204-216, which is below it).
    int64_t nodes = batch_size, edges = 0, max_hop_edges = 0, max_inputs = batch_size;
    for (int h = 0; h < hop_num; ++h) {
        p->fanout[h] = fanout[h];
        int64_t e = nodes * fanout[h];
        if (nodes > max_inputs) max_inputs = nodes;
        if (e > max_hop_edges) max_hop_edges = e;
        edges += e;
        nodes += e;
    }
    if (nodes >= kNewBase || edges >= kNewBase) {
        set_error("legion_pool_create: batch of up to %lld nodes / %lld edges is above the 2^30 limit",
                  (long long)nodes, (long long)edges);
        delete p;
        return LEGION_E_LIMIT;
    }
    p->max_nodes = nodes;
    p->max_edges = edges;
    p->max_hop_edges = max_hop_edges;
    p->max_inputs = max_inputs;
    p->feat_rows = nodes;
    p->rng_seed = 0;
    p->max_rounds = 64;
    p->sm_count = 148;
    cudaDeviceGetAttribute(&p->sm_count, cudaDevAttrMultiProcessorCount, dev_id);
    if (p->sm_count <= 0) p->sm_count = 148;

    uint32_t cap = 1024;
    while ((int64_t)cap * 5 < nodes * 8) cap <<= 1;  // load factor <= 0.625 in the worst case
    p->map_mask = cap - 1;
    // front region: what batches actually need is far below the worst case (a paper100M-shaped batch finds
    // ~2 x 10^5 of its 2.3 x 10^6 possible nodes), so an eighth of the worst-case size is enough; but not
    // below 2^20 slots (8 MB, at home in L2) when the worst case allows that much: a fuller region costs
    // probes (measured: products-shaped batches lost 13% with a front region at load 0.5)
    uint32_t front;
    if (g_map_front_shift >= 0) {
        front = cap >> (g_map_front_shift < 31 ? g_map_front_shift : 31);
    } else {
        front = cap >> 3;
        const uint32_t floor_slots = cap < (1u << 20) ? cap : (1u << 20);
        if (front < floor_slots) front = floor_slots;
    }
    if (front < 64) front = 64;
    if (front > cap) front = cap;
    p->map_front_mask = front - 1;
    if ((int64_t)front + cap >= (1ll << 31)) {  // slots are named by int32 indices
        set_error("legion_pool_create: a batch of up to %lld nodes needs an id map beyond 2^31 slots", (long long)nodes);
        delete p;
        return LEGION_E_LIMIT;
    }

    const int64_t pad_nodes = round_up(nodes, kTile) + kTile;
    const int64_t pad_edges = round_up(edges > 0 ? edges : 1, kTile) + kTile;
    const int64_t pad_hop_edges = round_up(max_hop_edges > 0 ? max_hop_edges : 1, kTile) + kTile;
    // node tiles: 1024 inputs each, except the seed hop, which may count in 256-seed tiles
    int64_t input_tiles = max_inputs / kTile + 2;
    if (batch_size / 256 + 2 > input_tiles) input_tiles = batch_size / 256 + 2;
    p->input_tiles = input_tiles;
    const int64_t tiles = input_tiles + max_hop_edges / kTile + 2;

    cudaError_t e = cudaSuccess;
    for (int i = 0; i < pipes && e == cudaSuccess; ++i) {
        e = dmalloc(&p->ids[i], pad_nodes);
        if (e == cudaSuccess) {
            if (i < slots) e = cudaMalloc(&p->features[i], (size_t)(nodes * (int64_t)row_bytes_out));
            else p->features[i] = p->features[i % slots];
        }
        if (e == cudaSuccess) e = dmalloc(&p->labels[i], batch_size);
        if (e == cudaSuccess) e = dmalloc(&p->agg_src[i], pad_edges);
        if (e == cudaSuccess) e = dmalloc(&p->agg_dst[i], pad_edges);
        if (e == cudaSuccess) e = dmalloc(&p->node_counter[i], 16);
        if (e == cudaSuccess) e = dmalloc(&p->edge_counter[i], 16);
        if (e == cudaSuccess) e = cudaMemset(p->node_counter[i], 0, 64);
        if (e == cudaSuccess) e = cudaMemset(p->edge_counter[i], 0, 64);
        if (e == cudaSuccess) e = cudaMemset(p->ids[i], 0xFF, sizeof(int32_t) * pad_nodes);
        if (e == cudaSuccess) e = dmalloc(&p->miss_rows[i], pad_nodes);
        if (e == cudaSuccess) e = dmalloc(&p->miss_count[i], 8);
        if (e == cudaSuccess) e = cudaMemset(p->miss_count[i], 0, 32);
        if (e == cudaSuccess) e = dmalloc(&p->cache_index[i], pad_nodes);
        if (e == cudaSuccess) e = dmalloc(&p->src_global[i], pad_edges);
        if (e == cudaSuccess) e = dmalloc(&p->map[i], (int64_t)front + cap);
        if (e == cudaSuccess) e = dmalloc(&p->node_rec[i], pad_nodes);
        if (e == cudaSuccess) e = dmalloc(&p->tile_sum[i], tiles);
        if (e == cudaSuccess) e = dmalloc(&p->tile_off[i], tiles);
        if (e == cudaSuccess) e = dmalloc(&p->eslot[i], pad_hop_edges);
        if (e == cudaSuccess) e = dmalloc(&p->erank[i], pad_hop_edges);
        if (e == cudaSuccess) e = dmalloc(&p->edge_cnt[i], (hop_num > 0 ? hop_num : 1) * pad_nodes);
        if (e == cudaSuccess) e = dmalloc(&p->lru_victim[i], pad_nodes);
        if (e == cudaSuccess) e = dmalloc(&p->ctl[i], CTL_WORDS);
        if (e == cudaSuccess) e = dmalloc(&p->bctl[i], 1);
        if (e == cudaSuccess) e = cudaMemset(p->ctl[i], 0, sizeof(int32_t) * CTL_WORDS);
        if (e == cudaSuccess) {
            // the back region of a new map is not empty yet: the first batch has to clear it
            const int32_t one = 1;
            e = cudaMemcpy(p->ctl[i] + CTL_BACK_DIRTY, &one, sizeof(one), cudaMemcpyHostToDevice);
        }
        if (e == cudaSuccess) e = cudaMemset(p->bctl[i], 0, sizeof(BatchCtl));
        if (e == cudaSuccess) e = cudaMemset(p->eslot[i], 0, sizeof(int32_t) * pad_hop_edges);
        // seeds and labels of a host-provided batch: one allocation, so that one copy brings both in
        if (e == cudaSuccess) e = dmalloc(&p->seed_stage[i], 2 * (int64_t)batch_size);
        if (e == cudaSuccess) p->label_stage[i] = p->seed_stage[i] + batch_size;
        if (e == cudaSuccess)
            e = cudaMallocHost(reinterpret_cast<void **>(&p->h_stage[i]), sizeof(int32_t) * (2 * (size_t)batch_size + 128));
    }
    for (int i = 0; i < slots && e == cudaSuccess; ++i) {
        if (slots == pipes) {
            p->pub_ids[i] = p->ids[i]; p->pub_labels[i] = p->labels[i]; p->pub_agg_src[i] = p->agg_src[i];
            p->pub_agg_dst[i] = p->agg_dst[i]; p->pub_nc[i] = p->node_counter[i]; p->pub_ec[i] = p->edge_counter[i];
            continue;
        }
        e = dmalloc(&p->pub_ids[i], pad_nodes);
        if (e == cudaSuccess) e = dmalloc(&p->pub_labels[i], batch_size);
        if (e == cudaSuccess) e = dmalloc(&p->pub_agg_src[i], pad_edges);
        if (e == cudaSuccess) e = dmalloc(&p->pub_agg_dst[i], pad_edges);
        if (e == cudaSuccess) e = dmalloc(&p->pub_nc[i], 16);
        if (e == cudaSuccess) e = dmalloc(&p->pub_ec[i], 16);
        if (e == cudaSuccess) e = cudaMemset(p->pub_nc[i], 0, 64);
        if (e == cudaSuccess) e = cudaMemset(p->pub_ec[i], 0, 64);
    }
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        set_error("legion_pool_create: %s", cudaGetErrorString(e));
        legion_pool_destroy(p);
        return LEGION_E_NOMEM;
    }
    *out = p;
    return LEGION_OK;
}

extern "C" int legion_pool_buffer(LegionPool *p, int32_t which, int32_t pipe, void **ptr, int64_t *bytes)
{
    LG_ARG(p != nullptr && ptr != nullptr, "NULL pointer");
    LG_ARG(pipe >= 0 && pipe < p->pipes, "pipe out of range");
    if (which <= LEGION_BUF_EDGE_COUNTER) LG_ARG(pipe < p->slots, "the hand-off buffers are numbered by slot");
    int64_t b = 0;
    void *q = nullptr;
    switch (which) {
    case LEGION_BUF_IDS: q = p->pub_ids[pipe]; b = p->max_nodes * 4; break;
    case LEGION_BUF_FEATURES: q = p->features[pipe]; b = p->feat_rows * (int64_t)p->row_bytes_out; break;
    case LEGION_BUF_LABELS: q = p->pub_labels[pipe]; b = (int64_t)p->batch_size * 4; break;
    case LEGION_BUF_AGG_SRC: q = p->pub_agg_src[pipe]; b = p->max_edges * 4; break;
    case LEGION_BUF_AGG_DST: q = p->pub_agg_dst[pipe]; b = p->max_edges * 4; break;
    case LEGION_BUF_NODE_COUNTER: q = p->pub_nc[pipe]; b = 64; break;
    case LEGION_BUF_EDGE_COUNTER: q = p->pub_ec[pipe]; b = 64; break;
    case LEGION_BUF_CACHE_INDEX: q = p->cache_index[pipe]; b = p->max_nodes * 8; break;
    case LEGION_BUF_SRC_GLOBAL: q = p->src_global[pipe]; b = p->max_edges * 4; break;
    default: LG_ARG(false, "unknown buffer");
    }
    *ptr = q;
    if (bytes) *bytes = b;
    return LEGION_OK;
}

extern "C" int legion_pool_limits(LegionPool *p, int64_t *max_nodes, int64_t *max_edges)
{
    LG_ARG(p != nullptr, "pool is NULL");
    if (max_nodes) *max_nodes = p->max_nodes;
    if (max_edges) *max_edges = p->max_edges;
    return LEGION_OK;
}

extern "C" int legion_pool_set_batch(LegionPool *p, int32_t iter, int32_t mode, int32_t pipe, uint32_t global_batch)
{
    LG_ARG(p != nullptr, "pool is NULL");
    LG_ARG(pipe >= 0 && pipe < p->pipes, "pipe out of range");
    LG_ARG(mode >= 0 && mode <= 2, "mode must be 0, 1 or 2");
    p->iter = iter;
    p->mode = mode;
    p->pipe = pipe;
    p->global_batch = global_batch;
    return LEGION_OK;
}

extern "C" int legion_pool_set_rng(LegionPool *p, uint64_t seed, int32_t max_rounds)
{
    LG_ARG(p != nullptr, "pool is NULL");
    LG_ARG(max_rounds >= 1 && max_rounds <= 1024, "max_rounds must be 1..1024");
    p->rng_seed = seed;
    p->max_rounds = max_rounds;
    return LEGION_OK;
}

// First error raised by a kernel of this pool since the last reset (0 = none): 1 id map full,
// 2 edge buffer overflow, 3 node buffer overflow, 4 bulk copy timed out (these stop the batch);
// 5 a seed or neighbour id outside [0, n_nodes) was met: it was skipped without being read, the
// rest of the batch is complete.  Synchronises the stream.
extern "C" int legion_pool_device_error(LegionPool *p, void *stream, int32_t *err, int32_t reset)
{
    LG_ARG(p != nullptr && err != nullptr, "NULL pointer");
    LG_CUDA(cudaSetDevice(p->dev_id));
    *err = 0;
    for (int i = 0; i < p->pipes; ++i) {
        int32_t w[CTL_WORDS];
        LG_CUDA(cudaMemcpyAsync(w, p->ctl[i], sizeof(w), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
        LG_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
        // an error that stopped the batch comes before "an id was skipped"
        const int32_t e = w[CTL_ERROR] != 0 ? w[CTL_ERROR] : (w[CTL_BAD_IDS] != 0 ? (int32_t)DERR_BAD_ID : 0);
        if (e != 0 && (*err == 0 || *err == DERR_BAD_ID)) *err = e;
        if (reset && w[CTL_ERROR] != 0) LG_CUDA(cudaMemsetAsync(p->ctl[i] + CTL_ERROR, 0, 4, (cudaStream_t)stream));
        if (reset && w[CTL_BAD_IDS] != 0) LG_CUDA(cudaMemsetAsync(p->ctl[i] + CTL_BAD_IDS, 0, 4, (cudaStream_t)stream));
    }
    return LEGION_OK;
}

// ---- operators ---------------------------------------------------------------------------------------

extern "C" int legion_batch_generate(void *stream, LegionFeatures *feature, LegionCache *cache, LegionPool *pool,
                                     int32_t batch_size, int32_t counter, int32_t part_id, int32_t dev_id,
                                     int32_t mode, int32_t is_presc, int32_t hop_num, int32_t dyn_cache)
{
    (void)part_id; (void)is_presc; (void)dyn_cache;
    LG_ARG(feature != nullptr && pool != nullptr, "NULL handle");
    LG_ARG(mode >= 0 && mode <= 2, "invalid mode");
    LG_ARG(batch_size > 0 && batch_size <= pool->batch_size, "batch_size above the pool's");
    LG_ARG(hop_num == pool->hop_num, "hop_num differs from the pool's");
    LG_ARG(counter >= 0, "negative batch counter");
    const int32_t *all_ids = feature->ids[mode];
    const int32_t *all_labels = feature->labels[mode];
    int32_t total_cap = feature->count[mode];
    LG_ARG(all_ids != nullptr && all_labels != nullptr && total_cap > 0, "no seed list for this mode");
    LG_CUDA(cudaSetDevice(dev_id));
    int64_t first = (int64_t)batch_size * counter;
    // tail batch is shortened, operator_impl.cu:162
    int64_t size = ((int64_t)batch_size * (counter + 1) >= total_cap) ? (total_cap - first) : batch_size;
    if (size < 0) size = 0;
    return launch_batch_generate((cudaStream_t)stream, pool,
                                 make_batch_ctl(pool, cache, all_ids, all_labels, total_cap, first, (int32_t)size,
                                                feature->n_nodes));
}

extern "C" int legion_random_sample(void *stream, LegionGraph *graph, LegionCache *cache, LegionPool *pool,
                                    int32_t count, int32_t dev_id, int32_t op_id, int32_t is_presc, int32_t dyn_cache)
{
    (void)cache; (void)is_presc; (void)dyn_cache;
    LG_ARG(graph != nullptr && pool != nullptr, "NULL handle");
    LG_ARG(op_id > 0 && op_id % LEGION_INTRABATCH_CON == 0 && op_id / LEGION_INTRABATCH_CON <= pool->hop_num,
           "op_id must be 3, 6 or 9 and within the pool's hop count");
    const int hop = op_id / LEGION_INTRABATCH_CON - 1;
    LG_ARG(count >= 1 && count <= LEGION_MAX_FANOUT, "Neighbor count must be at most 32");
    LG_ARG(count == pool->fanout[hop], "fanout differs from the pool's");
    LG_CUDA(cudaSetDevice(dev_id));
    return launch_sample_hop((cudaStream_t)stream, pool, graph, count, hop, op_id);
}

extern "C" int legion_feature_cache_lookup(void *stream, LegionCache *cache, LegionPool *pool, int32_t op_id,
                                           int32_t dev_id, int32_t dyn_cache)
{
    (void)dyn_cache;
    LG_ARG(pool != nullptr, "NULL handle");
    LG_ARG(op_id > 0 && op_id % LEGION_INTRABATCH_CON == 1 && op_id / LEGION_INTRABATCH_CON <= pool->hop_num,
           "op_id must be 1, 4, 7 or 10 and within the pool's hop count");
    if (cache != nullptr) LG_ARG(cache->row_bytes == pool->row_bytes_out, "cache and pool disagree on the row size");
    LG_CUDA(cudaSetDevice(dev_id));
    return launch_gather((cudaStream_t)stream, pool, cache, op_id);
}

extern "C" int legion_io_submit(void *stream, LegionFeatures *feature, LegionPool *pool, int32_t op_id, int32_t dev_id)
{
    (void)stream; (void)feature; (void)pool; (void)op_id; (void)dev_id;
    return LEGION_OK;
}

extern "C" int legion_io_complete(void *stream, LegionCache *cache, LegionPool *pool, int32_t dev_id, int32_t mode)
{
    (void)mode;
    LG_ARG(pool != nullptr, "NULL handle");
    LG_CUDA(cudaSetDevice(dev_id));
    int rc = launch_lru_insert((cudaStream_t)stream, pool, cache);
    if (rc == LEGION_OK && cache != nullptr && cache->kind == 1) cache->clock += 1;  // next batch, next stamp
    return rc;
}

// ---- whole batch ---------------------------------------------------------------------------------------

static int run_ops(cudaStream_t s, LegionGraph *graph, LegionCache *cache, LegionPool *pool, int32_t dev_id)
{
    int rc = legion_feature_cache_lookup(s, cache, pool, 1, dev_id, 0);
    for (int h = 0; h < pool->hop_num && rc == LEGION_OK; ++h) {
        int op = LEGION_INTRABATCH_CON * (h + 1);
        rc = legion_random_sample(s, graph, cache, pool, pool->fanout[h], dev_id, op, 0, 0);
        if (rc == LEGION_OK) rc = legion_feature_cache_lookup(s, cache, pool, op + 1, dev_id, 0);
    }
    if (rc == LEGION_OK) rc = legion_io_complete(s, cache, pool, dev_id, pool->mode);
    return rc;
}

extern "C" int legion_run_batch(void *stream, LegionGraph *graph, LegionFeatures *feature, LegionCache *cache,
                                LegionPool *pool, int32_t dev_id)
{
    LG_ARG(graph != nullptr && feature != nullptr && pool != nullptr, "NULL handle");
    int rc = legion_batch_generate(stream, feature, cache, pool, pool->batch_size, pool->iter, dev_id, dev_id,
                                   pool->mode, 0, pool->hop_num, 0);
    if (rc != LEGION_OK) return rc;
    return run_ops((cudaStream_t)stream, graph, cache, pool, dev_id);
}

extern "C" int legion_run_batch_host(LegionGraph *graph, LegionFeatures *feature, LegionCache *cache, LegionPool *pool,
                                     int32_t dev_id, const int32_t *seeds, const int32_t *labels, int32_t n_seeds,
                                     int32_t *ids_out, int32_t *labels_out, int32_t *agg_src_out, int32_t *agg_dst_out,
                                     int32_t node_counter_out[16], int32_t edge_counter_out[16], void *features_out)
{
    (void)feature;
    LG_ARG(graph != nullptr && pool != nullptr && seeds != nullptr && labels != nullptr, "NULL pointer");
    LG_ARG(n_seeds > 0 && n_seeds <= pool->batch_size, "n_seeds above the pool's batch size");
    LG_ARG(node_counter_out != nullptr && edge_counter_out != nullptr, "NULL counter output");
    LG_CUDA(cudaSetDevice(dev_id));
    cudaStream_t s = 0;
    const int pipe = pool->pipe;
    int32_t *hs = pool->h_stage[pipe];
    // inputs: host -> pinned staging -> device
    memcpy(hs, seeds, sizeof(int32_t) * n_seeds);
    memcpy(hs + pool->batch_size, labels, sizeof(int32_t) * n_seeds);
    LG_CUDA(cudaMemcpyAsync(pool->seed_stage[pipe], hs, sizeof(int32_t) * n_seeds, cudaMemcpyHostToDevice, s));
    LG_CUDA(cudaMemcpyAsync(pool->label_stage[pipe], hs + pool->batch_size, sizeof(int32_t) * n_seeds,
                            cudaMemcpyHostToDevice, s));
    int rc = launch_batch_generate(s, pool, make_batch_ctl(pool, cache, pool->seed_stage[pipe], pool->label_stage[pipe],
                                                            n_seeds, 0, n_seeds, graph->n_nodes));
    if (rc != LEGION_OK) return rc;
    rc = run_ops(s, graph, cache, pool, dev_id);
    if (rc != LEGION_OK) return rc;
    int32_t *hc = hs + 2 * (size_t)pool->batch_size;
    LG_CUDA(cudaMemcpyAsync(hc, pool->node_counter[pipe], 64, cudaMemcpyDeviceToHost, s));
    LG_CUDA(cudaMemcpyAsync(hc + 16, pool->edge_counter[pipe], 64, cudaMemcpyDeviceToHost, s));
    LG_CUDA(cudaStreamSynchronize(s));
    memcpy(node_counter_out, hc, 64);
    memcpy(edge_counter_out, hc + 16, 64);
    const int hops = hc[LEGION_INTRABATCH_CON * 3 - 1];
    const int64_t n_nodes = hc[LEGION_INTRABATCH_CON * 3 + hops];
    const int64_t n_edges = (int64_t)hc[16] + hc[17];
    if (ids_out) LG_CUDA(cudaMemcpyAsync(ids_out, pool->ids[pipe], 4 * n_nodes, cudaMemcpyDeviceToHost, s));
    if (labels_out) LG_CUDA(cudaMemcpyAsync(labels_out, pool->labels[pipe], 4 * (int64_t)n_seeds, cudaMemcpyDeviceToHost, s));
    if (agg_src_out) LG_CUDA(cudaMemcpyAsync(agg_src_out, pool->agg_src[pipe], 4 * n_edges, cudaMemcpyDeviceToHost, s));
    if (agg_dst_out) LG_CUDA(cudaMemcpyAsync(agg_dst_out, pool->agg_dst[pipe], 4 * n_edges, cudaMemcpyDeviceToHost, s));
    if (features_out)
        LG_CUDA(cudaMemcpyAsync(features_out, pool->features[pipe], n_nodes * (int64_t)pool->row_bytes_out,
                                cudaMemcpyDeviceToHost, s));
    LG_CUDA(cudaStreamSynchronize(s));
    return LEGION_OK;
}

// Plain copies for callers that hold raw pointers only (tests, consumers without a CUDA binding).
// kind: 1 host->device, 2 device->host, 3 device->device.  Blocking.
extern "C" int legion_copy(void *dst, const void *src, int64_t bytes, int32_t kind)
{
    LG_ARG(bytes >= 0 && (bytes == 0 || (dst != nullptr && src != nullptr)), "NULL pointer");
    LG_ARG(kind >= 1 && kind <= 3, "kind must be 1, 2 or 3");
    if (bytes == 0) return LEGION_OK;
    LG_CUDA(cudaMemcpy(dst, src, (size_t)bytes, (cudaMemcpyKind)kind));
    return LEGION_OK;
}

// Page-locks host memory that this process did not allocate through CUDA (a POSIX shared segment or a
// mapped file that several server processes share) so that kernels of this process can read it by
// zero-copy loads; the reference allocates its host tables with cudaHostAlloc inside its one process
// (storage/storage_management.cu:114-115,171).  If the driver refuses the range as a whole it is
// registered in 1 GiB pieces.  Already-registered memory is not an error.
extern "C" int legion_host_register(int32_t dev_id, void *ptr, int64_t bytes)
{
    LG_ARG(ptr != nullptr && bytes > 0, "bad range");
    LG_CUDA(cudaSetDevice(dev_id));
    cudaError_t e = cudaHostRegister(ptr, (size_t)bytes, cudaHostRegisterDefault);
    if (e == cudaSuccess || e == cudaErrorHostMemoryAlreadyRegistered) {
        cudaGetLastError();
        return LEGION_OK;
    }
    const cudaError_t whole = e;
    cudaGetLastError();
    const int64_t piece = 1ll << 30;
    int64_t done = 0;
    for (; done < bytes; done += piece) {
        int64_t len = bytes - done < piece ? bytes - done : piece;
        e = cudaHostRegister((char *)ptr + done, (size_t)len, cudaHostRegisterDefault);
        if (e != cudaSuccess && e != cudaErrorHostMemoryAlreadyRegistered) break;
    }
    cudaGetLastError();
    if (done >= bytes) return LEGION_OK;
    for (int64_t u = 0; u < done; u += piece) cudaHostUnregister((char *)ptr + u);
    cudaGetLastError();
    set_error("legion_host_register: %lld bytes: %s (%d); in 1 GiB pieces: %s (%d) after %lld bytes", (long long)bytes,
              cudaGetErrorName(whole), (int)whole, cudaGetErrorName(e), (int)e, (long long)done);
    return LEGION_E_CUDA;
}

// EnableP2PAccess (storage/storage_management.cu:9-27) for one pair: lets kernels of `dev_id` read
// memory of `peer_id` allocated in this process.  Already-enabled is not an error.
extern "C" int legion_enable_peer_access(int32_t dev_id, int32_t peer_id)
{
    LG_ARG(dev_id >= 0 && peer_id >= 0 && dev_id != peer_id, "need two different devices");
    int can = 0;
    LG_CUDA(cudaDeviceCanAccessPeer(&can, dev_id, peer_id));
    if (!can) {
        set_error("legion_enable_peer_access: device %d cannot access device %d", dev_id, peer_id);
        return LEGION_E_STATE;
    }
    LG_CUDA(cudaSetDevice(dev_id));
    cudaError_t e = cudaDeviceEnablePeerAccess(peer_id, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) {
        cudaGetLastError();
        return LEGION_OK;
    }
    LG_CUDA(e);
    return LEGION_OK;
}
