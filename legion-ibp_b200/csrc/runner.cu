// Per-GPU runner: the op list of one batch on three streams, the pipe rotation and the hand-off.
//
// Restates GPURunner (sampling_server/src/engine/server.cu:176-416).  The reference builds the
// op list [BatchGenerate, CacheLookup, IOSubmit, (RandomSample, CacheLookup, IOSubmit) x hops,
// IOComplete] over three streams and then blocks: it spins on the last event, and several ops
// read counters back to the host in between.  Here nothing is read back, and three streams carry
// the three resources the path is bound by: sampling (latency of random topology reads) on one,
// lookup + gather of cached rows (HBM / NVLink bandwidth) on a second one behind an event per
// segment, and the fetch of missed rows from pinned host memory (host link) on a third.  The
// gather of hop h overlaps the sampling of hop h+1, and the host-link traffic of batch k overlaps
// everything of batch k+1.  Scratch shared between pipes is touched by one stream only, so
// in-stream order keeps it consistent.
#include "common.cuh"

#include <vector>

struct LegionRunner {
    int32_t dev_id;
    LegionGraph *graph;
    LegionFeatures *feature;
    LegionCache *cache;
    LegionPool *pool;
    LegionIpcEnv *env;
    cudaStream_t s_sample, s_gather, s_miss;
    cudaEvent_t seg_ready[LEGION_MAX_HOPS + 1];
    cudaEvent_t hit_done[LEGION_MAX_HOPS + 1];
    cudaEvent_t pipe_done[LEGION_INTERBATCH_CON];
    bool pipe_busy[LEGION_INTERBATCH_CON];
    int current_pipe;
    // timing of the batches enqueued since the last sync
    cudaEvent_t t_begin, t_end;
    bool open_window;
    int window_batches;
    std::vector<cudaEvent_t> ev_free;
    std::vector<std::pair<cudaEvent_t, cudaEvent_t>> gather_ev, miss_ev;
    float last_batch_ms, last_gather_ms, last_miss_ms;
    int last_pipe;
    int last_batches;
    long long served;
    double served_us;
};

using namespace legion;

extern "C" int legion_ipc_wait(LegionIpcEnv *e, int32_t dev_id, int32_t pipe, int32_t timeout_ms);
extern "C" int legion_ipc_post(LegionIpcEnv *e, int32_t dev_id, int32_t pipe);
extern "C" int legion_ipc_current_batchsize(LegionIpcEnv *e, int32_t dev_id, int32_t mode);
extern "C" int legion_ipc_current_mode(LegionIpcEnv *e, int32_t global_batch_id);
extern "C" int legion_ipc_local_batch_id(LegionIpcEnv *e, int32_t global_batch_id);

static cudaEvent_t take_event(LegionRunner *r)
{
    cudaEvent_t e = nullptr;
    if (!r->ev_free.empty()) {
        e = r->ev_free.back();
        r->ev_free.pop_back();
    } else if (cudaEventCreate(&e) != cudaSuccess) {
        e = nullptr;
    }
    return e;
}

extern "C" int legion_runner_create(LegionRunner **out, int32_t dev_id, LegionGraph *graph, LegionFeatures *feature,
                                    LegionCache *cache, LegionPool *pool, LegionIpcEnv *env)
{
    LG_ARG(out != nullptr && graph != nullptr && feature != nullptr && pool != nullptr, "NULL handle");
    LG_CUDA(cudaSetDevice(dev_id));
    LegionRunner *r = new LegionRunner();
    r->dev_id = dev_id;
    r->graph = graph;
    r->feature = feature;
    r->cache = cache;
    r->pool = pool;
    r->env = env;
    r->current_pipe = 0;
    r->open_window = false;
    r->window_batches = 0;
    r->last_batch_ms = r->last_gather_ms = r->last_miss_ms = 0.0f;
    r->last_pipe = -1;
    r->last_batches = 0;
    r->served = 0;
    r->served_us = 0.0;
    LG_CUDA(cudaStreamCreateWithFlags(&r->s_sample, cudaStreamNonBlocking));
    LG_CUDA(cudaStreamCreateWithFlags(&r->s_gather, cudaStreamNonBlocking));
    LG_CUDA(cudaStreamCreateWithFlags(&r->s_miss, cudaStreamNonBlocking));
    for (int i = 0; i <= LEGION_MAX_HOPS; ++i) {
        LG_CUDA(cudaEventCreateWithFlags(&r->seg_ready[i], cudaEventDisableTiming));
        LG_CUDA(cudaEventCreateWithFlags(&r->hit_done[i], cudaEventDisableTiming));
    }
    for (int i = 0; i < LEGION_INTERBATCH_CON; ++i) {
        LG_CUDA(cudaEventCreateWithFlags(&r->pipe_done[i], cudaEventDisableTiming));
        r->pipe_busy[i] = false;
    }
    LG_CUDA(cudaEventCreate(&r->t_begin));
    LG_CUDA(cudaEventCreate(&r->t_end));
    *out = r;
    return LEGION_OK;
}

// One segment: cached rows on the gather stream, missed rows on the miss stream behind it.
static int timed_gather(LegionRunner *r, int op_id, int seg)
{
    LegionPool *p = r->pool;
    LegionCache *c = r->cache;
    if (c != nullptr) LG_ARG(c->row_bytes == p->row_bytes_out, "cache and pool disagree on the row size");
    const bool record = r->gather_ev.size() < 8192;
    cudaEvent_t a = record ? take_event(r) : nullptr, b = record ? take_event(r) : nullptr;
    if (a) cudaEventRecord(a, r->s_gather);
    int rc = launch_gather_hits(r->s_gather, p, c, op_id);
    if (b) cudaEventRecord(b, r->s_gather);
    if (a && b) r->gather_ev.push_back(std::make_pair(a, b));
    if (rc != LEGION_OK) return rc;
    LG_CUDA(cudaEventRecord(r->hit_done[seg], r->s_gather));
    LG_CUDA(cudaStreamWaitEvent(r->s_miss, r->hit_done[seg], 0));
    if (c != nullptr && c->host_table != nullptr) {
        cudaEvent_t m0 = record ? take_event(r) : nullptr, m1 = record ? take_event(r) : nullptr;
        if (m0) cudaEventRecord(m0, r->s_miss);
        rc = launch_gather_misses(r->s_miss, p, c, op_id);
        if (m1) cudaEventRecord(m1, r->s_miss);
        if (m0 && m1) r->miss_ev.push_back(std::make_pair(m0, m1));
    }
    return rc;
}

extern "C" int legion_runner_enqueue(LegionRunner *r, int32_t global_batch_id, int32_t mode, int32_t local_batch_id)
{
    LG_ARG(r != nullptr, "runner is NULL");
    LG_CUDA(cudaSetDevice(r->dev_id));
    LegionPool *p = r->pool;
    const int pipe = r->current_pipe;
    int rc = legion_pool_set_batch(p, local_batch_id, mode, pipe, (uint32_t)global_batch_id);
    if (rc != LEGION_OK) return rc;
    int32_t bs = p->batch_size;
    if (r->env != nullptr) {
        bs = legion_ipc_current_batchsize(r->env, r->dev_id, mode);
        LG_ARG(bs > 0 && bs <= p->batch_size, "batch size of this mode is above the pool's");
    }
    if (!r->open_window) {
        LG_CUDA(cudaEventRecord(r->t_begin, r->s_sample));
        r->open_window = true;
        r->window_batches = 0;
    }
    // the buffers of this pipe are rewritten: the gather that last read them must be over
    if (r->pipe_busy[pipe]) LG_CUDA(cudaStreamWaitEvent(r->s_sample, r->pipe_done[pipe], 0));
    rc = legion_batch_generate(r->s_sample, r->feature, r->cache, p, bs, local_batch_id, r->dev_id, r->dev_id, mode, 0,
                               p->hop_num, 0);
    if (rc != LEGION_OK) return rc;
    LG_CUDA(cudaEventRecord(r->seg_ready[0], r->s_sample));
    LG_CUDA(cudaStreamWaitEvent(r->s_gather, r->seg_ready[0], 0));
    // an LRU cache changes at the end of every batch: its next lookup has to see the insertions
    if (r->cache != nullptr && r->cache->kind == 1 && r->last_pipe >= 0 && r->pipe_busy[r->last_pipe])
        LG_CUDA(cudaStreamWaitEvent(r->s_gather, r->pipe_done[r->last_pipe], 0));
    rc = timed_gather(r, 1, 0);
    if (rc != LEGION_OK) return rc;
    for (int h = 0; h < p->hop_num; ++h) {
        const int op = LEGION_INTRABATCH_CON * (h + 1);
        rc = legion_random_sample(r->s_sample, r->graph, r->cache, p, p->fanout[h], r->dev_id, op, 0, 0);
        if (rc != LEGION_OK) return rc;
        LG_CUDA(cudaEventRecord(r->seg_ready[h + 1], r->s_sample));
        LG_CUDA(cudaStreamWaitEvent(r->s_gather, r->seg_ready[h + 1], 0));
        rc = timed_gather(r, op + 1, h + 1);
        if (rc != LEGION_OK) return rc;
    }
    rc = legion_io_complete(r->s_miss, r->cache, p, r->dev_id, mode);
    if (rc != LEGION_OK) return rc;
    LG_CUDA(cudaEventRecord(r->pipe_done[pipe], r->s_miss));
    r->pipe_busy[pipe] = true;
    r->last_pipe = pipe;
    r->window_batches += 1;
    r->current_pipe = (pipe + 1) % p->pipes;  // engine/server.cu:398-399
    return LEGION_OK;
}

extern "C" int legion_runner_sync(LegionRunner *r)
{
    LG_ARG(r != nullptr, "runner is NULL");
    LG_CUDA(cudaSetDevice(r->dev_id));
    if (r->open_window) LG_CUDA(cudaEventRecord(r->t_end, r->s_miss));  // the miss stream ends every batch
    LG_CUDA(cudaStreamSynchronize(r->s_sample));
    LG_CUDA(cudaStreamSynchronize(r->s_gather));
    LG_CUDA(cudaStreamSynchronize(r->s_miss));
    if (r->open_window) {
        float ms = 0.0f, g = 0.0f, m = 0.0f;
        LG_CUDA(cudaEventElapsedTime(&ms, r->t_begin, r->t_end));
        for (auto &pr : r->gather_ev) {
            float t = 0.0f;
            if (cudaEventElapsedTime(&t, pr.first, pr.second) == cudaSuccess) g += t;
            r->ev_free.push_back(pr.first);
            r->ev_free.push_back(pr.second);
        }
        for (auto &pr : r->miss_ev) {
            float t = 0.0f;
            if (cudaEventElapsedTime(&t, pr.first, pr.second) == cudaSuccess) m += t;
            r->ev_free.push_back(pr.first);
            r->ev_free.push_back(pr.second);
        }
        r->gather_ev.clear();
        r->miss_ev.clear();
        r->last_batch_ms = ms;
        r->last_gather_ms = g;
        r->last_miss_ms = m;
        r->last_batches = r->window_batches;
        r->open_window = false;
    }
    for (int i = 0; i < LEGION_INTERBATCH_CON; ++i) r->pipe_busy[i] = false;
    return LEGION_OK;
}

extern "C" int legion_runner_timing(LegionRunner *r, float *batch_ms, float *gather_ms, float *miss_ms,
                                    int32_t *n_batches)
{
    LG_ARG(r != nullptr, "runner is NULL");
    if (batch_ms) *batch_ms = r->last_batch_ms;
    if (gather_ms) *gather_ms = r->last_gather_ms;
    if (miss_ms) *miss_ms = r->last_miss_ms;
    if (n_batches) *n_batches = r->last_batches;
    return LEGION_OK;
}

extern "C" int legion_runner_current_pipe(LegionRunner *r) { return r ? r->current_pipe : LEGION_E_ARG; }

extern "C" int legion_runner_run_once(LegionRunner *r, int32_t global_batch_id, int32_t mode, int32_t local_batch_id,
                                      int32_t timeout_ms)
{
    LG_ARG(r != nullptr, "runner is NULL");
    const int pipe = r->current_pipe;
    if (r->env != nullptr) {
        int rc = legion_ipc_wait(r->env, r->dev_id, pipe, timeout_ms);  // engine/server.cu:337
        if (rc != LEGION_OK) return rc;
    }
    struct timespec t0, t1;
    clock_gettime(CLOCK_MONOTONIC, &t0);
    int rc = legion_runner_enqueue(r, global_batch_id, mode, local_batch_id);
    if (rc != LEGION_OK) return rc;
    LG_CUDA(cudaEventSynchronize(r->pipe_done[pipe]));  // engine/server.cu:356-361
    clock_gettime(CLOCK_MONOTONIC, &t1);
    r->served_us += (t1.tv_sec - t0.tv_sec) * 1e6 + (t1.tv_nsec - t0.tv_nsec) * 1e-3;
    r->served += 1;
    if (r->env != nullptr) {
        rc = legion_ipc_post(r->env, r->dev_id, pipe);  // engine/server.cu:377
        if (rc != LEGION_OK) return rc;
    }
    if (r->served % 1000 == 0 && r->dev_id == 0) {  // engine/server.cu:378-379
        printf("batch id: %d; %lld batches, time per sample: %lld us\n", global_batch_id, r->served,
               (long long)(r->served_us / r->served));
        fflush(stdout);
        r->served = 0;
        r->served_us = 0.0;
    }
    return LEGION_OK;
}

// Serves batches [first, first+count) through the IPC environment with one batch of look-ahead:
// batch b is enqueued as soon as the trainer has released its pipe, and batch b-1 is posted once
// its gather has finished, so the device always holds work for two batches.
extern "C" int legion_runner_serve(LegionRunner *r, int32_t first_global_batch, int32_t count, int32_t timeout_ms)
{
    LG_ARG(r != nullptr && r->env != nullptr, "runner has no IPC environment");
    int prev_pipe = -1;
    for (int32_t b = first_global_batch; b < first_global_batch + count; ++b) {
        const int pipe = r->current_pipe;
        int rc = legion_ipc_wait(r->env, r->dev_id, pipe, timeout_ms);
        if (rc != LEGION_OK) return rc;
        rc = legion_runner_enqueue(r, b, legion_ipc_current_mode(r->env, b), legion_ipc_local_batch_id(r->env, b));
        if (rc != LEGION_OK) return rc;
        if (prev_pipe >= 0) {
            LG_CUDA(cudaEventSynchronize(r->pipe_done[prev_pipe]));
            rc = legion_ipc_post(r->env, r->dev_id, prev_pipe);
            if (rc != LEGION_OK) return rc;
        }
        prev_pipe = pipe;
    }
    if (prev_pipe >= 0) {
        LG_CUDA(cudaEventSynchronize(r->pipe_done[prev_pipe]));
        int rc = legion_ipc_post(r->env, r->dev_id, prev_pipe);
        if (rc != LEGION_OK) return rc;
    }
    return legion_runner_sync(r);
}

extern "C" int legion_runner_destroy(LegionRunner *r)
{
    if (r == nullptr) return LEGION_OK;
    cudaSetDevice(r->dev_id);
    cudaStreamSynchronize(r->s_sample);
    cudaStreamSynchronize(r->s_gather);
    cudaStreamSynchronize(r->s_miss);
    for (auto &pr : r->gather_ev) { cudaEventDestroy(pr.first); cudaEventDestroy(pr.second); }
    for (auto &pr : r->miss_ev) { cudaEventDestroy(pr.first); cudaEventDestroy(pr.second); }
    for (auto e : r->ev_free) cudaEventDestroy(e);
    for (int i = 0; i <= LEGION_MAX_HOPS; ++i) { cudaEventDestroy(r->seg_ready[i]); cudaEventDestroy(r->hit_done[i]); }
    for (int i = 0; i < LEGION_INTERBATCH_CON; ++i) cudaEventDestroy(r->pipe_done[i]);
    cudaEventDestroy(r->t_begin);
    cudaEventDestroy(r->t_end);
    cudaStreamDestroy(r->s_sample);
    cudaStreamDestroy(r->s_gather);
    cudaStreamDestroy(r->s_miss);
    delete r;
    return LEGION_OK;
}
