// Per-GPU runner: the op list of one batch on three streams, the pipe rotation and the hand-off.
//
// Restates GPURunner (sampling_server/src/engine/server.cu:176-416).  The reference builds the
// op list [BatchGenerate, CacheLookup, IOSubmit, (RandomSample, CacheLookup, IOSubmit) x hops,
// IOComplete] over three streams and then blocks: it spins on the last event, and several ops
// read counters back to the host in between.  Here nothing is read back, and three streams carry
// the three resources the path is bound by: sampling (latency of random topology reads) on one,
// lookup + gather of cached rows (HBM / NVLink bandwidth) on a second one behind an event per
// segment, and the fetch of missed rows from pinned host memory (host link) on a third, as one
// launch per batch behind the last gather so that the link sees one long burst instead of three
// short ones.  The gather of hop h overlaps the sampling of hop h+1.
//
// A batch is ~15 small launches, so issuing it from the host costs more than running it.  Every
// size lives on the device and the per-batch parameters are written by the first kernel, so the
// sampling sequence of one pipe is captured once into a CUDA graph; a batch is then one parameter
// update of that first node, one graph launch, the gather launch and the host-link fetch.  The two
// pipes own separate scratch and are launched on two streams, so consecutive batches overlap.
//
// What may overlap with what is decided by who touches the pipe's buffers.  The host-link fetch
// reads nothing of the batch but its miss list (which carries node ids) and writes feature rows, so
// the SAMPLING of batch k+2 (same pipe) starts while the fetch of batch k is still running; only the
// gather of batch k+2, which writes the same feature buffer and miss list, waits for it.  The
// fetches of all batches run in order on one stream of their own at the highest priority: when they
// shared the link, two batches entered and left their host-link phase together and the link idled
// while both sampled.  An LRU cache, whose state changes every batch, keeps whole batches in order.
#include "common.cuh"

#include <string.h>
#include <time.h>

#include <vector>

namespace {

struct EvPair {
    cudaEvent_t a, b;
};

struct PipeGraph {
    cudaGraph_t graph;
    cudaGraphExec_t exec;
    cudaGraphNode_t ctl_node;
    cudaKernelNodeParams ctl_params;
    // argument storage of the first kernel (kept alive for cudaGraphExecKernelNodeSetParams)
    uint4 *a_slots;
    int64_t a_pairs, a_back_pairs;
    int32_t *a_ctl, *a_nc, *a_ec;
    legion::BatchCtl *a_bctl;
    legion::BatchCtl a_value;
    void *args[8];
    bool valid;
    bool launched;  // since the last sync
};

}  // namespace

struct HostOut {
    int32_t *ids, *labels, *agg_src, *agg_dst;
};

struct LegionRunner {
    int32_t dev_id;
    LegionGraph *graph;
    LegionFeatures *feature;
    LegionCache *cache;
    LegionPool *pool;
    LegionIpcEnv *env;
    cudaStream_t s_sample, s_gather, s_miss;
    cudaStream_t s_launch[LEGION_MAX_PIPES];
    cudaEvent_t hit_done[LEGION_MAX_PIPES];   // lookup + gather of the pipe's batch is over
    cudaEvent_t pipe_done[LEGION_MAX_PIPES];
    bool pipe_busy[LEGION_MAX_PIPES];
    int current_pipe, last_pipe;
    bool use_graph, time_kernels;
    PipeGraph pg[LEGION_MAX_PIPES];
    // timing of the batches enqueued since the last sync
    cudaEvent_t t_begin, t_end;
    bool open_window;
    int window_batches;
    std::vector<cudaEvent_t> ev_free;
    std::vector<EvPair> gather_ev, miss_ev, sample_ev;
    std::vector<float> trace;  // per batch of the last timed window: begin/end of sampling, gather, fetch (ms)
    float last_batch_ms, last_gather_ms, last_miss_ms;
    int last_batches, last_timed;
    long long served;
    double served_us;
    // host-buffer batches submitted and not yet collected (oldest first)
    int host_fifo[LEGION_MAX_PIPES + 1];
    int32_t host_seeds[LEGION_MAX_PIPES + 1];
    int host_pending;
    cudaStream_t s_copy;
    // pinned host buffers that the batch on a pipe exports its block structure into (submit_host_to)
    HostOut host_out[LEGION_MAX_PIPES + 1];   // of the submitted batches, oldest first (parallel to host_fifo)
    int64_t host_spec_nodes[LEGION_MAX_PIPES + 1], host_spec_edges[LEGION_MAX_PIPES + 1];  // elements copied ahead
    bool host_exported[LEGION_MAX_PIPES + 1];  // every element of the block structure is on the host
    int32_t host_nc[LEGION_MAX_PIPES + 1][32]; // final counters of an exported batch (the pipe's mirror may already
                                               // belong to the batch that samples ahead on the same pipe)
    int64_t spec_nodes, spec_edges;                 // sizes to copy ahead: the largest batch seen so far plus a margin
    int64_t spec_cnt, host_spec_cnt[LEGION_MAX_PIPES + 1];  // the same for the per-destination edge counts (bytes)
    bool edge_counts;                               // bound batches export edge counts in the place of agg_dst
    bool host_bound[LEGION_MAX_PIPES + 1];  // of the submitted batches, oldest first (parallel to host_fifo)
    bool host_deferred;                          // the newest submitted batch still lacks its back half
    bool host_released;                          // ... and the batch that held its pipe has been collected
    cudaEvent_t sampled[LEGION_MAX_PIPES], exported[LEGION_MAX_PIPES];
    // seed-row staging (stage.cu): one staging per mode's device-resident list, one for a registered host list
    legion::SeedStage stage[4];
    uint8_t *seed_rows[LEGION_MAX_PIPES];   // device: the staged rows of the batch on each pipe
    cudaStream_t s_h2d;                     // copy-engine transfers of staged rows
    cudaEvent_t staged_ev[LEGION_MAX_PIPES];
    bool hit_recorded[LEGION_MAX_PIPES];    // hit_done[pipe] has been recorded at least once
    const legion::SeedStage *pipe_stage[LEGION_MAX_PIPES];  // staging used by the batch on the pipe, or nullptr
    int64_t pipe_stage_first[LEGION_MAX_PIPES];
    int32_t pipe_stage_n[LEGION_MAX_PIPES];
    long long staged_rows;
    // sampling ahead of the hand-off (a pool with fewer slots than pipes)
    cudaEvent_t slot_done[LEGION_MAX_PIPES];   // the batch that used the slot has left it (its fetch is over)
    bool slot_busy[LEGION_MAX_PIPES];
    int32_t *mirror_front[LEGION_MAX_PIPES];   // counter mirror of the batch last sampled on the pipe ...
    int32_t *mirror_back[LEGION_MAX_PIPES];    // ... and of the batch whose gather was issued last
    // host time spent inside submit / collect since the last reset (us): [0] submit, [1] collect, [2] of which waiting
    // for the device, [3] calls
    double host_us[4];
};

static inline double now_us()
{
    struct timespec t;
    clock_gettime(CLOCK_MONOTONIC, &t);
    return t.tv_sec * 1e6 + t.tv_nsec * 1e-3;
}

using namespace legion;

extern "C" int legion_ipc_wait(LegionIpcEnv *e, int32_t dev_id, int32_t pipe, int32_t timeout_ms);
extern "C" int legion_ipc_post(LegionIpcEnv *e, int32_t dev_id, int32_t pipe);
extern "C" int legion_ipc_current_batchsize(LegionIpcEnv *e, int32_t dev_id, int32_t mode);
extern "C" int legion_ipc_current_mode(LegionIpcEnv *e, int32_t global_batch_id);
extern "C" int legion_ipc_local_batch_id(LegionIpcEnv *e, int32_t global_batch_id);
extern "C" int legion_ipc_publish_counters(LegionIpcEnv *e, int32_t dev_id, int32_t pipe, const int32_t *node_counter,
                                           const int32_t *edge_counter);

// Counter words of the finished batch on `pipe`, in the pipe's page-locked staging area.  With at least one hop
// the last sampling kernel has stored both arrays there itself; the lookup + gather over all nodes only adds the
// two snapshot words of the last lookup (nc[2], nc[3] = offset and size of the last hop's nodes,
// operator_impl.cu:85-87), which are a function of the cumulative counts.  Call after the batch has finished.
static const int32_t *final_counters(LegionRunner *r, int pipe)
{
    LegionPool *p = r->pool;
    int32_t *hc = p->h_stage[pipe] + 2 * (size_t)p->batch_size;
    if (p->hop_num > 0) {
        memcpy(hc, r->mirror_back[pipe] != nullptr ? r->mirror_back[pipe] : hc + 32, 128);
        const int hops = hc[LEGION_INTRABATCH_CON * 3 - 1];
        const int n = hc[LEGION_INTRABATCH_CON * 3 + hops];
        const int last = hops > 0 ? hc[LEGION_INTRABATCH_CON * 3 + hops - 1] : 0;
        hc[2] = last;
        hc[3] = n - last;
    }
    return hc;
}

// The finished batch of `pipe` goes to the consumer: counters into the host segment, then the post.
static int post_batch(LegionRunner *r, int pipe)
{
    const int32_t *hc = final_counters(r, pipe);
    const int slot = pipe % r->pool->slots;
    int rc = legion_ipc_publish_counters(r->env, r->dev_id, slot, hc, hc + 16);
    if (rc != LEGION_OK) return rc;
    return legion_ipc_post(r->env, r->dev_id, slot);
}

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
    LG_ARG(env == nullptr || pool->slots <= LEGION_INTERBATCH_CON, "a runner that serves trainers needs a pool of at most 2 hand-off slots");
    LG_ARG(cache == nullptr || cache->kind != 1 || pool->slots == pool->pipes,
           "an LRU cache keeps whole batches in order: it needs a pool whose pipes are its hand-off slots");
    LG_CUDA(cudaSetDevice(dev_id));
    LegionRunner *r = new LegionRunner();
    r->dev_id = dev_id;
    r->graph = graph;
    r->feature = feature;
    r->cache = cache;
    r->pool = pool;
    r->env = env;
    r->current_pipe = 0;
    r->last_pipe = -1;
    r->use_graph = true;
    r->time_kernels = false;
    r->open_window = false;
    r->window_batches = 0;
    r->last_batch_ms = r->last_gather_ms = r->last_miss_ms = 0.0f;
    r->last_batches = r->last_timed = 0;
    r->served = 0;
    r->served_us = 0.0;
    r->host_pending = 0;
    LG_CUDA(cudaStreamCreateWithFlags(&r->s_copy, cudaStreamNonBlocking));
    for (int i = 0; i < LEGION_MAX_PIPES; ++i) {
        LG_CUDA(cudaEventCreateWithFlags(&r->sampled[i], cudaEventDisableTiming));
        LG_CUDA(cudaEventCreateWithFlags(&r->exported[i], cudaEventDisableTiming));
        r->host_bound[i] = false;
    }
    r->host_deferred = false;
    r->host_released = false;
    r->spec_nodes = r->spec_edges = 0;
    r->spec_cnt = 0;
    r->edge_counts = false;
    memset(r->stage, 0, sizeof(r->stage));
    r->staged_rows = 0;
    r->host_us[0] = r->host_us[1] = r->host_us[2] = r->host_us[3] = 0.0;
    LG_CUDA(cudaStreamCreateWithFlags(&r->s_h2d, cudaStreamNonBlocking));
    for (int i = 0; i < LEGION_MAX_PIPES; ++i) {
        r->seed_rows[i] = nullptr;
        r->hit_recorded[i] = false;
        r->slot_busy[i] = false;
        r->mirror_front[i] = r->mirror_back[i] = nullptr;
        LG_CUDA(cudaEventCreateWithFlags(&r->slot_done[i], cudaEventDisableTiming));
        r->pipe_stage[i] = nullptr;
        LG_CUDA(cudaEventCreateWithFlags(&r->staged_ev[i], cudaEventDisableTiming));
    }
    LG_CUDA(cudaStreamCreateWithFlags(&r->s_sample, cudaStreamNonBlocking));
    LG_CUDA(cudaStreamCreateWithFlags(&r->s_gather, cudaStreamNonBlocking));
    {
        // The host-link fetch needs few SM resources but a long time: at the highest priority its
        // CTAs take the next free slots instead of queueing behind the wide kernels of the other batch.
        int lo = 0, hi = 0;
        LG_CUDA(cudaDeviceGetStreamPriorityRange(&lo, &hi));
        LG_CUDA(cudaStreamCreateWithPriority(&r->s_miss, cudaStreamNonBlocking, hi));
    }
    for (int i = 0; i < LEGION_MAX_PIPES; ++i)
        LG_CUDA(cudaEventCreateWithFlags(&r->hit_done[i], cudaEventDisableTiming));
    for (int i = 0; i < LEGION_MAX_PIPES; ++i) {
        LG_CUDA(cudaStreamCreateWithFlags(&r->s_launch[i], cudaStreamNonBlocking));
        LG_CUDA(cudaEventCreateWithFlags(&r->pipe_done[i], cudaEventDisableTiming));
        r->pipe_busy[i] = false;
        r->pg[i] = PipeGraph();
    }
    LG_CUDA(cudaEventCreate(&r->t_begin));
    LG_CUDA(cudaEventCreate(&r->t_end));
    *out = r;
    return LEGION_OK;
}

static void drop_graphs(LegionRunner *r)
{
    for (int i = 0; i < LEGION_MAX_PIPES; ++i) {
        if (r->pg[i].valid) {
            cudaGraphExecDestroy(r->pg[i].exec);
            cudaGraphDestroy(r->pg[i].graph);
            r->pg[i].valid = false;
        }
    }
}

// use_graph: replay each batch as a CUDA graph (default) or issue it launch by launch.
// time_kernels: bracket the gather launches with CUDA events on their streams.
extern "C" int legion_runner_set_options(LegionRunner *r, int32_t use_graph, int32_t time_kernels)
{
    LG_ARG(r != nullptr, "runner is NULL");
    LG_CUDA(cudaSetDevice(r->dev_id));
    LG_CUDA(cudaDeviceSynchronize());
    if ((use_graph != 0) != r->use_graph || (time_kernels != 0) != r->time_kernels) drop_graphs(r);
    r->use_graph = use_graph != 0;
    r->time_kernels = time_kernels != 0;
    return LEGION_OK;
}

// Lookup + gather of cached rows over every node of the batch (one launch; the operator entry
// points still gather hop by hop like the reference: one launch over ~2x10^5 rows runs near HBM
// speed, three launches of 8 k / 60 k / 140 k rows mostly pay start-up and tail).  Missed rows are
// only listed here.
static int issue_gather(LegionRunner *r, cudaStream_t s)
{
    LegionPool *p = r->pool;
    LegionCache *c = r->cache;
    if (c != nullptr) LG_ARG(c->row_bytes == p->row_bytes_out, "cache and pool disagree on the row size");
    EvPair h = { nullptr, nullptr };
    if (r->time_kernels && r->gather_ev.size() < 8192) {
        h.a = take_event(r);
        h.b = take_event(r);
    }
    if (h.a) LG_CUDA(cudaEventRecord(h.a, s));
    int rc = launch_gather_hits(s, p, c, kOpGatherAll);
    if (rc != LEGION_OK) return rc;
    if (h.b) LG_CUDA(cudaEventRecord(h.b, s));
    if (h.a && h.b) r->gather_ev.push_back(h);
    return LEGION_OK;
}

// Seed batch and all hops, on one stream: the part that is captured into the pipe's graph.
static int issue_sampling(LegionRunner *r, const BatchCtl &v, cudaStream_t s)
{
    LegionPool *p = r->pool;
    // with at least one hop, the first hop's counting kernel also takes the seed slice
    const bool defer = p->hop_num > 0;
    int rc = launch_batch_generate(s, p, v, defer);
    for (int h = 0; h < p->hop_num && rc == LEGION_OK; ++h)
        rc = launch_sample_hop(s, p, r->graph, p->fanout[h], h, LEGION_INTRABATCH_CON * (h + 1), defer && h == 0);
    return rc;
}

// The rows that missed (all on the list once the gather is over) and the end-of-batch cache
// maintenance, on s_miss, which every batch shares.
static int issue_back(LegionRunner *r)
{
    LegionPool *p = r->pool;
    LegionCache *c = r->cache;
    if (c != nullptr && c->host_table != nullptr) {
        EvPair m = { nullptr, nullptr };
        if (r->time_kernels && r->miss_ev.size() < 8192) {
            m.a = take_event(r);
            m.b = take_event(r);
        }
        if (m.a) LG_CUDA(cudaEventRecord(m.a, r->s_miss));
        int rc = launch_gather_misses(r->s_miss, p, c);
        if (rc != LEGION_OK) return rc;
        if (m.b) LG_CUDA(cudaEventRecord(m.b, r->s_miss));
        if (m.a && m.b) r->miss_ev.push_back(m);
    }
    return launch_lru_insert(r->s_miss, p, c);  // IOComplete
}

static int capture_pipe(LegionRunner *r, int pipe, const BatchCtl &v)
{
    PipeGraph &g = r->pg[pipe];
    LG_CUDA(cudaStreamBeginCapture(r->s_sample, cudaStreamCaptureModeThreadLocal));
    int rc = issue_sampling(r, v, r->s_sample);
    cudaError_t e = cudaSuccess;
    cudaGraph_t graph = nullptr;
    cudaError_t e2 = cudaStreamEndCapture(r->s_sample, &graph);
    if (rc != LEGION_OK) {
        if (graph) cudaGraphDestroy(graph);
        return rc;
    }
    if (e != cudaSuccess || e2 != cudaSuccess) {
        set_error("graph capture failed: %s", cudaGetErrorString(e != cudaSuccess ? e : e2));
        if (graph) cudaGraphDestroy(graph);
        return LEGION_E_CUDA;
    }
    // the node that carries the per-batch parameters: the first kernel of the batch
    size_t n_nodes = 0;
    LG_CUDA(cudaGraphGetNodes(graph, nullptr, &n_nodes));
    std::vector<cudaGraphNode_t> nodes(n_nodes);
    LG_CUDA(cudaGraphGetNodes(graph, nodes.data(), &n_nodes));
    bool found = false;
    for (size_t i = 0; i < n_nodes && !found; ++i) {
        cudaGraphNodeType t;
        LG_CUDA(cudaGraphNodeGetType(nodes[i], &t));
        if (t != cudaGraphNodeTypeKernel) continue;
        cudaKernelNodeParams kp;
        LG_CUDA(cudaGraphKernelNodeGetParams(nodes[i], &kp));
        if (kp.func == map_clear_kernel_address()) {
            g.ctl_node = nodes[i];
            g.ctl_params = kp;
            g.a_slots = *(uint4 **)kp.kernelParams[0];
            g.a_pairs = *(int64_t *)kp.kernelParams[1];
            g.a_ctl = *(int32_t **)kp.kernelParams[2];
            g.a_nc = *(int32_t **)kp.kernelParams[3];
            g.a_ec = *(int32_t **)kp.kernelParams[4];
            g.a_bctl = *(BatchCtl **)kp.kernelParams[5];
            g.a_value = v;
            g.a_back_pairs = *(int64_t *)kp.kernelParams[7];
            found = true;
        }
    }
    if (!found) {
        set_error("graph capture: parameter node not found");
        cudaGraphDestroy(graph);
        return LEGION_E_STATE;
    }
    g.args[0] = &g.a_slots; g.args[1] = &g.a_pairs; g.args[2] = &g.a_ctl; g.args[3] = &g.a_nc;
    g.args[4] = &g.a_ec; g.args[5] = &g.a_bctl; g.args[6] = &g.a_value; g.args[7] = &g.a_back_pairs;
    g.ctl_params.kernelParams = g.args;
    g.ctl_params.extra = nullptr;
    LG_CUDA(cudaGraphInstantiate(&g.exec, graph, 0));
    g.graph = graph;
    g.valid = true;
    return LEGION_OK;
}

// Enqueues one batch described by `v` on the current pipe.  host_seeds > 0: the seeds and labels
// wait in the pipe's pinned staging area and are copied in first, and both counter arrays are
// copied back to it behind the batch.
// A batch is issued in two halves.  The front half (seed copy, sampling, export of the block structure
// to bound host buffers) only needs the pipe's sampling scratch and its id / edge buffers; the back half
// (lookup + gather, host-link fetch, cache maintenance, counters to the host) needs the pipe's feature
// buffer.  enqueue_ctl issues both at once.  A host-buffer batch with bound outputs may be submitted
// while both pipes still hold uncollected batches: its front half runs at once, its back half is issued
// when the older batch on its pipe has been collected (its features released).
static int issue_front(LegionRunner *r, const BatchCtl &v, int32_t host_seeds, const HostOut *bound, bool pipe_is_held,
                       const SeedStage *st = nullptr, int64_t st_first = 0)
{
    LegionPool *p = r->pool;
    LegionCache *c = r->cache;
    const int pipe = r->current_pipe;
    int rc;
    // Rows of this batch's uncached seeds: one contiguous block of the staging array, brought in by the copy
    // engine while the batch samples.  The pipe's staging area was last read by the gather of the batch that
    // used this pipe before (hit_done).
    r->pipe_stage[pipe] = nullptr;
    if (st != nullptr && st->valid && c != nullptr && st->cache == c && st->fill_gen == c->fill_gen && v.size > 0 &&
        st_first >= 0 && st_first + v.size <= st->count && r->seed_rows[pipe] != nullptr) {
        const int64_t lo = st->pos[st_first], hi = st->pos[st_first + v.size];
        if (hi > lo) {
            if (r->hit_recorded[pipe]) LG_CUDA(cudaStreamWaitEvent(r->s_h2d, r->hit_done[pipe], 0));
            LG_CUDA(cudaMemcpyAsync(r->seed_rows[pipe], st->rows_host + lo * (int64_t)c->row_bytes,
                                    (size_t)(hi - lo) * c->row_bytes, cudaMemcpyHostToDevice, r->s_h2d));
        }
        LG_CUDA(cudaEventRecord(r->staged_ev[pipe], r->s_h2d));
        r->pipe_stage[pipe] = st;
        r->pipe_stage_first[pipe] = st_first;
        r->pipe_stage_n[pipe] = v.size;
        r->staged_rows += hi - lo;
    }
    const bool lru = c != nullptr && c->kind == 1;
    cudaStream_t front = r->use_graph ? r->s_launch[pipe] : r->s_sample;
    if (!r->open_window) {
        LG_CUDA(cudaEventRecord(r->t_begin, front));
        r->open_window = true;
        r->window_batches = 0;
    }
    // With a static cache sampling only rewrites buffers that the last fetch on this pipe does not touch, so it
    // starts at once; the wait for that fetch comes before the gather (issue_rest).  The insertion kernels of
    // an LRU cache read the pipe's ids, so there sampling waits for the pipe's own previous batch.
    const bool early_sampling = !lru && host_seeds == 0;
    if (pipe_is_held) {
        // the older batch on this pipe is still uncollected: its ids and edge lists have left for the
        // host once its export is over, which is all that this half overwrites
        LG_CUDA(cudaStreamWaitEvent(front, r->exported[pipe], 0));
    } else if (!early_sampling && r->pipe_busy[pipe]) {
        LG_CUDA(cudaStreamWaitEvent(front, r->pipe_done[pipe], 0));
    }
    // (an LRU cache has to hold the previous batch's insertions before this batch looks anything up: that wait
    // stands in front of the gather, issue_rest; sampling reads no cache state and runs beside the previous
    // batch's fetch)
    // (the seeds and labels of a host-provided batch wait in the pipe's page-locked staging area, which the
    // batch's first sampling kernel reads in place: 64 KB of zero-copy loads instead of one more transfer to issue)
    EvPair se = { nullptr, nullptr };
    if (r->time_kernels && r->sample_ev.size() < 8192) {
        se.a = take_event(r);
        se.b = take_event(r);
    }
    if (r->use_graph) {
        PipeGraph &g = r->pg[pipe];
        if (!g.valid) {
            rc = capture_pipe(r, pipe, v);
            if (rc != LEGION_OK) return rc;
        }
        g.a_value = v;
        LG_CUDA(cudaGraphExecKernelNodeSetParams(g.exec, g.ctl_node, &g.ctl_params));
        if (se.a) LG_CUDA(cudaEventRecord(se.a, front));
        LG_CUDA(cudaGraphLaunch(g.exec, front));
        g.launched = true;
    } else {
        if (se.a) LG_CUDA(cudaEventRecord(se.a, front));
        rc = issue_sampling(r, v, front);
        if (rc != LEGION_OK) return rc;
    }
    if (se.b) LG_CUDA(cudaEventRecord(se.b, front));
    if (se.a && se.b) r->sample_ev.push_back(se);
    if (bound != nullptr) {
        // ids and edge lists are final once sampling is over: they leave for the host on a stream of
        // their own while the gather and the host-link fetch of the same batch run.  Their sizes are only
        // on the device at this point, so the copies take the size of the largest batch seen so far plus
        // a margin; finish_export moves what a larger batch leaves behind.
        int32_t *early = p->h_stage[pipe] + 2 * (size_t)p->batch_size + 32;
        LG_CUDA(cudaEventRecord(r->sampled[pipe], front));
        LG_CUDA(cudaStreamWaitEvent(r->s_copy, r->sampled[pipe], 0));
        if (p->hop_num == 0) {  // no sampling kernel has stored the counters on the host
            LG_CUDA(cudaMemcpyAsync(early, p->node_counter[pipe], 64, cudaMemcpyDeviceToHost, r->s_copy));
            LG_CUDA(cudaMemcpyAsync(early + 16, p->edge_counter[pipe], 64, cudaMemcpyDeviceToHost, r->s_copy));
        }
        // the labels of a host-provided batch are the labels that came in
        if (bound->labels) memcpy(bound->labels, p->h_stage[pipe] + p->batch_size, 4 * (size_t)host_seeds);
        if (bound->ids && r->spec_nodes > 0)
            LG_CUDA(cudaMemcpyAsync(bound->ids, p->ids[pipe], 4 * (size_t)r->spec_nodes, cudaMemcpyDeviceToHost, r->s_copy));
        if (bound->agg_src && r->spec_edges > 0)
            LG_CUDA(cudaMemcpyAsync(bound->agg_src, p->agg_src[pipe], 4 * (size_t)r->spec_edges, cudaMemcpyDeviceToHost, r->s_copy));
        if (bound->agg_dst && r->edge_counts) {
            if (r->spec_cnt > 0)
                LG_CUDA(cudaMemcpyAsync(bound->agg_dst, p->edge_cnt[pipe], (size_t)r->spec_cnt, cudaMemcpyDeviceToHost, r->s_copy));
        } else if (bound->agg_dst && r->spec_edges > 0) {
            LG_CUDA(cudaMemcpyAsync(bound->agg_dst, p->agg_dst[pipe], 4 * (size_t)r->spec_edges, cudaMemcpyDeviceToHost, r->s_copy));
        }
        LG_CUDA(cudaEventRecord(r->exported[pipe], r->s_copy));
    }
    r->mirror_front[pipe] = v.mirror;
    r->current_pipe = (pipe + 1) % p->pipes;  // engine/server.cu:398-399
    return LEGION_OK;
}

// pipe_was_synced: the host has already waited for the older batch on this pipe (collect), so no
// device-side wait for it is needed.
static int issue_rest(LegionRunner *r, int pipe, int32_t host_seeds, bool bound, bool pipe_was_synced)
{
    LegionPool *p = r->pool;
    LegionCache *c = r->cache;
    int rc;
    const bool lru = c != nullptr && c->kind == 1;
    cudaStream_t front = r->use_graph ? r->s_launch[pipe] : r->s_sample;
    const bool early_sampling = !lru && host_seeds == 0;
    p->pipe = pipe;
    if (early_sampling && r->pipe_busy[pipe] && !pipe_was_synced) LG_CUDA(cudaStreamWaitEvent(front, r->pipe_done[pipe], 0));
    if (lru && r->last_pipe >= 0 && r->last_pipe != pipe && r->pipe_busy[r->last_pipe])
        LG_CUDA(cudaStreamWaitEvent(front, r->pipe_done[r->last_pipe], 0));
    r->mirror_back[pipe] = r->mirror_front[pipe];
    const int slot = pipe % p->slots;
    if (p->slots < p->pipes) {
        // the batch was sampled ahead into the pipe's private buffers: once the batch that used the hand-off slot
        // before has left it, the block structure is copied into the slot, and the gather fills the slot's rows
        if (r->slot_busy[slot] && !pipe_was_synced) LG_CUDA(cudaStreamWaitEvent(front, r->slot_done[slot], 0));
        rc = launch_publish(front, p);
        if (rc != LEGION_OK) return rc;
    }
    if (r->pipe_stage[pipe] != nullptr) {
        const SeedStage *st = r->pipe_stage[pipe];
        LG_CUDA(cudaStreamWaitEvent(front, r->staged_ev[pipe], 0));
        p->stage_rows = r->seed_rows[pipe];
        p->stage_pos = st->pos_dev + r->pipe_stage_first[pipe];
        p->stage_base = st->pos[r->pipe_stage_first[pipe]];
        p->stage_n = r->pipe_stage_n[pipe];
    }
    rc = issue_gather(r, front);
    p->stage_rows = nullptr;
    p->stage_pos = nullptr;
    if (rc != LEGION_OK) return rc;
    if ((host_seeds > 0 || r->env != nullptr) && p->hop_num == 0) {
        // without a sampling kernel nothing has stored the counters on the host (final_counters): copied on this
        // stream so that the next batch on this pipe, which resets them, is ordered behind the copy
        int32_t *hc = p->h_stage[pipe] + 2 * (size_t)p->batch_size;
        LG_CUDA(cudaMemcpyAsync(hc, p->node_counter[pipe], 64, cudaMemcpyDeviceToHost, front));
        LG_CUDA(cudaMemcpyAsync(hc + 16, p->edge_counter[pipe], 64, cudaMemcpyDeviceToHost, front));
    }
    LG_CUDA(cudaEventRecord(r->hit_done[pipe], front));
    r->hit_recorded[pipe] = true;
    LG_CUDA(cudaStreamWaitEvent(r->s_miss, r->hit_done[pipe], 0));
    rc = issue_back(r);
    if (rc != LEGION_OK) return rc;
    // (the export of a bound batch is waited for where it matters -- by collect, and by the batch that samples
    // ahead on this pipe -- not here: the fetch stream is shared by all batches and must not idle behind a copy)
    LG_CUDA(cudaEventRecord(r->pipe_done[pipe], r->s_miss));
    if (p->slots < p->pipes) {
        LG_CUDA(cudaEventRecord(r->slot_done[slot], r->s_miss));
        r->slot_busy[slot] = true;
    }
    if (lru) c->clock += 1;
    r->pipe_busy[pipe] = true;
    r->last_pipe = pipe;
    r->window_batches += 1;
    return LEGION_OK;
}

static int enqueue_ctl(LegionRunner *r, const BatchCtl &v, int32_t host_seeds, const HostOut *bound = nullptr,
                       const SeedStage *st = nullptr, int64_t st_first = 0)
{
    const int pipe = r->current_pipe;
    int rc = issue_front(r, v, host_seeds, bound, false, st, st_first);
    if (rc != LEGION_OK) return rc;
    return issue_rest(r, pipe, host_seeds, bound != nullptr, false);
}

static int enqueue_impl(LegionRunner *r, int32_t global_batch_id, int32_t mode, int32_t local_batch_id, bool front_only);

extern "C" int legion_runner_enqueue(LegionRunner *r, int32_t global_batch_id, int32_t mode, int32_t local_batch_id)
{
    return enqueue_impl(r, global_batch_id, mode, local_batch_id, false);
}

// front_only: sampling (and the staging of seed rows) only; the caller issues the gather half with issue_rest
// when the batch's hand-off slot is free.
static int enqueue_impl(LegionRunner *r, int32_t global_batch_id, int32_t mode, int32_t local_batch_id, bool front_only)
{
    LG_ARG(r != nullptr, "runner is NULL");
    LG_ARG(mode >= 0 && mode <= 2, "invalid mode");
    LG_ARG(r->host_pending == 0, "host-buffer batches are waiting to be collected");
    LG_CUDA(cudaSetDevice(r->dev_id));
    LegionPool *p = r->pool;
    const int pipe = r->current_pipe;
    int rc = legion_pool_set_batch(p, local_batch_id, mode, pipe, (uint32_t)global_batch_id);
    if (rc != LEGION_OK) return rc;
    if (p->slots < p->pipes) p->mirror_flip[pipe] ^= 1;
    int32_t bs = p->batch_size;
    if (r->env != nullptr) {
        bs = legion_ipc_current_batchsize(r->env, r->dev_id, mode);
        LG_ARG(bs > 0 && bs <= p->batch_size, "batch size of this mode is above the pool's");
    }
    const int32_t total_cap = r->feature->count[mode];
    LG_ARG(r->feature->ids[mode] != nullptr && total_cap > 0, "no seed list for this mode");
    LG_ARG(local_batch_id >= 0, "negative batch number");
    const int64_t first = (int64_t)bs * local_batch_id;
    int64_t size = ((int64_t)bs * (local_batch_id + 1) >= total_cap) ? (total_cap - first) : bs;  // operator_impl.cu:162
    if (size < 0) size = 0;
    const SeedStage *st = (r->stage[mode].valid && r->stage[mode].ids_dev == r->feature->ids[mode] &&
                           r->stage[mode].count == total_cap) ? &r->stage[mode] : nullptr;
    const BatchCtl v = make_batch_ctl(p, r->cache, r->feature->ids[mode], r->feature->labels[mode], total_cap, first,
                                      (int32_t)size, r->graph->n_nodes);
    if (front_only) return issue_front(r, v, 0, nullptr, false, st, first);
    return enqueue_ctl(r, v, 0, nullptr, st, first);
}

// Host-buffer interface with batches in flight.  submit copies the seeds in and starts the batch;
// collect waits for the oldest submitted batch and copies its block structure (and, optionally, its
// gathered rows) out.  Up to `pipes` batches may be submitted before the first collect, so the copies
// of one batch overlap the sampling and gathering of the next.
// Completes the export of the i-th submitted batch: waits for its copies, reads its sizes and moves
// whatever lies beyond the sizes that were copied ahead.  Must run before the batch's id / edge buffers
// are reused.  Also raises the sizes that later batches copy ahead.
static int finish_export(LegionRunner *r, int i)
{
    if (!r->host_bound[i] || r->host_exported[i]) return LEGION_OK;
    LegionPool *p = r->pool;
    const int pipe = r->host_fifo[i];
    {
        const double w0 = now_us();
        LG_CUDA(cudaEventSynchronize(r->exported[pipe]));
        r->host_us[2] += now_us() - w0;
    }
    const int32_t *early = p->h_stage[pipe] + 2 * (size_t)p->batch_size + 32;
    {
        // the batch's final counters: what sampling left plus the snapshot words of the last lookup (final_counters)
        int32_t *nc = r->host_nc[i];
        memcpy(nc, early, 128);
        const int h = nc[LEGION_INTRABATCH_CON * 3 - 1];
        const int last = h > 0 ? nc[LEGION_INTRABATCH_CON * 3 + h - 1] : 0;
        nc[2] = last;
        nc[3] = nc[LEGION_INTRABATCH_CON * 3 + h] - last;
    }
    const int hops = early[LEGION_INTRABATCH_CON * 3 - 1];
    const int64_t n_nodes = early[LEGION_INTRABATCH_CON * 3 + hops];
    const int64_t n_edges = (int64_t)early[16] + early[17];
    const HostOut &o = r->host_out[i];
    const int64_t sn = r->host_spec_nodes[i], se = r->host_spec_edges[i];
    bool tail = false;
    if (o.ids && n_nodes > sn) {
        LG_CUDA(cudaMemcpyAsync(o.ids + sn, p->ids[pipe] + sn, 4 * (size_t)(n_nodes - sn), cudaMemcpyDeviceToHost, r->s_copy));
        tail = true;
    }
    if (o.agg_src && n_edges > se) {
        LG_CUDA(cudaMemcpyAsync(o.agg_src + se, p->agg_src[pipe] + se, 4 * (size_t)(n_edges - se), cudaMemcpyDeviceToHost, r->s_copy));
        tail = true;
    }
    // per-destination edge counts: one byte for every node known at the start of each hop
    int64_t n_cnt = 0;
    for (int h = 0; h < hops; ++h) n_cnt += early[LEGION_INTRABATCH_CON * 3 + h];
    if (o.agg_dst && r->edge_counts) {
        const int64_t sc = r->host_spec_cnt[i];
        if (n_cnt > sc) {
            LG_CUDA(cudaMemcpyAsync(reinterpret_cast<uint8_t *>(o.agg_dst) + sc, p->edge_cnt[pipe] + sc, (size_t)(n_cnt - sc),
                                    cudaMemcpyDeviceToHost, r->s_copy));
            tail = true;
        }
    } else if (o.agg_dst && n_edges > se) {
        LG_CUDA(cudaMemcpyAsync(o.agg_dst + se, p->agg_dst[pipe] + se, 4 * (size_t)(n_edges - se), cudaMemcpyDeviceToHost, r->s_copy));
        tail = true;
    }
    if (tail) LG_CUDA(cudaStreamSynchronize(r->s_copy));
    r->host_exported[i] = true;
    // the sizes copied ahead follow the largest batch seen so far: 1/64 of headroom above it, rounded up to 256 elements
    // (every byte of headroom crosses the host link for nothing)
    int64_t want_n = (n_nodes + n_nodes / 64 + 255) / 256 * 256, want_e = (n_edges + n_edges / 64 + 255) / 256 * 256;
    if (want_n > p->max_nodes) want_n = p->max_nodes;
    if (want_e > p->max_edges) want_e = p->max_edges;
    if (want_n > r->spec_nodes) r->spec_nodes = want_n;
    if (want_e > r->spec_edges) r->spec_edges = want_e;
    int64_t want_c = (n_cnt + n_cnt / 64 + 255) / 256 * 256;
    const int64_t cap_c = (int64_t)(p->hop_num > 0 ? p->hop_num : 1) * p->max_nodes;
    if (want_c > cap_c) want_c = cap_c;
    if (want_c > r->spec_cnt) r->spec_cnt = want_c;
    return LEGION_OK;
}

// Back half of the batch that sampled ahead, once the batch that held its pipe has been collected and
// the caller has come back (its rows in the pipe's feature buffer are given up by that next call).
static int flush_deferred(LegionRunner *r)
{
    if (!r->host_deferred || !r->host_released) return LEGION_OK;
    r->host_deferred = false;
    r->host_released = false;
    const int last = r->host_pending - 1;
    return issue_rest(r, r->host_fifo[last], r->host_seeds[last], true, true);
}

static int submit_host_impl(LegionRunner *r, const int32_t *seeds, const int32_t *labels, int32_t n_seeds,
                            int32_t global_batch_id, const HostOut *bound);

extern "C" int legion_runner_submit_host(LegionRunner *r, const int32_t *seeds, const int32_t *labels, int32_t n_seeds,
                                         int32_t global_batch_id)
{
    return submit_host_impl(r, seeds, labels, n_seeds, global_batch_id, nullptr);
}

// Output arrays are checked once: the driver query costs as much as a launch, and a caller rotates a handful of
// arrays.  (A stale entry cannot make a kernel fault: these arrays are only ever the target of copy-engine
// transfers.)
static bool device_can_write_query(const void *p);

static bool device_can_write(const void *p)
{
    if (p == nullptr) return true;
    static thread_local const void *known[32];
    static thread_local int n_known = 0;
    for (int i = 0; i < n_known; ++i)
        if (known[i] == p) return true;
    if (!device_can_write_query(p)) return false;
    known[n_known < 32 ? n_known++ : (n_known = 1, 0)] = p;
    return true;
}

static bool device_can_write_query(const void *p)
{
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return (a.type == cudaMemoryTypeHost || a.type == cudaMemoryTypeManaged) && ((uintptr_t)p & 15) == 0;
}

extern "C" int legion_runner_set_edge_counts(LegionRunner *r, int32_t on)
{
    LG_ARG(r != nullptr, "runner is NULL");
    if (r->host_pending != 0) {
        set_error("legion_runner_set_edge_counts: %d batches are waiting to be collected", r->host_pending);
        return LEGION_E_STATE;
    }
    r->edge_counts = on != 0;
    return LEGION_OK;
}

extern "C" int legion_runner_submit_host_to(LegionRunner *r, const int32_t *seeds, const int32_t *labels, int32_t n_seeds,
                                            int32_t global_batch_id, int32_t *ids_out, int32_t *labels_out,
                                            int32_t *agg_src_out, int32_t *agg_dst_out)
{
    LG_ARG(device_can_write(ids_out) && device_can_write(labels_out) && device_can_write(agg_src_out) &&
               device_can_write(agg_dst_out),
           "output buffers must be page-locked host memory (cudaHostAlloc / cudaHostRegister), 16-byte aligned");
    HostOut b{ ids_out, labels_out, agg_src_out, agg_dst_out };
    return submit_host_impl(r, seeds, labels, n_seeds, global_batch_id, &b);
}

static int submit_host_body(LegionRunner *r, const int32_t *seeds, const int32_t *labels, int32_t n_seeds,
                            int32_t global_batch_id, const HostOut *bound);

static int submit_host_impl(LegionRunner *r, const int32_t *seeds, const int32_t *labels, int32_t n_seeds,
                            int32_t global_batch_id, const HostOut *bound)
{
    const double t0 = now_us();
    int rc = submit_host_body(r, seeds, labels, n_seeds, global_batch_id, bound);
    if (r != nullptr) {
        r->host_us[0] += now_us() - t0;
        r->host_us[3] += 1.0;
    }
    return rc;
}

static int submit_host_body(LegionRunner *r, const int32_t *seeds, const int32_t *labels, int32_t n_seeds,
                            int32_t global_batch_id, const HostOut *bound)
{
    LG_ARG(r != nullptr && seeds != nullptr && labels != nullptr, "NULL pointer");
    LegionPool *p = r->pool;
    LG_ARG(n_seeds > 0 && n_seeds <= p->batch_size, "n_seeds above the pool's batch size");
    LG_ARG(p->slots == p->pipes, "the host-buffer calls need a pool whose pipes are its hand-off slots (legion_pool_create)");
    LG_CUDA(cudaSetDevice(r->dev_id));
    {
        int frc = flush_deferred(r);
        if (frc != LEGION_OK) return frc;
    }
    const bool lru = r->cache != nullptr && r->cache->kind == 1;
    // one batch beyond the pipes may start its sampling early when its own and the held batch's block
    // structure go to bound host buffers (the held batch's ids and edge lists are then on the host already)
    const bool extra = r->host_pending == p->pipes && bound != nullptr && !r->host_deferred && !lru &&
                       r->host_bound[0] && r->host_fifo[0] == r->current_pipe;
    if (r->host_pending >= p->pipes && !extra) {
        set_error("legion_runner_submit_host: %d batches are in flight, collect one first", r->host_pending);
        return LEGION_E_STATE;
    }
    LG_CUDA(cudaSetDevice(r->dev_id));
    const int pipe = r->current_pipe;
    int rc = legion_pool_set_batch(p, 0, LEGION_TRAINMODE, pipe, (uint32_t)global_batch_id);
    if (rc != LEGION_OK) return rc;
    if (extra) {
        // the held batch's ids and edge lists must be on the host in full before this batch's sampling
        // overwrites them; the staging area of this pipe still holds the held batch's counters (read by
        // its collect), the seed words were consumed when that batch started
        rc = finish_export(r, 0);
        if (rc != LEGION_OK) return rc;
    }
    memcpy(p->h_stage[pipe], seeds, sizeof(int32_t) * n_seeds);
    memcpy(p->h_stage[pipe] + p->batch_size, labels, sizeof(int32_t) * n_seeds);
    const BatchCtl v = make_batch_ctl(p, r->cache, p->h_stage[pipe], p->h_stage[pipe] + p->batch_size, n_seeds, 0, n_seeds,
                                      r->graph->n_nodes);
    const int64_t spec_n = r->spec_nodes, spec_e = r->spec_edges, spec_c = r->spec_cnt;  // what issue_front copies ahead
    // a batch that is a slice of the registered host list (by address, and still holding what the list held
    // at registration) gets the rows of its uncached seeds by the copy engine
    const SeedStage *st = nullptr;
    int64_t st_first = 0;
    const SeedStage &hs = r->stage[3];
    if (hs.valid && hs.host_base != nullptr && seeds >= hs.host_base && seeds + n_seeds <= hs.host_base + hs.count) {
        st_first = seeds - hs.host_base;
        if (memcmp(seeds, hs.host_copy + st_first, sizeof(int32_t) * (size_t)n_seeds) == 0) st = &hs;
    }
    if (extra) {
        rc = issue_front(r, v, n_seeds, bound, true, st, st_first);
        if (rc == LEGION_OK) r->host_deferred = true;
    } else {
        rc = enqueue_ctl(r, v, n_seeds, bound, st, st_first);
    }
    if (rc != LEGION_OK) return rc;
    r->host_bound[r->host_pending] = bound != nullptr;
    r->host_out[r->host_pending] = bound != nullptr ? *bound : HostOut{ nullptr, nullptr, nullptr, nullptr };
    r->host_spec_nodes[r->host_pending] = spec_n;
    r->host_spec_edges[r->host_pending] = spec_e;
    r->host_spec_cnt[r->host_pending] = spec_c;
    r->host_exported[r->host_pending] = false;
    r->host_fifo[r->host_pending] = pipe;
    r->host_seeds[r->host_pending] = n_seeds;
    r->host_pending += 1;
    return LEGION_OK;
}

static int collect_host_body(LegionRunner *r, int32_t *ids_out, int32_t *labels_out, int32_t *agg_src_out,
                             int32_t *agg_dst_out, int32_t node_counter_out[16], int32_t edge_counter_out[16],
                             void *features_out);

extern "C" int legion_runner_collect_host(LegionRunner *r, int32_t *ids_out, int32_t *labels_out, int32_t *agg_src_out,
                                          int32_t *agg_dst_out, int32_t node_counter_out[16],
                                          int32_t edge_counter_out[16], void *features_out)
{
    const double t0 = now_us();
    int rc = collect_host_body(r, ids_out, labels_out, agg_src_out, agg_dst_out, node_counter_out, edge_counter_out, features_out);
    if (r != nullptr) r->host_us[1] += now_us() - t0;
    return rc;
}

// Host time inside legion_runner_submit_host[_to] and legion_runner_collect_host since the last call of this
// function, in microseconds: out[0] submit, out[1] collect, out[2] the part of collect spent waiting for the
// device, out[3] batches submitted.  Tells a host-bound hand-off from a device-bound one.
extern "C" int legion_runner_host_times(LegionRunner *r, double out[4])
{
    LG_ARG(r != nullptr && out != nullptr, "NULL pointer");
    for (int i = 0; i < 4; ++i) {
        out[i] = r->host_us[i];
        r->host_us[i] = 0.0;
    }
    return LEGION_OK;
}

static int collect_host_body(LegionRunner *r, int32_t *ids_out, int32_t *labels_out, int32_t *agg_src_out,
                             int32_t *agg_dst_out, int32_t node_counter_out[16], int32_t edge_counter_out[16],
                             void *features_out)
{
    LG_ARG(r != nullptr && node_counter_out != nullptr && edge_counter_out != nullptr, "NULL pointer");
    if (r->host_pending == 0) {
        set_error("legion_runner_collect_host: nothing was submitted");
        return LEGION_E_STATE;
    }
    LG_CUDA(cudaSetDevice(r->dev_id));
    {
        int frc = flush_deferred(r);
        if (frc != LEGION_OK) return frc;
    }
    if (r->host_deferred && r->host_pending == 1) {
        set_error("legion_runner_collect_host: internal: a batch without its gather is the only one pending");
        return LEGION_E_STATE;
    }
    LegionPool *p = r->pool;
    const int pipe = r->host_fifo[0];
    const int32_t n_seeds = r->host_seeds[0];
    const bool bound = r->host_bound[0];
    {
        int frc = finish_export(r, 0);
        if (frc != LEGION_OK) return frc;
    }
    int32_t kept[32];
    memcpy(kept, r->host_nc[0], sizeof(kept));  // this batch's, if it was exported (taken before the fifo moves)
    for (int i = 1; i < r->host_pending; ++i) {
        r->host_fifo[i - 1] = r->host_fifo[i];
        r->host_seeds[i - 1] = r->host_seeds[i];
        r->host_bound[i - 1] = r->host_bound[i];
        r->host_out[i - 1] = r->host_out[i];
        r->host_spec_nodes[i - 1] = r->host_spec_nodes[i];
        r->host_spec_edges[i - 1] = r->host_spec_edges[i];
        r->host_spec_cnt[i - 1] = r->host_spec_cnt[i];
        r->host_exported[i - 1] = r->host_exported[i];
        memcpy(r->host_nc[i - 1], r->host_nc[i], sizeof(r->host_nc[0]));
    }
    r->host_pending -= 1;
    {
        const double w0 = now_us();
        LG_CUDA(cudaEventSynchronize(r->pipe_done[pipe]));
        r->host_us[2] += now_us() - w0;
    }
    const int32_t *hc = (bound && p->hop_num > 0) ? kept : final_counters(r, pipe);
    memcpy(node_counter_out, hc, 64);
    memcpy(edge_counter_out, hc + 16, 64);
    // the caller reads this batch's rows from the pipe's feature buffer now; the batch that already
    // sampled on this pipe gathers into it at the next call on this runner (flush_deferred)
    if (r->host_deferred) r->host_released = true;
    const int hops = hc[LEGION_INTRABATCH_CON * 3 - 1];
    const int64_t n_nodes = hc[LEGION_INTRABATCH_CON * 3 + hops];
    const int64_t n_edges = (int64_t)hc[16] + hc[17];
    cudaStream_t s = r->s_copy;
    if (bound) {
        // the batch wrote its block structure into the buffers named at submit time
        if (features_out == nullptr) return LEGION_OK;
        ids_out = labels_out = agg_src_out = agg_dst_out = nullptr;
    }
    if (ids_out) LG_CUDA(cudaMemcpyAsync(ids_out, p->ids[pipe], 4 * n_nodes, cudaMemcpyDeviceToHost, s));
    if (labels_out) LG_CUDA(cudaMemcpyAsync(labels_out, p->labels[pipe], 4 * (int64_t)n_seeds, cudaMemcpyDeviceToHost, s));
    if (agg_src_out) LG_CUDA(cudaMemcpyAsync(agg_src_out, p->agg_src[pipe], 4 * n_edges, cudaMemcpyDeviceToHost, s));
    if (agg_dst_out && r->edge_counts) {
        int64_t n_cnt = 0;
        for (int h = 0; h < hops; ++h) n_cnt += hc[LEGION_INTRABATCH_CON * 3 + h];
        if (n_cnt > 0) LG_CUDA(cudaMemcpyAsync(agg_dst_out, p->edge_cnt[pipe], (size_t)n_cnt, cudaMemcpyDeviceToHost, s));
    } else if (agg_dst_out) {
        LG_CUDA(cudaMemcpyAsync(agg_dst_out, p->agg_dst[pipe], 4 * n_edges, cudaMemcpyDeviceToHost, s));
    }
    if (features_out)
        LG_CUDA(cudaMemcpyAsync(features_out, p->features[pipe], n_nodes * (int64_t)p->row_bytes_out,
                                cudaMemcpyDeviceToHost, s));
    LG_CUDA(cudaStreamSynchronize(s));
    return LEGION_OK;
}

extern "C" int legion_runner_sync(LegionRunner *r)
{
    LG_ARG(r != nullptr, "runner is NULL");
    LG_CUDA(cudaSetDevice(r->dev_id));
    {
        int frc = flush_deferred(r);
        if (frc != LEGION_OK) return frc;
    }
    if (r->open_window) LG_CUDA(cudaEventRecord(r->t_end, r->s_miss));  // the miss stream ends every batch
    LG_CUDA(cudaStreamSynchronize(r->s_sample));
    LG_CUDA(cudaStreamSynchronize(r->s_gather));
    LG_CUDA(cudaStreamSynchronize(r->s_miss));
    LG_CUDA(cudaStreamSynchronize(r->s_h2d));
    LG_CUDA(cudaStreamSynchronize(r->s_copy));
    for (int i = 0; i < LEGION_MAX_PIPES; ++i) LG_CUDA(cudaStreamSynchronize(r->s_launch[i]));
    if (r->open_window) {
        float ms = 0.0f, g = 0.0f, m = 0.0f;
        int timed = 0;
        LG_CUDA(cudaEventElapsedTime(&ms, r->t_begin, r->t_end));
        for (auto &pr : r->gather_ev) {
            float t = 0.0f;
            if (cudaEventElapsedTime(&t, pr.a, pr.b) == cudaSuccess) g += t;
            r->ev_free.push_back(pr.a);
            r->ev_free.push_back(pr.b);
        }
        for (auto &pr : r->miss_ev) {
            float t = 0.0f;
            if (cudaEventElapsedTime(&t, pr.a, pr.b) == cudaSuccess) m += t;
            r->ev_free.push_back(pr.a);
            r->ev_free.push_back(pr.b);
        }
        if (r->time_kernels) timed = (int)r->gather_ev.size();
        r->trace.clear();
        if (r->time_kernels && r->sample_ev.size() == r->gather_ev.size() &&
            (r->miss_ev.empty() || r->miss_ev.size() == r->gather_ev.size())) {
            for (size_t i = 0; i < r->gather_ev.size(); ++i) {
                float v6[6] = { 0, 0, 0, 0, 0, 0 };
                cudaEventElapsedTime(&v6[0], r->t_begin, r->sample_ev[i].a);
                cudaEventElapsedTime(&v6[1], r->t_begin, r->sample_ev[i].b);
                cudaEventElapsedTime(&v6[2], r->t_begin, r->gather_ev[i].a);
                cudaEventElapsedTime(&v6[3], r->t_begin, r->gather_ev[i].b);
                if (!r->miss_ev.empty()) {
                    cudaEventElapsedTime(&v6[4], r->t_begin, r->miss_ev[i].a);
                    cudaEventElapsedTime(&v6[5], r->t_begin, r->miss_ev[i].b);
                }
                r->trace.insert(r->trace.end(), v6, v6 + 6);
            }
        }
        for (auto &pr : r->sample_ev) {
            r->ev_free.push_back(pr.a);
            r->ev_free.push_back(pr.b);
        }
        r->sample_ev.clear();
        r->gather_ev.clear();
        r->miss_ev.clear();
        r->last_batch_ms = ms;
        r->last_gather_ms = g;
        r->last_miss_ms = m;
        r->last_batches = r->window_batches;
        r->last_timed = timed;
        r->open_window = false;
    }
    for (int i = 0; i < LEGION_MAX_PIPES; ++i) {
        r->pipe_busy[i] = false;
        r->slot_busy[i] = false;
        r->pg[i].launched = false;
    }
    return LEGION_OK;
}

extern "C" int legion_runner_timing(LegionRunner *r, float *batch_ms, float *gather_ms, float *miss_ms,
                                    int32_t *n_batches, int32_t *n_timed)
{
    LG_ARG(r != nullptr, "runner is NULL");
    if (batch_ms) *batch_ms = r->last_batch_ms;
    if (gather_ms) *gather_ms = r->last_gather_ms;
    if (miss_ms) *miss_ms = r->last_miss_ms;
    if (n_batches) *n_batches = r->last_batches;
    if (n_timed) *n_timed = r->last_timed;
    return LEGION_OK;
}

// Stage times of the last window that ran with time_kernels: six floats per batch, the begin and
// end of its sampling, of its gather and of its host-link fetch, in ms since the window's start.
// Returns the number of batches written (at most max_batches).
extern "C" int legion_runner_trace(LegionRunner *r, float *out, int32_t max_batches)
{
    if (r == nullptr || out == nullptr || max_batches < 0) return LEGION_E_ARG;
    int n = (int)(r->trace.size() / 6);
    if (n > max_batches) n = max_batches;
    memcpy(out, r->trace.data(), sizeof(float) * 6 * (size_t)n);
    return n;
}

extern "C" int legion_runner_current_pipe(LegionRunner *r) { return r ? r->current_pipe : LEGION_E_ARG; }

extern "C" int legion_runner_run_once(LegionRunner *r, int32_t global_batch_id, int32_t mode, int32_t local_batch_id,
                                      int32_t timeout_ms)
{
    LG_ARG(r != nullptr, "runner is NULL");
    const int pipe = r->current_pipe;
    if (r->env != nullptr) {
        int rc = legion_ipc_wait(r->env, r->dev_id, pipe % r->pool->slots, timeout_ms);  // engine/server.cu:337
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
        rc = post_batch(r, pipe);  // engine/server.cu:377
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
    LegionPool *p = r->pool;
    if (p->slots < p->pipes) {
        // Sampling ahead of the hand-off: the pool has more pipes than the segment has slots, so up to `pipes`
        // batches are sampled (into private buffers) while the trainer still holds the slots; the gather half of
        // batch b is issued when the trainer has released b's slot, batch b - 1 is posted once it has finished.
        LG_ARG(r->host_pending == 0, "host-buffer batches are waiting to be collected");
        const int32_t end = first_global_batch + count;
        const int pipe0 = r->current_pipe;
        int32_t nf = first_global_batch;
        for (int32_t b = first_global_batch; b < end; ++b) {
            int rc;
            while (nf < end && nf < b + p->pipes) {
                rc = enqueue_impl(r, nf, legion_ipc_current_mode(r->env, nf), legion_ipc_local_batch_id(r->env, nf), true);
                if (rc != LEGION_OK) return rc;
                ++nf;
            }
            const int pipe = (pipe0 + (b - first_global_batch)) % p->pipes;
            rc = legion_ipc_wait(r->env, r->dev_id, pipe % p->slots, timeout_ms);
            if (rc != LEGION_OK) return rc;
            LG_CUDA(cudaSetDevice(r->dev_id));
            rc = issue_rest(r, pipe, 0, false, false);
            if (rc != LEGION_OK) return rc;
            if (prev_pipe >= 0) {
                LG_CUDA(cudaEventSynchronize(r->pipe_done[prev_pipe]));
                rc = post_batch(r, prev_pipe);
                if (rc != LEGION_OK) return rc;
            }
            prev_pipe = pipe;
        }
        if (prev_pipe >= 0) {
            LG_CUDA(cudaEventSynchronize(r->pipe_done[prev_pipe]));
            int rc = post_batch(r, prev_pipe);
            if (rc != LEGION_OK) return rc;
        }
        return legion_runner_sync(r);
    }
    for (int32_t b = first_global_batch; b < first_global_batch + count; ++b) {
        const int pipe = r->current_pipe;
        int rc = legion_ipc_wait(r->env, r->dev_id, pipe, timeout_ms);
        if (rc != LEGION_OK) return rc;
        rc = legion_runner_enqueue(r, b, legion_ipc_current_mode(r->env, b), legion_ipc_local_batch_id(r->env, b));
        if (rc != LEGION_OK) return rc;
        if (prev_pipe >= 0) {
            LG_CUDA(cudaEventSynchronize(r->pipe_done[prev_pipe]));
            rc = post_batch(r, prev_pipe);
            if (rc != LEGION_OK) return rc;
        }
        prev_pipe = pipe;
    }
    if (prev_pipe >= 0) {
        LG_CUDA(cudaEventSynchronize(r->pipe_done[prev_pipe]));
        int rc = post_batch(r, prev_pipe);
        if (rc != LEGION_OK) return rc;
    }
    return legion_runner_sync(r);
}

// The presampling epoch (GPUServer::PreSc -> GPURunner::RunPreSc, engine/server.cu:94-122,313-328): batches
// [first, first+count) of the training list are sampled (no lookup, no gather) and every node they touch
// is counted in counts_dev (one uint32 per node, the caller zeroes it), the input of
// legion_cache_hotness_order.
extern "C" int legion_runner_presample(LegionRunner *r, int32_t first_batch, int32_t count, uint32_t *counts_dev)
{
    LG_ARG(r != nullptr && counts_dev != nullptr && count >= 0 && first_batch >= 0, "bad argument");
    LG_ARG(r->host_pending == 0, "host-buffer batches are waiting to be collected");
    int rc = legion_runner_sync(r);
    if (rc != LEGION_OK) return rc;
    LegionPool *p = r->pool;
    const int32_t total_cap = r->feature->count[LEGION_TRAINMODE];
    LG_ARG(r->feature->ids[LEGION_TRAINMODE] != nullptr && total_cap > 0, "no training seed list");
    for (int32_t b = first_batch; b < first_batch + count; ++b) {
        rc = legion_pool_set_batch(p, b, LEGION_TRAINMODE, 0, (uint32_t)b);
        if (rc != LEGION_OK) return rc;
        const int64_t first = (int64_t)p->batch_size * b;
        int64_t size = ((int64_t)p->batch_size * (b + 1) >= total_cap) ? (total_cap - first) : p->batch_size;
        if (size <= 0) break;
        rc = launch_batch_generate(r->s_sample, p, make_batch_ctl(p, r->cache, r->feature->ids[LEGION_TRAINMODE],
                                                                   r->feature->labels[LEGION_TRAINMODE], total_cap, first,
                                                                   (int32_t)size, r->graph->n_nodes));
        for (int h = 0; h < p->hop_num && rc == LEGION_OK; ++h)
            rc = launch_sample_hop(r->s_sample, p, r->graph, p->fanout[h], h, LEGION_INTRABATCH_CON * (h + 1));
        if (rc == LEGION_OK) rc = launch_hotness(r->s_sample, p, counts_dev);
        if (rc != LEGION_OK) return rc;
    }
    LG_CUDA(cudaStreamSynchronize(r->s_sample));
    return LEGION_OK;
}

// ---- seed-row staging ------------------------------------------------------------------------------------

static int stage_prepare(LegionRunner *r, SeedStage *st)
{
    LG_ARG(r->cache != nullptr, "the runner has no cache");
    LG_CUDA(cudaSetDevice(r->dev_id));
    int rc = legion_runner_sync(r);
    if (rc != LEGION_OK) return rc;
    stage_free(st);
    for (int i = 0; i < r->pool->pipes; ++i) {
        if (r->seed_rows[i] == nullptr)
            LG_CUDA(cudaMalloc(reinterpret_cast<void **>(&r->seed_rows[i]), (size_t)r->pool->batch_size * r->pool->row_bytes_out));
    }
    return LEGION_OK;
}

extern "C" int legion_runner_stage_seeds(LegionRunner *r, int32_t mode, int64_t *staged_rows_out)
{
    LG_ARG(r != nullptr && mode >= 0 && mode <= 2, "bad argument");
    LG_ARG(r->feature->ids[mode] != nullptr && r->feature->count[mode] > 0, "no seed list for this mode");
    LG_ARG(r->host_pending == 0, "host-buffer batches are waiting to be collected");
    SeedStage *st = &r->stage[mode];
    int rc = stage_prepare(r, st);
    if (rc != LEGION_OK) return rc;
    rc = stage_build(r->cache, r->feature->ids[mode], r->feature->count[mode], r->pool->sm_count, st);
    if (rc == LEGION_OK && staged_rows_out != nullptr) *staged_rows_out = st->rows;
    return rc;
}

extern "C" int legion_runner_register_host_seeds(LegionRunner *r, const int32_t *seeds_host, int32_t count,
                                                 int64_t *staged_rows_out)
{
    LG_ARG(r != nullptr && seeds_host != nullptr && count > 0, "bad argument");
    LG_ARG(r->host_pending == 0, "host-buffer batches are waiting to be collected");
    SeedStage *st = &r->stage[3];
    int rc = stage_prepare(r, st);
    if (rc != LEGION_OK) return rc;
    int32_t *dev = nullptr;
    LG_CUDA(cudaMalloc(reinterpret_cast<void **>(&dev), sizeof(int32_t) * (size_t)count));
    cudaError_t e = cudaMemcpy(dev, seeds_host, sizeof(int32_t) * (size_t)count, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
        cudaFree(dev);
        LG_CUDA(e);
    }
    rc = stage_build(r->cache, dev, count, r->pool->sm_count, st);
    if (rc != LEGION_OK) {
        cudaFree(dev);
        return rc;
    }
    st->own_ids_dev = dev;
    st->host_base = seeds_host;
    st->host_copy = new int32_t[(size_t)count];
    memcpy(st->host_copy, seeds_host, sizeof(int32_t) * (size_t)count);
    if (staged_rows_out != nullptr) *staged_rows_out = st->rows;
    return LEGION_OK;
}

extern "C" int legion_runner_staged_rows(LegionRunner *r, int64_t *rows)
{
    LG_ARG(r != nullptr && rows != nullptr, "NULL pointer");
    *rows = r->staged_rows;
    return LEGION_OK;
}

extern "C" int legion_runner_destroy(LegionRunner *r)
{
    if (r == nullptr) return LEGION_OK;
    cudaSetDevice(r->dev_id);
    cudaDeviceSynchronize();
    drop_graphs(r);
    for (auto &pr : r->gather_ev) { cudaEventDestroy(pr.a); cudaEventDestroy(pr.b); }
    for (auto &pr : r->miss_ev) { cudaEventDestroy(pr.a); cudaEventDestroy(pr.b); }
    for (auto &pr : r->sample_ev) { cudaEventDestroy(pr.a); cudaEventDestroy(pr.b); }
    for (auto e : r->ev_free) cudaEventDestroy(e);
    for (int i = 0; i < LEGION_MAX_PIPES; ++i) cudaEventDestroy(r->hit_done[i]);
    for (int i = 0; i < LEGION_MAX_PIPES; ++i) {
        cudaEventDestroy(r->pipe_done[i]);
        cudaStreamDestroy(r->s_launch[i]);
    }
    cudaEventDestroy(r->t_begin);
    cudaEventDestroy(r->t_end);
    cudaStreamDestroy(r->s_sample);
    cudaStreamDestroy(r->s_gather);
    cudaStreamDestroy(r->s_miss);
    cudaStreamDestroy(r->s_copy);
    cudaStreamDestroy(r->s_h2d);
    for (int i = 0; i < LEGION_MAX_PIPES; ++i) { cudaEventDestroy(r->sampled[i]); cudaEventDestroy(r->exported[i]); }
    for (int i = 0; i < LEGION_MAX_PIPES; ++i) { cudaEventDestroy(r->staged_ev[i]); cudaEventDestroy(r->slot_done[i]); cudaFree(r->seed_rows[i]); }
    for (int i = 0; i < 4; ++i) stage_free(&r->stage[i]);
    delete r;
    return LEGION_OK;
}
