// sampling_server: the server binary of the reference (sampling_server/src/main.cu:5-17 ->
// GPUServer::Initialize / PreSc / Run / Finalize, engine/server.cu:46-170) on top of the C ABI.
//
//   sampling_server <ngpu> <cache_agg_mode> <dyn_flags> [fanout ...]
//
// reads ./meta_config (written by legion_server.py:45-46), loads the Legion-format dataset, runs one
// host thread per GPU, builds the caches (presampled hotness order like the reference; set
// LEGION_ORDER=degree for the degree order; with more than one GPU the per-GPU budget is planned into a
// stripe of the clique's cache plus private copies of the hottest peer rows), stages the rows of uncached
// seeds in page-locked memory for the copy engine, rewrites the host table in packed order (uncached rows by
// rising rank; LEGION_HOST_LAYOUT=id keeps the file's order), publishes the hand-off buffers, prints
// "System is ready for serving" (engine/server.cu:121; scripts/wait_file.sh waits for that line) and
// serves every batch of the schedule to the trainers.  cache_agg_mode is accepted and ignored: an
// NVSwitch box is one clique.  dyn_flags: bit 3 (DYN_COMP, comp_cache/cache_helper.cuh:34-45) selects
// int8-compressed cache rows, bit 0 (DYN_ENABLE) the per-GPU LRU cache, 0 the static cache.  The
// fanout defaults to the reference's hard-coded {25, 10} (main.cu:9-11).
#include <pthread.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <thread>
#include <vector>

#include <cuda_runtime.h>

#include "../../include/legion_b200.h"

#define CHECK(call)                                                              \
    do {                                                                         \
        int rc_ = (call);                                                        \
        if (rc_ != LEGION_OK) {                                                  \
            fprintf(stderr, "%s:%d: %s\n", __FILE__, __LINE__, legion_last_error()); \
            exit(EXIT_FAILURE);                                                  \
        }                                                                        \
    } while (0)
#define CUCHECK(call)                                                            \
    do {                                                                         \
        cudaError_t e_ = (call);                                                 \
        if (e_ != cudaSuccess) {                                                 \
            fprintf(stderr, "%s:%d: %s\n", __FILE__, __LINE__, cudaGetErrorString(e_)); \
            exit(EXIT_FAILURE);                                                  \
        }                                                                        \
    } while (0)

struct Rank {
    int dev;
    LegionGraph *graph = nullptr;
    LegionFeatures *feature = nullptr;
    LegionCache *cache = nullptr;
    LegionPool *pool = nullptr;
    LegionRunner *runner = nullptr;
    int64_t *d_indptr = nullptr;
    int32_t *d_indices = nullptr;
    int32_t *d_ids[3] = { nullptr, nullptr, nullptr }, *d_labels[3] = { nullptr, nullptr, nullptr };
    int32_t count[3] = { 0, 0, 0 };
};

static pthread_barrier_t g_barrier;
static pthread_mutex_t g_sum_lock = PTHREAD_MUTEX_INITIALIZER;
static std::vector<uint32_t> g_total_counts;  // presampled access counts of all GPUs, added up

int main(int argc, char **argv)
{
    if (argc < 4) {
        fprintf(stderr, "usage: %s <ngpu> <cache_agg_mode> <dyn_flags> [fanout ...]\n", argv[0]);
        return 1;
    }
    const int ngpu = atoi(argv[1]);
    const int dyn_flags = atoi(argv[3]);
    std::vector<int32_t> fanout;
    for (int i = 4; i < argc; ++i) fanout.push_back(atoi(argv[i]));
    if (fanout.empty()) fanout = { 25, 10 };
    const char *order_env = getenv("LEGION_ORDER");
    const bool degree_order = order_env != nullptr && strcmp(order_env, "degree") == 0;
    const char *shm_env = getenv("LEGION_SHM_NAME");  // tests only; the trainers expect the default
    const char *seed_env = getenv("LEGION_SEED");
    const uint64_t seed = seed_env ? strtoull(seed_env, nullptr, 0) : 0;
    const int timeout_ms = getenv("LEGION_TIMEOUT_MS") ? atoi(getenv("LEGION_TIMEOUT_MS")) : -1;
    const int pipes = (getenv("LEGION_PIPES") && atoi(getenv("LEGION_PIPES")) == 2) ? 2 : LEGION_MAX_PIPES;
    const bool packed_layout = !(getenv("LEGION_HOST_LAYOUT") != nullptr && strcmp(getenv("LEGION_HOST_LAYOUT"), "id") == 0);
    const bool stripe_only = getenv("LEGION_STRIPE_ONLY") != nullptr && getenv("LEGION_STRIPE_ONLY")[0] == '1';
    const bool no_staging = getenv("LEGION_NO_SEED_STAGING") != nullptr && getenv("LEGION_NO_SEED_STAGING")[0] == '1';
    if (ngpu < 1 || ngpu > LEGION_MAX_DEVICE) {
        fprintf(stderr, "ngpu must be 1..%d\n", LEGION_MAX_DEVICE);
        return 1;
    }

    LegionMetaConfig meta;
    CHECK(legion_meta_config_read("./meta_config", &meta));
    printf("Dataset path:       %s\nRaw Batchsize:      %d\nGraph nodes num:    %lld\nGraph edges num:    %lld\n"
           "Feature dim:        %d\nTraining set num:   %d\nValidation set num: %d\nTesting set num:    %d\n"
           "Cache memory:       %lld\nTrain epoch:        %d\n",
           meta.dataset_path, meta.raw_batch_size, (long long)meta.node_num, (long long)meta.edge_num,
           meta.float_feature_len, meta.training_set_num, meta.validation_set_num, meta.testing_set_num,
           (long long)meta.cache_memory, meta.epoch);
    CUCHECK(cudaSetDevice(0));
    LegionDataset *ds = nullptr;
    CHECK(legion_dataset_load(&ds, &meta, 1, 1));
    const int64_t *indptr;
    const int32_t *indices, *labels;
    const float *features;
    CHECK(legion_dataset_arrays(ds, &indptr, &indices, &features, &labels));
    const int64_t n = meta.node_num, e = meta.edge_num;
    const int32_t row_bytes = meta.float_feature_len * 4;

    // IPCEnv + Coordinate (storage_management.cu:303-305, ipc_service.cu:60-128)
    std::vector<Rank> ranks(ngpu);
    std::vector<int32_t> ntrain(ngpu), nvalid(ngpu), ntest(ngpu);
    for (int g = 0; g < ngpu; ++g) {
        ranks[g].dev = g;
        for (int m = 0; m < 3; ++m) CHECK(legion_dataset_split(ds, m, ngpu, g, nullptr, nullptr, &ranks[g].count[m]));
        ntrain[g] = ranks[g].count[0];
        nvalid[g] = ranks[g].count[1] > 0 ? ranks[g].count[1] : 1;
        ntest[g] = ranks[g].count[2] > 0 ? ranks[g].count[2] : 1;
    }
    LegionIpcEnv *env = nullptr;
    CHECK(legion_ipc_create(&env, ngpu, shm_env));
    CHECK(legion_ipc_coordinate(env, ntrain.data(), nvalid.data(), ntest.data(), ngpu, meta.raw_batch_size, meta.epoch));
    int32_t steps[3];
    CHECK(legion_ipc_steps(env, steps));
    printf("Train Steps: %d\nValid Steps: %d\nTest Steps: %d\n", steps[0], steps[1], steps[2]);
    int32_t max_bs = meta.raw_batch_size;
    for (int g = 0; g < ngpu; ++g)
        for (int m = 1; m < 3; ++m) {
            int b = legion_ipc_current_batchsize(env, g, m);
            if (b > max_bs) max_bs = b;
        }
    int64_t cap64 = meta.cache_memory / row_bytes;  // rows per GPU
    if (cap64 > n) cap64 = n;
    const int64_t budget_rows = cap64;
    if (cap64 * ngpu >= n) cap64 = (n + ngpu - 1) / ngpu;
    const int32_t capacity = (int32_t)cap64;
    const int max_step = legion_ipc_max_step(env);
    pthread_barrier_init(&g_barrier, nullptr, ngpu);

    auto worker = [&](int g) {
        Rank &r = ranks[g];
        CUCHECK(cudaSetDevice(g));
        // topology in HBM when it fits next to the cache, else read in place from pinned host memory
        size_t free_b = 0, total_b = 0;
        CUCHECK(cudaMemGetInfo(&free_b, &total_b));
        const size_t topo = 8 * (size_t)(n + 1) + 4 * (size_t)e;
        const int64_t *ip = indptr;
        const int32_t *ix = indices;
        if (topo + (size_t)capacity * row_bytes + ((size_t)8 << 30) < free_b) {
            CUCHECK(cudaMalloc(&r.d_indptr, 8 * (size_t)(n + 1)));
            CUCHECK(cudaMalloc(&r.d_indices, 4 * (size_t)(e > 0 ? e : 1)));
            CUCHECK(cudaMemcpy(r.d_indptr, indptr, 8 * (size_t)(n + 1), cudaMemcpyHostToDevice));
            CUCHECK(cudaMemcpy(r.d_indices, indices, 4 * (size_t)e, cudaMemcpyHostToDevice));
            ip = r.d_indptr;
            ix = r.d_indices;
        }
        CHECK(legion_graph_create(&r.graph, g, n, e, ip, ix));
        CHECK(legion_features_create(&r.feature, g, n, row_bytes, features));
        for (int m = 0; m < 3; ++m) {
            if (r.count[m] <= 0) continue;
            std::vector<int32_t> ids(r.count[m]), lab(r.count[m]);
            int32_t cnt = 0;
            CHECK(legion_dataset_split(ds, m, ngpu, g, ids.data(), lab.data(), &cnt));
            CUCHECK(cudaMalloc(&r.d_ids[m], 4 * (size_t)cnt));
            CUCHECK(cudaMalloc(&r.d_labels[m], 4 * (size_t)cnt));
            CUCHECK(cudaMemcpy(r.d_ids[m], ids.data(), 4 * (size_t)cnt, cudaMemcpyHostToDevice));
            CUCHECK(cudaMemcpy(r.d_labels[m], lab.data(), 4 * (size_t)cnt, cudaMemcpyHostToDevice));
            CHECK(legion_features_set_split(r.feature, m, r.d_ids[m], r.d_labels[m], cnt));
        }
        // two hand-off slots (what the trainers' segment holds); behind a static cache up to four batches are
        // sampled ahead of them into private buffers (LEGION_PIPES=2 samples into the slots like the reference)
        CHECK(legion_pool_create_ahead(&r.pool, g, max_bs, (int32_t)fanout.size(), fanout.data(), row_bytes,
                                       LEGION_INTERBATCH_CON, (dyn_flags & 1) ? LEGION_INTERBATCH_CON : pipes));
        CHECK(legion_pool_set_rng(r.pool, seed + (uint64_t)g, 64));

        // PreSc (engine/server.cu:94-122): rank the nodes, fill the cache
        int32_t *order = nullptr;
        CUCHECK(cudaMalloc(&order, 4 * (size_t)n));
        if (degree_order) {
            const int64_t *ip_dev = r.d_indptr;
            int64_t *tmp_ip = nullptr;
            if (ip_dev == nullptr) {
                CUCHECK(cudaMalloc(&tmp_ip, 8 * (size_t)(n + 1)));
                CUCHECK(cudaMemcpy(tmp_ip, indptr, 8 * (size_t)(n + 1), cudaMemcpyHostToDevice));
                ip_dev = tmp_ip;
            }
            CHECK(legion_cache_degree_order(g, ip_dev, n, order, nullptr));
            if (tmp_ip) cudaFree(tmp_ip);
        } else {
            uint32_t *counts = nullptr;
            CUCHECK(cudaMalloc(&counts, 4 * (size_t)n));
            CUCHECK(cudaMemset(counts, 0, 4 * (size_t)n));
            LegionRunner *pre = nullptr;
            CHECK(legion_runner_create(&pre, g, r.graph, r.feature, nullptr, r.pool, nullptr));
            CHECK(legion_runner_presample(pre, 0, steps[0], counts));
            CHECK(legion_runner_destroy(pre));
            if (ngpu > 1) {
                // The clique shares ONE ranking (rank t lives on GPU t % ngpu for every member), so the access
                // counts of all GPUs are added up before any of them ranks (the reference merges the per-GPU
                // counters of a clique in CandidateSelection, cache/cache.cu:354-447).
                std::vector<uint32_t> mine((size_t)n);
                CUCHECK(cudaMemcpy(mine.data(), counts, 4 * (size_t)n, cudaMemcpyDeviceToHost));
                pthread_mutex_lock(&g_sum_lock);
                if (g_total_counts.empty()) g_total_counts.assign((size_t)n, 0u);
                for (int64_t i = 0; i < n; ++i) g_total_counts[(size_t)i] += mine[(size_t)i];
                pthread_mutex_unlock(&g_sum_lock);
                pthread_barrier_wait(&g_barrier);
                CUCHECK(cudaMemcpy(counts, g_total_counts.data(), 4 * (size_t)n, cudaMemcpyHostToDevice));
            }
            CHECK(legion_cache_hotness_order(g, counts, n, order, nullptr));
            cudaFree(counts);
        }
        if (dyn_flags & 1) {
            int64_t sets = capacity / 8 > 0 ? capacity / 8 : 1;  // 8 ways, cache/cache.cu:628-629
            CHECK(legion_cache_create_lru(&r.cache, g, n, row_bytes, sets, 8));
            CHECK(legion_cache_set_host_table(r.cache, features));
        } else {
            int codec = (dyn_flags & 8) ? LEGION_CODEC_INT8 : LEGION_CODEC_RAW;
            // The per-GPU budget is split into this GPU's stripe of the clique's cache and private copies of
            // the hottest rows that the striping gave to peers (the capacity split of the reference's cost
            // model, cache/cache.cu:449-557, for one process-wide clique); LEGION_STRIPE_ONLY=1 keeps the
            // reference's placement.  Every thread computes the same plan.
            int64_t stripe = capacity, replicas = 0;
            if (ngpu > 1 && !stripe_only) {
                const int64_t *ip_dev = r.d_indptr;
                int64_t *tmp_ip = nullptr;
                if (ip_dev == nullptr) {
                    CUCHECK(cudaMalloc(&tmp_ip, 8 * (size_t)(n + 1)));
                    CUCHECK(cudaMemcpy(tmp_ip, indptr, 8 * (size_t)(n + 1), cudaMemcpyHostToDevice));
                    ip_dev = tmp_ip;
                }
                CHECK(legion_cache_plan(g, order, ip_dev, nullptr, n, budget_rows, ngpu, nullptr, &stripe, &replicas, nullptr));
                if (tmp_ip) cudaFree(tmp_ip);
            }
            CHECK(legion_cache_create(&r.cache, g, n, row_bytes, ngpu, g, (int32_t)stripe, codec));
            // The host table is rewritten once in packed order: uncached rows by rising rank, cached rows last
            // (LEGION_HOST_LAYOUT=id keeps the node-id order of the feature file).  Thread 0 moves the rows, every
            // GPU gets the matching row-of-id array.
            int32_t *row_of = nullptr;
            const float *table = features;
            if (packed_layout) {
                int64_t n_cached = stripe * ngpu < n ? stripe * ngpu : n;
                CUCHECK(cudaMalloc(&row_of, 4 * (size_t)n));
                CHECK(legion_cache_pack_order(g, order, n, n_cached, row_of, nullptr));
                pthread_barrier_wait(&g_barrier);
                if (g == 0) CHECK(legion_dataset_pack_features(ds, g, order, n_cached));
                pthread_barrier_wait(&g_barrier);
                CHECK(legion_dataset_arrays(ds, nullptr, nullptr, &table, nullptr));
            }
            CHECK(legion_cache_fill_static_rows(r.cache, order, n, table, row_of, nullptr));
            if (replicas > 0) CHECK(legion_cache_add_replicas(r.cache, order, n, replicas, row_of, nullptr));
            if (row_of) cudaFree(row_of);
            if (g == 0) printf("Cache rows per GPU: %lld striped + %lld private copies\n", (long long)stripe, (long long)replicas);
        }
        cudaFree(order);
        pthread_barrier_wait(&g_barrier);
        if (!(dyn_flags & 1) && ngpu > 1) {
            for (int k = 0; k < ngpu; ++k) {
                if (k == g) continue;
                CHECK(legion_cache_allow_device(ranks[k].cache, g));
                void *ptr = nullptr;
                int64_t bytes = 0;
                CHECK(legion_cache_partition(ranks[k].cache, &ptr, &bytes));
                CHECK(legion_cache_set_peer(r.cache, k, ptr));
            }
        }
        CHECK(legion_ipc_publish_pool(env, r.pool, g));
        CHECK(legion_runner_create(&r.runner, g, r.graph, r.feature, r.cache, r.pool, env));
        if (!(dyn_flags & 1) && !(dyn_flags & 8) && !no_staging) {
            // rows of the uncached seeds of every list into page-locked memory, in list order: the copy engine
            // then brings each batch's block in while the batch samples
            for (int m = 0; m < 3; ++m) {
                int64_t staged = 0;
                if (r.count[m] > 0) CHECK(legion_runner_stage_seeds(r.runner, m, &staged));
                if (g == 0 && r.count[m] > 0) printf("Seed rows staged in host memory, mode %d: %lld\n", m, (long long)staged);
            }
        }
        pthread_barrier_wait(&g_barrier);
        if (g == 0) {
            printf("System is ready for serving\n");
            fflush(stdout);
        }
        CHECK(legion_runner_serve(r.runner, 0, max_step, timeout_ms));  // GPUServer::Run, engine/server.cu:124-143
        // GPURunner::Finalize (engine/server.cu:402-407): the trainer must have released every slot
        // before the buffers go away
        for (int p = 0; p < LEGION_INTERBATCH_CON; ++p) CHECK(legion_ipc_wait(env, g, p, timeout_ms));
        pthread_barrier_wait(&g_barrier);
        CHECK(legion_runner_destroy(r.runner));
        CHECK(legion_cache_destroy(r.cache));
        CHECK(legion_pool_destroy(r.pool));
        CHECK(legion_features_destroy(r.feature));
        CHECK(legion_graph_destroy(r.graph));
        for (int m = 0; m < 3; ++m) { cudaFree(r.d_ids[m]); cudaFree(r.d_labels[m]); }
        cudaFree(r.d_indptr);
        cudaFree(r.d_indices);
    };
    std::vector<std::thread> threads;
    for (int g = 0; g < ngpu; ++g) threads.emplace_back(worker, g);
    for (auto &t : threads) t.join();
    CHECK(legion_ipc_destroy(env));
    CHECK(legion_dataset_destroy(ds));
    printf("System finalized\n");
    return 0;
}
