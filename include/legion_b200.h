/*
 * legion_b200.h -- C ABI of the B200 sampling-server hot path.
 *
 * Plain pointers and sizes only; no C++ or torch types cross this boundary.  Every entry
 * point names the reference interface it replaces (paths relative to the reference
 * repository root).  All functions return 0 on success or a negative LEGION_E_* code and
 * leave a message for legion_last_error(); nothing here calls exit().  The five operator
 * entry points also exist under the reference's own symbol names (BatchGenerate,
 * RandomSample, FeatureCacheLookup, IOSubmit, IOComplete) in legion_b200_compat.h.
 *
 * Threading: one host thread per device, as in GPURunner (engine/server.cu:330-331).
 * Streams are passed as void* (a cudaStream_t).
 */
#ifndef LEGION_B200_H
#define LEGION_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LEGION_OK 0
#define LEGION_E_ARG (-1)     /* bad argument */
#define LEGION_E_CUDA (-2)    /* a CUDA call failed */
#define LEGION_E_NOMEM (-3)   /* allocation failed */
#define LEGION_E_LIMIT (-4)   /* size above a documented limit */
#define LEGION_E_STATE (-5)   /* call out of order */
#define LEGION_E_SYS (-6)     /* shm / semaphore failure */
#define LEGION_E_TIMEOUT (-7) /* peer did not answer in time */

#define LEGION_MAX_DEVICE 8      /* include/system_config.cuh:50 */
#define LEGION_INTERBATCH_CON 2  /* include/system_config.cuh:47 */
#define LEGION_INTRABATCH_CON 3  /* include/system_config.cuh:48 */
#define LEGION_MAX_PIPES 4       /* batches a pool can hold in flight; the hand-off to trainers uses INTERBATCH_CON of them */
#define LEGION_MEMORY_USAGE 7    /* include/system_config.cuh:51 */
#define LEGION_TRAINMODE 0
#define LEGION_VALIDMODE 1
#define LEGION_TESTMODE 2
#define LEGION_CACHEMISS_FLAG (-2) /* include/system_config.cuh:56 */
#define LEGION_MAX_FANOUT 32       /* engine/operator_impl.cu:504 */
#define LEGION_MAX_HOPS 3          /* counter slots 9+h / 12+h, engine/operator_impl.cu:80-82 */

#define LEGION_CODEC_RAW 0
#define LEGION_CODEC_INT8 1
#define LEGION_CODEC_E4M3 2

typedef struct LegionGraph LegionGraph;       /* GraphStorage,   storage/graph_storage.cuh:7-24 */
typedef struct LegionFeatures LegionFeatures; /* FeatureStorage, storage/feature_storage.cuh:6-34 */
typedef struct LegionCache LegionCache;       /* UnifiedCache,   cache/cache.cuh:66-188 */
typedef struct LegionPool LegionPool;         /* MemoryPool,     engine/memorypool.cuh:20-221 */
typedef struct LegionIpcEnv LegionIpcEnv;     /* IPCEnv,         engine/ipc_service.h:6-35 */
typedef struct LegionRunner LegionRunner;     /* Runner,         engine/server.h:23-34 */

const char *legion_last_error(void);
int legion_abi_version(void);
/* Blocking copy between raw pointers, for callers without a CUDA binding of their own (the
 * reference's alloc/copy helpers, engine/server_imp.cuh:1-51).  kind: 1 host->device,
 * 2 device->host, 3 device->device. */
int legion_copy(void *dst, const void *src, int64_t bytes, int32_t kind);
/* Page-locks a range of host memory that CUDA did not allocate (a shared segment or mapped file that
 * several server processes share) so that this process's kernels can read it by zero-copy loads.  The
 * reference has one process and allocates its host tables with cudaHostAlloc
 * (storage/storage_management.cu:114-115,171). */
int legion_host_register(int32_t dev_id, void *ptr, int64_t bytes);
/* Launch-shape knobs for measurements (the reference hard-codes its grids, e.g. cache/cache.cu:746-752).
 * "miss_ctas": CTAs of the host-link fetch kernel, 0 = one per SM. */
int legion_set_tunable(const char *name, int32_t value);
/* Names: "miss_ctas", "miss_threads", "miss_rows" (launch shape of the host-link fetch and the rows a warp keeps
 * in flight: 1, 2, 4 or 8); "gather_rows_per_warp" (32, 16 or 8 rows looked up and copied per warp and chunk of
 * the 512-byte-class gather); "gather_ctas_per_sm",
 * "gather_rows_in_flight" (2/4/8/16, register path); "gather_engine" 0 = rows move through registers,
 * 1 = rows move by bulk asynchronous copies through shared memory (start value from the environment
 * variable LEGION_GATHER_ENGINE); "pdl" 1 = the sampling kernels of a batch are launched as programmatic
 * dependents of one another (start value from LEGION_PDL; applies to runners created afterwards);
 * "map_front_shift" s: the front region of a pool's id map gets 1 / 2^s of the worst-case slots
 * (-1, the default: an eighth, but at least 2^20 slots where the worst case has that many; pools
 * created afterwards). */

/* EnableP2PAccess (storage/storage_management.cu:9-27) for one ordered pair of devices of this
 * process; needed when the clique's partitions are allocated by threads of one process. */
int legion_enable_peer_access(int32_t dev_id, int32_t peer_id);

/* ---- storage --------------------------------------------------------------------- */

/* NewCompleteGraphStorage + Build (storage/graph_storage.cu:12-74).  indptr/indices must be
 * readable from device dev_id: device memory or mapped pinned host memory (UVA), as the
 * reference keeps them (storage/storage_management.cu:114-115).  Not owned. */
int legion_graph_create(LegionGraph **out, int32_t dev_id, int64_t n_nodes, int64_t n_edges,
                        const int64_t *indptr, const int32_t *indices);
int legion_graph_destroy(LegionGraph *g);

/* NewCompleteFeatureStorage + Build (storage/feature_storage.cu:18-90).  host_table is the
 * full feature table in mapped pinned host memory (row i at i*row_bytes), or NULL when every
 * row is cached.  row_bytes = feature_len * element size; rows are opaque bytes. */
int legion_features_create(LegionFeatures **out, int32_t dev_id, int64_t n_nodes, int32_t row_bytes,
                           const void *host_table);
/* This GPU's seed list of one mode (GetTrainingSetIds/Labels..., feature_storage.cuh:12-29):
 * device arrays of `count` int32, not owned. */
int legion_features_set_split(LegionFeatures *f, int32_t mode, const int32_t *ids_dev,
                              const int32_t *labels_dev, int32_t count);
int legion_features_destroy(LegionFeatures *f);

/* ---- Legion-format datasets (storage/storage_management.cu:33-279) -------------------- */

/* The single line of ./meta_config in in-memory mode, written by legion_server.py:45-46 and parsed by
 * StorageManagement::ReadMetaFIle (storage/storage_management.cu:33-68). */
typedef struct LegionMetaConfig {
    char dataset_path[512];
    char feature_path[512];   /* same as dataset_path when the line has no 11th field */
    int32_t raw_batch_size;
    int64_t node_num, edge_num;
    int32_t float_feature_len;
    int32_t training_set_num, validation_set_num, testing_set_num;
    int64_t cache_memory;     /* bytes per GPU */
    int32_t epoch;
} LegionMetaConfig;
typedef struct LegionDataset LegionDataset;
int legion_meta_config_read(const char *file, LegionMetaConfig *out);
int legion_meta_config_write(const char *file, const LegionMetaConfig *m);
/* LoadGraph + LoadFeature (storage/storage_management.cu:106-279, storage_management_impl.cuh:48-196):
 * reads edge_src (int64 offsets), edge_dst (int32), features (fp32), labels, trainingset /
 * validationset / testingset and the optional partition file.  pin != 0 puts topology and features
 * in mapped pinned host memory (needs a GPU), pin == 0 in plain host memory. */
int legion_dataset_load(LegionDataset **out, const LegionMetaConfig *meta, int32_t pin, int32_t load_features);
int legion_dataset_arrays(LegionDataset *d, const int64_t **indptr, const int32_t **indices, const float **features,
                          const int32_t **labels);
/* Seeds of one GPU (storage/storage_management.cu:214-250): partition file for the training set when
 * present, else id % partition_count.  ids_out == NULL returns the count only. */
int legion_dataset_split(LegionDataset *d, int32_t mode, int32_t partition_count, int32_t part_id, int32_t *ids_out,
                         int32_t *labels_out, int32_t *count_out);
/* Host table packed by rank.  The reference keeps the table in node-id order (cache/cache_impl.cuh:283-286,
 * storage/storage_management.cu:160-175); random zero-copy reads of widely scattered host pages are slow on this
 * platform, and the better a node's rank, the more often its row is asked for.  Packed order: the rows of the
 * nodes that the clique's caches do not hold (rank >= n_cached) by rising rank, then the rows of the cached
 * nodes.  legion_dataset_pack_features rewrites the loaded table in that order (a second page-locked copy exists
 * while it runs; legion_dataset_arrays returns the new table afterwards); legion_cache_pack_order gives every
 * GPU the matching row_of_id array for legion_cache_fill_static_rows / legion_cache_add_replicas. */
int legion_dataset_pack_features(LegionDataset *d, int32_t dev_id, const int32_t *order_dev, int64_t n_cached);
int legion_cache_pack_order(int32_t dev_id, const int32_t *order_dev, int64_t n_nodes, int64_t n_cached,
                            int32_t *row_of_dev, void *stream);
int legion_dataset_destroy(LegionDataset *d);

/* ---- cache ----------------------------------------------------------------------- */

/* UnifiedCache::Initialize + the allocation half of FillUp (cache/cache.cu:559-600).
 * Static cache striped over a clique of kg GPUs, this GPU being member ki; `capacity` rows
 * per GPU.  codec RAW keeps rows as they are; INT8 / E4M3 keep feature_len codes plus one
 * fp32 scale per row (row_bytes must then be feature_len*4).  Allocates the lookup table
 * (one int32 per node) and this GPU's partition. */
int legion_cache_create(LegionCache **out, int32_t dev_id, int64_t n_nodes, int32_t row_bytes,
                        int32_t kg, int32_t ki, int32_t capacity, int32_t codec);
/* Descending-degree order of all nodes, ties by ascending id; the ranking that
 * CandidateSelection produces from presampled hotness (cache/cache.cu:405-440), with degree as
 * the key.  order_dev: n_nodes int32 in device memory. */
int legion_cache_degree_order(int32_t dev_id, const int64_t *indptr, int64_t n_nodes,
                              int32_t *order_dev, void *stream);
/* The reference's own ranking: nodes by descending presampled hotness (CandidateSelection,
 * cache/cache.cu:354-447), ties by ascending id.  counts_dev: one uint32 per node, filled by
 * legion_runner_presample (HotnessMeasure, cache/cache_impl.cuh:190-198). */
int legion_cache_hotness_order(int32_t dev_id, const uint32_t *counts_dev, int64_t n_nodes, int32_t *order_dev,
                               void *stream);
/* InitPair + Insert + FeatFillUp (cache/cache_impl.cuh:104-109,183-188; cache/cache.cu:74-141):
 * rank t of `order` lives on GPU t % kg at row t / kg.  Builds the whole lookup table and copies
 * (and encodes) this GPU's rows from host_table. */
int legion_cache_fill_static(LegionCache *c, const int32_t *order_dev, int64_t n_order,
                             const void *host_table, void *stream);
/* Same for a host table that is NOT laid out in node-id order: row_of_id_dev[id] (device, one int32
 * per node) is the row of the table that holds node id.  The reference keeps the table in id order
 * (cpu_float_features[id * F], cache/cache_impl.cuh:283-286); on this platform random zero-copy
 * reads are limited by address translation of widely scattered host pages (50 GB/s inside 1 GB,
 * 26 GB/s across 48 GB), so a loader may pack the rows it expects to miss most (seed nodes, then
 * nodes by falling degree) next to each other.  The lookup table then remembers the row of every
 * uncached node. */
int legion_cache_fill_static_rows(LegionCache *c, const int32_t *order_dev, int64_t n_order, const void *host_table,
                                  const int32_t *row_of_id_dev, void *stream);
/* Placement without fill (InitPair + table insert, cache/cache_impl.cuh:104-109, cache/cache.cu:74-112,
 * without FeatFillUp): builds the lookup table for `order` and leaves the rows to the caller, who writes
 * row s of this GPU's partition (legion_cache_partition) with the row of node order[s * kg + ki].  For a
 * table that exists nowhere as a whole: the MAG240M-shaped configuration spreads 375 GB over eight
 * caches, each GPU loading (or generating) only its own stripe.  Uncompressed caches only; without a host
 * table every node outside the clique's caches is a miss that nothing serves. */
int legion_cache_place_static(LegionCache *c, const int32_t *order_dev, int64_t n_order, void *stream);
/* Host table stored compressed ("IBP(M)" of the reference: compress_cpu_transfer_kernel,
 * comp_cache/static_cache.cu:656-772, with the int8 / e4m3 per-row codec in place of the absent
 * bit-packing): every row of the host table is feature_len one-byte codes + one fp32 scale, padded to
 * 16 bytes, exactly a cache slot.  A miss then moves that many bytes over the host link and is decoded
 * in the fetch kernel; cache fill copies slots.  Hits and misses decode to the same values.  Call on a
 * cache of the same codec before legion_cache_fill_static[_rows]. */
int legion_cache_set_host_codec(LegionCache *c, int32_t codec);
/* Encodes n_rows fp32 rows (device-accessible: device or pinned host memory) into compressed rows of
 * (feature_len + 4) bytes rounded up to 16, with the quantiser the caches use. */
int legion_quantize_table(int32_t dev_id, int32_t codec, const void *rows, int64_t n_rows, int32_t feature_len,
                          void *out_rows, void *stream);
/* The capacity split of the reference's cost model (CandidateSelection / CostModel, cache/cache.cu:354-557)
 * for a clique of one process per GPU: how many rows of a per-GPU budget go to this GPU's stripe of
 * the clique's cache and how many to private copies of hot rows held by peers.  Node weights in rank
 * order come from the degrees (indptr_dev) or from presampled access counts (counts_dev; one of the two
 * may be NULL); cost_local_peer_host gives the relative cost of a row served locally / by a peer / by
 * the host table (NULL: 0.16, 1, 15 as measured on B200).  Every rank computes the same plan. */
int legion_cache_plan(int32_t dev_id, const int32_t *order_dev, const int64_t *indptr_dev, const uint32_t *counts_dev,
                      int64_t n_nodes, int64_t budget_rows, int32_t world, const double cost_local_peer_host[3],
                      int64_t *stripe_rows, int64_t *replica_rows, void *stream);
/* Private copies of the hottest rows that the striping gave to OTHER clique members, so that this
 * GPU serves them from its own memory instead of over NVLink.  The reference stripes only
 * (cache/cache_impl.cuh:104-109): when the clique's budget exceeds the table (8 GPUs x 20%), its
 * spare memory stays empty and 7 of 8 hits cross NVLink.  Call after legion_cache_fill_static[_rows]
 * with the same order (and row_of_id_dev, or NULL): replica row s holds the s-th rank t with
 * t % kg != ki.  n_rows <= capacity; ranks that the striping did not place are not replicated.  The
 * lookup table names a replica as member `kg` of the clique; peers never see it.  Gathered rows do not
 * change, only where they are read from.  A refill drops the replicas. */
int legion_cache_add_replicas(LegionCache *c, const int32_t *order_dev, int64_t n_order, int64_t n_rows,
                              const int32_t *row_of_id_dev, void *stream);
/* Pointer tables of the clique (d_float_feature_cache_ptr_, cache/cache.cu:601-622). */
int legion_cache_partition(LegionCache *c, void **ptr, int64_t *bytes);
int legion_cache_set_peer(LegionCache *c, int32_t k, const void *partition_ptr);
/* The lookup table of a cache of uncompressed rows without replicas (LEGION_E_ARG otherwise: such tables
 * only make sense together with the cache's own slot size and replica region). */
int legion_cache_lut(LegionCache *c, int32_t **lut_dev);
/* The same pointer table across processes (one process per GPU).  With kg > 1 the partition is
 * allocated as shareable memory: export it as a POSIX file descriptor (pass it to the peers over a
 * unix socket with SCM_RIGHTS, then close it), and map member k's partition from the descriptor
 * its process sent.  Peers are then read by plain loads over NVLink.  LEGION_E_STATE when the
 * partition is ordinary cudaMalloc memory; legion_ipc_get_handle / legion_ipc_open_handle +
 * legion_cache_set_peer remain as the fallback. */
int legion_cache_export_partition(LegionCache *c, int32_t *fd_out, int64_t *bytes_out);
int legion_cache_import_peer(LegionCache *c, int32_t k, int32_t fd, int64_t bytes);
/* One process with a thread per GPU, as the reference runs (engine/server.cu:127-135): give device
 * `dev` read access to this cache's partition, whose pointer the other thread then hands to
 * legion_cache_set_peer. */
int legion_cache_allow_device(LegionCache *c, int32_t dev);
/* Table that serves the misses (cpu_float_features_, cache/cache.cu:771-776); set by
 * legion_cache_fill_static, or here for a cache that is filled some other way. */
int legion_cache_set_host_table(LegionCache *c, const void *host_table);
/* Per-GPU set-associative cache with LRU replacement: sets*ways rows.  Addressing follows
 * comp_cache/static_cache_kernel.cuh:6-29; lookup = retrieve_and_touch, the insertion of missed
 * rows runs in legion_io_complete (comp_cache/tests/test_cache.cu:57-58 names the calls). */
int legion_cache_create_lru(LegionCache **out, int32_t dev_id, int64_t n_nodes, int32_t row_bytes,
                            int64_t sets, int32_t ways);
int legion_cache_lru_state(LegionCache *c, int32_t **keys_dev, int32_t **stamps_dev, void **rows_dev);
/* Batch clock used for the stamps: 1 at creation, +1 at every legion_io_complete. */
int legion_cache_lru_clock(LegionCache *c, int32_t *clock);
/* counters since creation: [0] local hits, [1] peer hits, [2] misses, [3] lru inserts */
int legion_cache_stats(LegionCache *c, int64_t stats[4], void *stream);
int legion_cache_destroy(LegionCache *c);

/* ---- memory pool ------------------------------------------------------------------- */

/* MemoryPool + GPURunner::Initialize buffer allocation + IPCEnv::Initialize{Samples,Features}Buffer
 * (engine/server.cu:204-265, engine/ipc_service.cu:134-206).  Buffers are sized for the true
 * worst case of the fanout list.  `pipes` output sets: INTERBATCH_CON (2) for a pool that is published to
 * trainers, up to LEGION_MAX_PIPES for a consumer inside the process (more batches in flight hide more of
 * the sampling kernels' latency).  row_bytes_out is the size of one gathered row. */
int legion_pool_create(LegionPool **out, int32_t dev_id, int32_t batch_size, int32_t hop_num,
                       const int32_t *fanout, int32_t row_bytes_out, int32_t pipes);
/* A pool that samples AHEAD of the hand-off: `slots` (<= 2 when it is published to trainers) sets of the seven
 * hand-off buffers, and `pipes` (a multiple of slots, <= LEGION_MAX_PIPES) sets of sampling buffers and scratch.
 * Batches are sampled into private buffers while the consumer still holds the slots; when a batch's slot
 * (pipe % slots) is free its block structure is copied in (~3 MB) and its rows are gathered into the slot's
 * feature buffer.  The reference samples into the hand-off buffers themselves (engine/server.cu:237-265,
 * engine/ipc_service.cu:134-206), so it can only overlap INTERBATCH_CON batches.  For legion_runner_enqueue /
 * run_once / serve; the per-operator entry points and the host-buffer calls need slots == pipes.
 * legion_pool_buffer numbers the seven hand-off buffers by slot. */
int legion_pool_create_ahead(LegionPool **out, int32_t dev_id, int32_t batch_size, int32_t hop_num,
                             const int32_t *fanout, int32_t row_bytes_out, int32_t slots, int32_t pipes);
int legion_pool_destroy(LegionPool *p);
#define LEGION_BUF_IDS 0          /* slot order of engine/ipc_service.cu:163-169 */
#define LEGION_BUF_FEATURES 1
#define LEGION_BUF_LABELS 2
#define LEGION_BUF_AGG_SRC 3
#define LEGION_BUF_AGG_DST 4
#define LEGION_BUF_NODE_COUNTER 5
#define LEGION_BUF_EDGE_COUNTER 6
#define LEGION_BUF_CACHE_INDEX 7  /* cache_search_buffer, engine/server.cu:238 (scratch, one per pipe here) */
#define LEGION_BUF_SRC_GLOBAL 8   /* agg_src_ids, engine/server.cu:244 (scratch, one per pipe here) */
int legion_pool_buffer(LegionPool *p, int32_t which, int32_t pipe, void **ptr, int64_t *bytes);
int legion_pool_limits(LegionPool *p, int64_t *max_nodes, int64_t *max_edges);
/* SetIter / SetCurrentMode / SetCurrentPipe (engine/memorypool.cuh) plus the number of the batch
 * in the whole run, which seeds the sampler's counter RNG. */
int legion_pool_set_batch(LegionPool *p, int32_t iter, int32_t mode, int32_t pipe, uint32_t global_batch);
int legion_pool_set_rng(LegionPool *p, uint64_t seed, int32_t max_rounds);
/* First error raised on the device since the last reset (the reference prints and exits,
 * engine/operator_impl.cu:17-25): 0 none, 1 id map full, 2 edge buffer overflow, 3 node buffer
 * overflow, 4 a bulk copy of the gather timed out (the pipe's output is invalid; stop issuing on it);
 * 5 a seed id (or a neighbour id stored in the topology) outside [0, n_nodes) was met: such an id is
 * never used as an index, its slot in the batch reads -1 like a slot past the end of the seed list
 * (engine/operator_impl.cu:41-43), and the rest of the batch is complete.  Synchronises `stream`. */
int legion_pool_device_error(LegionPool *p, void *stream, int32_t *err, int32_t reset);

/* ---- the five operators (engine/operator_impl.cuh:11-69) ---------------------------- */

/* BatchGenerate, engine/operator_impl.cu:93-175 (same argument order; `counter` is the batch
 * number within the mode's seed list). */
int legion_batch_generate(void *stream, LegionFeatures *feature, LegionCache *cache, LegionPool *pool,
                          int32_t batch_size, int32_t counter, int32_t part_id, int32_t dev_id,
                          int32_t mode, int32_t is_presc, int32_t hop_num, int32_t dyn_cache);
/* RandomSample, engine/operator_impl.cu:439-553: one hop (op_id = 3, 6, 9) of sampling,
 * dedup, relabel and counter bookkeeping; `count` is the fanout. */
int legion_random_sample(void *stream, LegionGraph *graph, LegionCache *cache, LegionPool *pool,
                         int32_t count, int32_t dev_id, int32_t op_id, int32_t is_presc, int32_t dyn_cache);
/* FeatureCacheLookup, engine/operator_impl.cu:555-575: cache lookup + feature gather of the
 * current node segment (op_id = 1, 4, 7, 10). */
int legion_feature_cache_lookup(void *stream, LegionCache *cache, LegionPool *pool, int32_t op_id,
                                int32_t dev_id, int32_t dyn_cache);
/* IOSubmit, engine/operator_impl.cu:577-595: a no-op in the reference, kept for the op list. */
int legion_io_submit(void *stream, LegionFeatures *feature, LegionPool *pool, int32_t op_id, int32_t dev_id);
/* IOComplete, engine/operator_impl.cu:606-636: end-of-batch maintenance (the reference clears
 * position_map; here the LRU insertion phase runs). */
int legion_io_complete(void *stream, LegionCache *cache, LegionPool *pool, int32_t dev_id, int32_t mode);

/* Lookup + gather of one id list without any allocation.  No counterpart in the reference (there
 * FeatureCacheLookup always works on a MemoryPool that was allocated beforehand).
 *
 * For callers that must not allocate device memory at the moment they call in: a trainer-side
 * process whose framework allocator already owns the GPU's memory, or a serving loop that cannot
 * take the device-wide synchronisation, the fragmentation or the failure of a cudaMalloc in the
 * middle of a step.  The caller passes inputs and output only; the scratch the gather needs (hit /
 * miss index per row, the list of missed rows, its counters) lives in a fixed array inside the
 * library image, so every GPU that loads the library holds about 3 MB for it until the process
 * exits.  This call, and everything it calls, performs no cudaMalloc / cudaFree.
 *
 *   dev_id       the GPU to run on; the call makes it the calling thread's current device
 *                (cudaSetDevice) and leaves it so
 *   ids_dev      n_rows int32 node ids on the device (ids outside [0, n_nodes) leave their output
 *                row untouched)
 *   lut_dev      one int32 per node: gpu*capacity + row for a cached node, LEGION_CACHEMISS_FLAG
 *                otherwise (legion_cache_lut); NULL = nothing is cached.  capacity, kg and
 *                partitions must be the ones the table was built for; an entry that names a member
 *                >= kg or a NULL partition is served from host_table like a miss
 *   partitions   host array of kg device pointers, the clique's cache partitions (uncompressed rows)
 *   host_table   pinned host table that serves the misses, or NULL (missed rows stay untouched)
 *   out_dev      n_rows * row_bytes bytes on the device, rows in the order of ids_dev
 *
 * Limits and rules: n_rows <= LEGION_NOALLOC_MAX_ROWS (LEGION_E_LIMIT with a message otherwise;
 * split the list or use a LegionPool); rows are multiples of 4 bytes.  The first call on a device
 * looks up the device address of the built-in array; make that first call before starting any
 * stream capture.  All calls share the one array: calls whose kernels overlap on the same GPU
 * (different streams, different threads) race on it, so keep them on one stream or order them with
 * events.  The array keeps the previous call's contents; the call resets what has to start from zero. */
#define LEGION_NOALLOC_MAX_ROWS (1 << 18)
int legion_gather_rows_noalloc(void *stream, int32_t dev_id, const int32_t *ids_dev, int64_t n_rows,
                               const int32_t *lut_dev, int32_t capacity, int32_t kg, int32_t ki,
                               const void *const *partitions, const void *host_table, int64_t n_nodes,
                               int32_t row_bytes, void *out_dev);

/* ---- whole batch --------------------------------------------------------------------- */

/* The op list of GPURunner::RunOnce (engine/server.cu:342-351) for one batch on one stream set.
 * Seeds come from the mode's device-resident seed list. */
int legion_run_batch(void *stream, LegionGraph *graph, LegionFeatures *feature, LegionCache *cache,
                     LegionPool *pool, int32_t dev_id);
/* Same batch with HOST buffers: seeds and labels are copied in from host memory, and the block
 * structure (ids, labels, edge lists, both counters) is copied back; `features_out` may be NULL,
 * in which case gathered rows stay in the pool's feature buffer on the device, where the trainer
 * reads them (training_backend/ipc_cuda_kernel.cu:205-211).  Blocks until done. */
int legion_run_batch_host(LegionGraph *graph, LegionFeatures *feature, LegionCache *cache, LegionPool *pool,
                          int32_t dev_id, const int32_t *seeds, const int32_t *labels, int32_t n_seeds,
                          int32_t *ids_out, int32_t *labels_out, int32_t *agg_src_out, int32_t *agg_dst_out,
                          int32_t node_counter_out[16], int32_t edge_counter_out[16], void *features_out);

/* ---- server <-> trainer hand-off (engine/ipc_service.h:6-35) --------------------------- */

/* NewIPCEnv (engine/ipc_service.cu:35-58): creates and zero-fills the POSIX shared segment
 * "simpleIPCshm" (steps[3] + cudaIpcMemHandle_t[8][2][7]).  shm_name NULL = that default. */
int legion_ipc_create(LegionIpcEnv **out, int32_t device_count, const char *shm_name);
/* Coordinate (engine/ipc_service.cu:60-128): step counts and per-device batch sizes. */
int legion_ipc_coordinate(LegionIpcEnv *e, const int32_t *train_num, const int32_t *valid_num,
                          const int32_t *test_num, int32_t partition_count, int32_t raw_batch_size,
                          int32_t epochs);
int legion_ipc_steps(LegionIpcEnv *e, int32_t steps[3]);
int legion_ipc_max_step(LegionIpcEnv *e);                                           /* GetMaxStep */
int legion_ipc_current_mode(LegionIpcEnv *e, int32_t global_batch_id);               /* GetCurrentMode */
int legion_ipc_local_batch_id(LegionIpcEnv *e, int32_t global_batch_id);             /* GetLocalBatchId */
int legion_ipc_current_batchsize(LegionIpcEnv *e, int32_t dev_id, int32_t mode);     /* GetCurrentBatchsize */
/* InitializeSamplesBuffer + InitializeFeaturesBuffer (engine/ipc_service.cu:134-206): publishes
 * the pool's output buffers as CUDA IPC handles and opens sem_r_<dev>_<pipe> / sem_w_<dev>_<pipe>. */
int legion_ipc_publish_pool(LegionIpcEnv *e, LegionPool *pool, int32_t dev_id);
/* Same, for a process without a GPU (tests): opens the semaphores only. */
int legion_ipc_open_semaphores(LegionIpcEnv *e, int32_t dev_id, int32_t pipes);
/* IPCWait / IPCPost (engine/ipc_service.cu:283-291).  timeout_ms < 0 blocks for ever like the
 * reference; otherwise LEGION_E_TIMEOUT is returned when the trainer does not answer. */
int legion_ipc_wait(LegionIpcEnv *e, int32_t dev_id, int32_t pipe, int32_t timeout_ms);
int legion_ipc_post(LegionIpcEnv *e, int32_t dev_id, int32_t pipe);
/* Counter words of the batch just finished on (dev, pipe), written to the companion host segment
 * "<segment name>_ctr" (int32 [8][2][32]: node_counter then edge_counter) before the batch is posted.
 * The reference's trainer reads both arrays from the device with two blocking copies per batch
 * (training_backend/ipc_cuda_kernel.cu:194-203); a consumer that knows the segment (legion_client_*)
 * reads them from host memory instead, one that does not is unaffected.  The runner calls this itself. */
int legion_ipc_publish_counters(LegionIpcEnv *e, int32_t dev_id, int32_t pipe, const int32_t *node_counter,
                                const int32_t *edge_counter);
/* Finalize (engine/ipc_service.cu:293-320): closes and unlinks semaphores and the segment. */
int legion_ipc_destroy(LegionIpcEnv *e);
/* Byte layout of the shared segment, for consumers written in other languages. */
int legion_ipc_layout(int64_t *segment_bytes, int64_t *handle_bytes, int64_t *handles_offset);
/* Trainer side of one buffer (GPUIPCEnv::Initialize / Finalize, training_backend/ipc_cuda_kernel.cu:62-68,
 * 143-149): map / unmap a 64-byte handle taken from the segment.  Must run in another process than
 * the one that published the buffer. */
int legion_ipc_open_handle(const void *handle_bytes, void **dev_ptr);
/* Handle of one cudaMalloc allocation (cudaIpcGetMemHandle, engine/ipc_service.cu:163-169); also used
 * to share cache partitions between one-process-per-GPU ranks. */
int legion_ipc_get_handle(const void *dev_ptr, void *handle_bytes_out);
int legion_ipc_close_handle(void *dev_ptr);

/* ---- trainer side of the hand-off (training_backend/ipc_service.cpp:30-100) ---------------- */

/* One batch as the trainer sees it (cuda_get_next, training_backend/ipc_cuda_kernel.cu:177-243, and
 * get_block_size, ipc_service.cpp:61-79).  Pointers are device pointers into the server's buffers,
 * valid until legion_client_synchronize.  Hop entries are ordered last hop first. */
typedef struct LegionBatchView {
    int32_t hop_num;
    int32_t n_ids;      /* rows of ids and of features */
    int32_t n_labels;   /* seeds */
    const int32_t *ids;
    const void *features;
    const int32_t *labels;
    const int32_t *agg_src[LEGION_MAX_HOPS];
    const int32_t *agg_dst[LEGION_MAX_HOPS];
    int32_t n_edges[LEGION_MAX_HOPS];
    int32_t block_src[LEGION_MAX_HOPS];  /* num_src of the DGL block */
    int32_t block_dst[LEGION_MAX_HOPS];  /* num_dst of the DGL block */
    int32_t node_counter[16];
    int32_t edge_counter[16];
} LegionBatchView;
typedef struct LegionClient LegionClient;
/* initialize (GPUIPCEnv::Initialize, ipc_cuda_kernel.cu:37-95): maps the segment, opens the 7 buffers
 * of both pipes of device slot dev_id, opens the semaphores and marks both slots free. */
int legion_client_open(LegionClient **out, int32_t dev_id, const char *shm_name);
int legion_client_steps(LegionClient *c, int32_t steps[3]);                                   /* get_steps */
int legion_client_get_next(LegionClient *c, int32_t timeout_ms, LegionBatchView *out);       /* get_next */
/* 1 when legion_client_get_next takes the counters from the server's host segment, 0 when it reads
 * them from the device buffers (a server without the segment). */
int legion_client_counters_on_host(LegionClient *c);
int legion_client_synchronize(LegionClient *c);                                              /* synchronize */
int legion_client_close(LegionClient *c);                                                    /* finalize */

/* ---- runner (engine/server.h:23-34, engine/server.cu:176-416) ---------------------------- */

/* GPURunner::Initialize: binds storage, cache, pool and (optionally) an IPC environment. */
int legion_runner_create(LegionRunner **out, int32_t dev_id, LegionGraph *graph, LegionFeatures *feature,
                         LegionCache *cache, LegionPool *pool, LegionIpcEnv *env);
/* GPURunner::RunOnce: wait for a free slot, run batch `global_batch_id`, post it, rotate the pipe.
 * Without an IPC environment the slot is considered free at once. */
int legion_runner_run_once(LegionRunner *r, int32_t global_batch_id, int32_t mode, int32_t local_batch_id,
                           int32_t timeout_ms);
/* Enqueue without waiting for completion (keeps INTERBATCH_CON batches in flight);
 * legion_runner_sync waits for everything enqueued. */
int legion_runner_enqueue(LegionRunner *r, int32_t global_batch_id, int32_t mode, int32_t local_batch_id);
int legion_runner_sync(LegionRunner *r);
/* The batch interface with HOST buffers and batches in flight: submit copies `n_seeds` seeds and
 * labels in from host memory and starts the batch; collect waits for the oldest submitted batch and
 * copies ids, labels, both edge lists and both counter arrays out (features_out may be NULL: the
 * gathered rows then stay in the device hand-off buffer, where the trainer reads them,
 * training_backend/ipc_cuda_kernel.cu:205-211).  At most `pipes` batches may be in flight;
 * LEGION_E_STATE otherwise.  Pinned output buffers make the copies asynchronous. */
int legion_runner_submit_host(LegionRunner *r, const int32_t *seeds, const int32_t *labels, int32_t n_seeds,
                              int32_t global_batch_id);
/* submit with the output buffers named up front: ids, labels and both edge lists of the batch are
 * copied into these page-locked host buffers (cudaHostAlloc / cudaHostRegister, 16-byte aligned, sized
 * for the pool's limits; NULL skips one) as soon as the batch's sampling is over and while its rows are
 * still being gathered.  The sizes are only on the device at that point, so the copies are issued with
 * the size of the largest batch seen so far plus 1/64 (elements past the batch's own counts are
 * scratch), and whatever a larger batch leaves behind is moved when it is collected.  The matching
 * legion_runner_collect_host only waits and returns the counters (its array arguments are ignored), so
 * the host never sits between "sizes known" and "copy issued".  The buffers belong to the batch until
 * that collect returns.
 * One batch more than the pool has pipes may be submitted this way (static caches): it samples and
 * exports at once, behind the export of the uncollected batch that holds its pipe, and gathers as soon
 * as that batch has been collected and the caller comes back: the rows of a collected batch stay in
 * the pipe's feature buffer until the next call on this runner.  The batches in flight then need
 * pipes + 1 sets of output arrays. */
int legion_runner_submit_host_to(LegionRunner *r, const int32_t *seeds, const int32_t *labels, int32_t n_seeds,
                                 int32_t global_batch_id, int32_t *ids_out, int32_t *labels_out, int32_t *agg_src_out,
                                 int32_t *agg_dst_out);
int legion_runner_collect_host(LegionRunner *r, int32_t *ids_out, int32_t *labels_out, int32_t *agg_src_out,
                               int32_t *agg_dst_out, int32_t node_counter_out[16], int32_t edge_counter_out[16],
                               void *features_out);
/* on = 1: the host-buffer calls of this runner deliver, in the place of agg_dst, the number of edges sampled
 * for every destination, one byte each (fanout <= 32): for hop 0 the counts of the batch's seeds 0 .. n0-1,
 * behind them for hop 1 the counts of all nodes known when hop 1 began (node_counter[9 + 1] of them), and so on;
 * sum over h < hops of node_counter[9 + h] bytes in all.  Within a hop the destinations of the edge list are
 * non-decreasing (engine/operator_impl.cu:178-301 appends the edges node by node here, in node order), so
 * agg_dst of hop h is destination d repeated count[d] times and a CSC block (what
 * training_backend/ipc_cuda_kernel.cu:194-240 hands to the model) needs only the running sum of the counts.
 * The array passed as agg_dst_out is then written as bytes; it needs hops x max_nodes of them at most.  About a
 * third of a batch's block structure no longer crosses the host link.  No counterpart in the reference; default
 * off; call with no batch in flight (LEGION_E_STATE otherwise). */
int legion_runner_set_edge_counts(LegionRunner *r, int32_t on);
/* Host time spent inside submit / collect since the last call of this function (microseconds): out[0]
 * submit, out[1] collect, out[2] the part of collect spent waiting for the device, out[3] batches submitted
 * (the per-op times of the reference's MONITOR build, engine/server.cu:346-395, for the host side). */
int legion_runner_host_times(LegionRunner *r, double out[4]);
int legion_runner_current_pipe(LegionRunner *r);
/* The presampling epoch (GPUServer::PreSc / GPURunner::RunPreSc, engine/server.cu:94-122,313-328): samples
 * training batches [first_batch, first_batch+count) without lookup or gather and counts every node they
 * touch in counts_dev (uint32 per node, zeroed by the caller). */
int legion_runner_presample(LegionRunner *r, int32_t first_batch, int32_t count, uint32_t *counts_dev);
/* Seed-row staging.  No counterpart in the reference, whose every missed row is read by zero-copy loads
 * inside the gather kernel (cache/cache_impl.cuh:283-286).  On B200 a kernel that reads pinned host memory
 * slows the HBM-bound kernels beside it by 2.4-3.6x while it runs, a copy-engine transfer does not; and
 * seeds (random training nodes) are more than half of the rows that miss a degree-ordered cache.  The seed
 * list of a mode is fixed for the run (engine/operator_impl.cu:28-56 slices it batch by batch), so the rows
 * of its uncached nodes are copied once into a page-locked array in list order; the uncached seeds of one
 * batch are then one contiguous block that the copy engine brings to the device while the batch samples,
 * and the gather reads them from device memory.  Rows of sampled neighbours that miss keep the zero-copy
 * path.  Static caches of uncompressed rows with a host table only (LEGION_E_ARG otherwise); call after the
 * cache is filled (and replicas added): a later refill switches the staging off until it is rebuilt.
 * Gathered rows do not change.  staged_rows_out (may be NULL): rows held in the page-locked array.
 *   legion_runner_stage_seeds          the device-resident list of `mode` (batches of legion_runner_enqueue /
 *                                      run_once / serve)
 *   legion_runner_register_host_seeds  a list in the caller's host memory: a later legion_runner_submit_host[_to]
 *                                      whose `seeds` pointer is a slice of [seeds_host, seeds_host + count) and
 *                                      still holds what the list held now is recognised by address and staged;
 *                                      any other batch takes the zero-copy path as before
 *   legion_runner_staged_rows          rows that reached the device this way since the runner was created */
int legion_runner_stage_seeds(LegionRunner *r, int32_t mode, int64_t *staged_rows_out);
int legion_runner_register_host_seeds(LegionRunner *r, const int32_t *seeds_host, int32_t count, int64_t *staged_rows_out);
int legion_runner_staged_rows(LegionRunner *r, int64_t *rows);
/* use_graph (default 1): replay every batch as one CUDA graph per pipe instead of ~25 launches and
 * ~20 event calls from the host.  time_kernels (default 0): bracket the gather launches with CUDA
 * events on the streams they run on.  Call between batches; waits for the device. */
int legion_runner_set_options(LegionRunner *r, int32_t use_graph, int32_t time_kernels);
/* Device time of the batches enqueued between the last two legion_runner_sync calls, measured
 * with CUDA events (ms).  With time_kernels: gather_ms is the sum over the launches that gather
 * cached rows (HBM / peer memory), miss_ms the sum over the launches that fetch missed rows from
 * pinned host memory (every batch of the window); gather_ms covers n_timed batches: all batches of
 * the window when launching one by one, the last batch of each pipe when replaying graphs, whose
 * events are overwritten per launch. */
int legion_runner_timing(LegionRunner *r, float *batch_ms, float *gather_ms, float *miss_ms, int32_t *n_batches,
                         int32_t *n_timed);
/* Stage times of the last window that ran with time_kernels (the per-op times of the reference's
 * MONITOR build, engine/server.cu:346-395): six floats per batch = begin / end of sampling, of the
 * gather and of the host-link fetch, in ms since the window's start.  Returns the batch count. */
int legion_runner_trace(LegionRunner *r, float *out, int32_t max_batches);
/* The serving loop of GPUServer (engine/server.cu:39-44,124-143) for `count` batches starting at
 * first_global_batch, with mode and local batch number taken from the IPC environment. */
int legion_runner_serve(LegionRunner *r, int32_t first_global_batch, int32_t count, int32_t timeout_ms);
int legion_runner_destroy(LegionRunner *r);

#ifdef __cplusplus
}
#endif
#endif
