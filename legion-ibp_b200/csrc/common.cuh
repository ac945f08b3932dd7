// Internal definitions shared by the kernels and the C ABI.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string>
#include <string.h>

#include "../../include/legion_b200.h"

namespace legion {

// ---- error reporting -------------------------------------------------------------------
void set_error(const char *fmt, ...);

#define LG_CUDA(call)                                                                      \
    do {                                                                                   \
        cudaError_t _e = (call);                                                           \
        if (_e != cudaSuccess) {                                                           \
            legion::set_error("%s:%d: %s -> %s", __FILE__, __LINE__, #call,                \
                              cudaGetErrorString(_e));                                     \
            cudaGetLastError(); /* reported here: it must not surface again at a later launch check */ \
            return LEGION_E_CUDA;                                                          \
        }                                                                                  \
    } while (0)

#define LG_ARG(cond, msg)                                                                  \
    do {                                                                                   \
        if (!(cond)) {                                                                     \
            legion::set_error("%s:%d: %s", __FILE__, __LINE__, msg);                       \
            return LEGION_E_ARG;                                                           \
        }                                                                                  \
    } while (0)

#define LG_LAUNCH_CHECK() LG_CUDA(cudaGetLastError())

// ---- device-side batch state --------------------------------------------------------------
// Tile = number of items (nodes or edges) one CTA scans at a time.
constexpr int kTile = 1024;
constexpr int kScanThreads = 256;  // kTile / 4 items per thread

// Values stored in the batch-local id map while a hop is in flight: a node that is new in
// this hop carries kNewBase + (index of the first edge that reached it) until it gets its
// local id.  Local ids stay below kNewBase.
constexpr int32_t kNewBase = 0x40000000;
// op id of the runner's single lookup + gather over every node of a batch
constexpr int32_t kOpGatherAll = -1;
constexpr int32_t kEmptyKey = -1;
constexpr int32_t kEmptyVal = 0x7FFFFFFF;

// ctl[] words (device scratch, one int32 each)
enum Ctl {
    CTL_N_NODES = 0,   // nodes known so far (== nc[0] + nc[1])
    CTL_E_TOTAL = 1,   // edges of the hops already finished
    CTL_E_HOP = 2,     // edges of the hop in flight
    CTL_C_HOP = 3,     // new nodes of the hop in flight
    CTL_TICKET_A = 4,  // "last CTA done" tickets, one per kernel that needs one
    CTL_TICKET_B = 5,
    CTL_TICKET_C = 6,
    CTL_ERROR = 7,     // first error raised by a kernel (0 = none)
    CTL_MISS_COUNT = 8,
    CTL_BACK_DIRTY = 9,  // the back region of the id map holds entries (kept across batches until it is cleared)
    CTL_TICKET_D = 10,
    CTL_BAD_IDS = 11,   // sticky: an id outside [0, n_nodes) was met and skipped (reported as DERR_BAD_ID; the batch goes on)
    CTL_WORDS = 16
};

enum DeviceError { DERR_NONE = 0, DERR_MAP_FULL = 1, DERR_EDGE_OVERFLOW = 2, DERR_NODE_OVERFLOW = 3,
                   DERR_BULK_TIMEOUT = 4,  // a bulk copy of the gather did not complete within its wait limit
                   DERR_BAD_ID = 5 };      // a node id outside [0, n_nodes) reached the path; it was skipped, not read

struct NodeRec {  // per input node of a hop, written by the count kernel
    int64_t start;  // first CSR position of the adjacency list
    int32_t loff;   // exclusive prefix of min(deg, fanout) inside the node's tile
    int32_t deg;
};
static_assert(sizeof(NodeRec) == 16, "NodeRec is read and written as one 16-byte vector");

struct MapSlot {
    int32_t key;
    int32_t val;
};

// The id map of a pipe is one array of slots in two regions.  The front region is sized for the
// batches that actually occur (an eighth of the worst case), so that it stays in L2 and costs little to
// clear; a key whose first kFrontProbes slots there are taken goes to the back region, which is sized
// for the worst case and is only cleared after a batch that used it.
struct MapDims {
    uint32_t front_mask;  // front slots - 1 (power of two)
    uint32_t back_mask;   // back slots - 1 (power of two); the back region starts at slot front_mask + 1
};
constexpr int kFrontProbes = 32;

// Per-batch parameters, kept in device memory (one copy per pipe) so that the launch sequence of a
// batch does not depend on them and can be replayed as a CUDA graph: only the kernel that writes
// this struct takes them by value.
struct BatchCtl {
    const int32_t *all_ids;     // seed list of the batch's mode
    const int32_t *all_labels;
    int64_t first;              // position of the batch's first seed in the list
    int32_t total_cap;          // length of the list
    int32_t size;               // seeds in this batch (the tail batch is shorter)
    int32_t hop_num;
    uint32_t global_batch;      // counter word of the sampler's RNG
    uint32_t k0, k1;            // RNG key
    int32_t max_rounds;
    int32_t clock;              // LRU batch clock
    int32_t *mirror;            // page-locked host words that receive both counter arrays after the last hop
    int32_t n_nodes;            // ids outside [0, n_nodes) are skipped and raise DERR_BAD_ID
};

}  // namespace legion

namespace legion {
struct VmmBlock {  // one mapping made through the virtual memory management API
    void *ptr;
    int64_t size;
    unsigned long long handle;
    int32_t imported;
};
int vmm_alloc(int dev, int64_t bytes, VmmBlock *out);
int vmm_export_fd(const VmmBlock *b, int *fd_out);
int vmm_import_fd(int dev, int fd, int64_t size, VmmBlock *out);
void vmm_free(VmmBlock *b);
}  // namespace legion

// ---- handle structs (opaque in the C ABI) ------------------------------------------------------
struct LegionGraph {
    int32_t dev_id;
    int64_t n_nodes, n_edges;
    const int64_t *indptr;
    const int32_t *indices;
};

struct LegionFeatures {
    int32_t dev_id;
    int64_t n_nodes;
    int32_t row_bytes;
    const void *host_table;
    const int32_t *ids[3];
    const int32_t *labels[3];
    int32_t count[3];
};

struct LegionCache {
    int32_t dev_id;
    int64_t n_nodes;
    int32_t row_bytes;   // bytes of one source (and output) row
    int32_t slot_bytes;  // bytes of one cached row (== row_bytes for RAW)
    int32_t codec;
    int32_t kind;  // 0 static, 1 lru
    // static
    int32_t kg, ki, capacity;
    int32_t *lut;                      // n_nodes entries, global index or CACHEMISS
    void *part[LEGION_MAX_DEVICE + 1]; // part[ki] is owned; part[kg] = private copies of hot rows that peers hold
    int32_t replica_rows;              // rows of part[kg] (legion_cache_add_replicas)
    int32_t fill_by_caller;            // set while legion_cache_place_static builds the table without copying rows
    int64_t fill_gen;                  // counts the changes of the lookup table (fill, replicas)
    legion::VmmBlock own_block;        // set when part[ki] is shareable memory (clique of more than one GPU)
    legion::VmmBlock peer_block[LEGION_MAX_DEVICE];  // partitions mapped from other processes
    // lru
    int64_t sets;
    int32_t ways;
    int32_t *keys, *stamps;
    int64_t *claim;
    void *rows;
    int32_t clock;
    const void *host_table;
    int32_t host_codec;         // codec of the host table's rows (RAW unless legion_cache_set_host_codec)
    unsigned long long *stats;  // 4 counters on the device
};

namespace legion {
// Rows of a seed list's uncached nodes in page-locked host memory, in list order (stage.cu).
struct SeedStage {
    int32_t valid;
    int32_t count;               // entries of the list
    const int32_t *ids_dev;      // the list on the device
    int32_t *own_ids_dev;        // owned device copy of a list that was registered from host memory, or nullptr
    const int32_t *host_base;    // where the registered host list lives in the caller's memory, or nullptr
    int32_t *host_copy;          // what it held at registration (batches are compared against it)
    int32_t *pos_dev;            // count + 1 entries: uncached entries before each list position
    int32_t *pos;                // the same on the host
    uint8_t *rows_host;          // pos[count] rows
    int64_t rows;
    int64_t fill_gen;            // generation of the cache's contents the staging was built for
    LegionCache *cache;
};
int stage_build(LegionCache *c, const int32_t *ids_dev, int32_t count, int sm_count, SeedStage *st);
void stage_free(SeedStage *st);
}  // namespace legion

struct LegionPool {
    int32_t dev_id;
    int32_t batch_size, hop_num;
    int32_t fanout[LEGION_MAX_HOPS];
    int32_t row_bytes_out;
    int32_t pipes;
    int64_t max_nodes, max_edges, max_hop_edges, max_inputs;
    int64_t input_tiles;  // entries of tile_sum / tile_off reserved for the counting kernels (edge tiles follow)
    int64_t feat_rows;
    // Hand-off buffers, `slots` sets: what a consumer reads (the seven buffers that are published to trainers).
    // With slots == pipes they ARE the pipes' own output buffers below.  With fewer slots than pipes
    // (legion_pool_create_ahead) every pipe samples into private buffers, ahead of the hand-off, and the block
    // structure is copied into the slot (pipe % slots) when the batch's gather is issued; features[pipe] is the
    // slot's feature buffer either way.
    int32_t slots;
    int32_t mirror_flip[LEGION_MAX_PIPES];  // which of a pipe's two counter mirrors the next batch on it writes (sampling ahead only)
    int32_t *pub_ids[LEGION_MAX_PIPES], *pub_labels[LEGION_MAX_PIPES], *pub_agg_src[LEGION_MAX_PIPES],
        *pub_agg_dst[LEGION_MAX_PIPES], *pub_nc[LEGION_MAX_PIPES], *pub_ec[LEGION_MAX_PIPES];
    // per pipe outputs
    int32_t *ids[LEGION_MAX_PIPES];
    void *features[LEGION_MAX_PIPES];
    int32_t *labels[LEGION_MAX_PIPES];
    int32_t *agg_src[LEGION_MAX_PIPES];
    int32_t *agg_dst[LEGION_MAX_PIPES];
    int32_t *node_counter[LEGION_MAX_PIPES];
    int32_t *edge_counter[LEGION_MAX_PIPES];
    // per pipe scratch (two batches may be in flight)
    int64_t *cache_index[LEGION_MAX_PIPES];      // one entry per node of the batch
    int32_t *src_global[LEGION_MAX_PIPES];       // sampled neighbour ids, all hops
    legion::MapSlot *map[LEGION_MAX_PIPES];      // batch-local id map
    uint32_t map_mask;        // back region of the id map: slots - 1
    uint32_t map_front_mask;  // front region: slots - 1
    legion::NodeRec *node_rec[LEGION_MAX_PIPES];
    int32_t *tile_sum[LEGION_MAX_PIPES], *tile_off[LEGION_MAX_PIPES];
    int32_t *eslot[LEGION_MAX_PIPES], *erank[LEGION_MAX_PIPES];
    uint8_t *edge_cnt[LEGION_MAX_PIPES];         // edges sampled for every destination, hop after hop (one byte each)
    int64_t *lru_victim[LEGION_MAX_PIPES];       // per node: way chosen for insertion, or -1
    int2 *miss_rows[LEGION_MAX_PIPES];           // (row, node id) to fetch from the host table
    int32_t *miss_count[LEGION_MAX_PIPES];       // [0] entries, [4] ticket
    int32_t *ctl[LEGION_MAX_PIPES];
    legion::BatchCtl *bctl[LEGION_MAX_PIPES];
    int32_t *seed_stage[LEGION_MAX_PIPES], *label_stage[LEGION_MAX_PIPES];  // device staging for host-provided seeds
    int32_t *h_stage[LEGION_MAX_PIPES];  // pinned host staging: seeds, labels, then both counter arrays
    // seed rows that the copy engine staged for the batch about to be gathered (set by the runner, else null)
    const uint8_t *stage_rows;
    const int32_t *stage_pos;
    int32_t stage_base, stage_n;
    // batch state
    int32_t iter, mode, pipe;
    uint32_t global_batch;
    uint64_t rng_seed;
    int32_t max_rounds;
    int32_t sm_count;
};

namespace legion {
// kernel launchers (defined in sample.cu / gather.cu / cache.cu)
extern int g_pdl;
extern int g_map_front_shift;
int launch_batch_generate(cudaStream_t s, LegionPool *p, const BatchCtl &ctl, bool defer_seeds = false);
BatchCtl make_batch_ctl(const LegionPool *p, const LegionCache *c, const int32_t *all_ids, const int32_t *all_labels,
                        int32_t total_cap, int64_t first, int32_t size, int64_t n_nodes);
const void *map_clear_kernel_address();
int launch_sample_hop(cudaStream_t s, LegionPool *p, const LegionGraph *g, int32_t fanout, int32_t hop,
                      int32_t op_id, bool seeds_pending = false);
int launch_gather(cudaStream_t s, LegionPool *p, LegionCache *c, int32_t op_id);
int launch_publish(cudaStream_t s, LegionPool *p);
int launch_gather_hits(cudaStream_t s, LegionPool *p, LegionCache *c, int32_t op_id);
int launch_gather_misses(cudaStream_t s, LegionPool *p, LegionCache *c);
int launch_lru_insert(cudaStream_t s, LegionPool *p, LegionCache *c);
int launch_hotness(cudaStream_t s, LegionPool *p, uint32_t *counts);
}  // namespace legion
