// Cache lookup fused with the feature gather.
//
// One warp owns 32 consecutive rows of the segment: every lane looks up one id (one coalesced id
// load, one 4-byte table read), turns the answer into a source pointer (this GPU's partition, a
// peer's partition reached by plain loads over NVLink, or the pinned host table reached by
// zero-copy loads), and the warp then copies the rows four at a time with 16-byte loads so that
// 4 x 512 B per warp are in flight before the first store.  Stores are streaming (the trainer
// reads the rows once).  Hit / miss sets leave the kernel in cache_index exactly as FindFeat
// would have written them.
//
// Replaces bght::bcht::find + multiGPU_feat_cache_lookup (sampling_server/src/cache/cache.cu:157-192,
// 743-781; cache/cache_impl.cuh:239-303: thread-per-float, 4-byte loads, 32-64 CTAs) and
// static_retrieve_kernel + static_transfer_kernel (comp_cache/static_cache_kernel.cuh:185-266).
#include "common.cuh"
#include <cstdlib>

#include <cuda_fp8.h>
#include <string.h>

namespace legion {

static constexpr unsigned kFull = 0xFFFFFFFFu;

struct GatherParams {
    const int32_t *ids;
    int32_t *nc;  // node_counter of the pipe
    int32_t op_id;
    const int32_t *lut;
    int32_t capacity, kg, ki;
    const uint8_t *part[LEGION_MAX_DEVICE + 1];  // part[kg]: this GPU's private copies of rows that peers hold
    const uint8_t *host;
    int64_t n_nodes;
    uint8_t *dst;
    int32_t *cache_index;
    unsigned long long *stats;
    int32_t row_bytes;   // bytes of one output row
    int32_t slot_bytes;  // bytes of one cached row
    int32_t feature_len; // elements per row (quantised codecs)
    int2 *miss_rows;     // (position in ids, host table row) of rows whose source is the host table
    int32_t *miss_count; // [0] number of entries
    int32_t *err;        // device error word of the pipe (sticky), or nullptr
    // rows of uncached seeds that the copy engine staged in device memory for this batch: entry r < stage_n of the
    // id list, when it misses the cache, is row stage_pos[r] - stage_base of stage_rows (nullptr: no staging)
    const uint8_t *stage_rows;
    const int32_t *stage_pos;
    int32_t stage_base, stage_n;
};

// A missed row that sits in the batch's staging area is served from there like a cached row; `where` 4 keeps
// it out of the hit / miss counters and off the miss list.
__device__ __forceinline__ void use_staged(const GatherParams &p, int index, int &where, const uint8_t *&src)
{
    if (where == 2 && p.stage_rows != nullptr && index < p.stage_n) {
        src = p.stage_rows + (int64_t)(__ldg(&p.stage_pos[index]) - p.stage_base) * p.row_bytes;
        where = 4;
    }
}

__device__ __forceinline__ const uint8_t *shfl_ptr(const uint8_t *p, int src)
{
    unsigned long long v = (unsigned long long)p;
    unsigned lo = __shfl_sync(kFull, (unsigned)v, src);
    unsigned hi = __shfl_sync(kFull, (unsigned)(v >> 32), src);
    return (const uint8_t *)(((unsigned long long)hi << 32) | lo);
}

// Segment of a lookup op: the seeds (op 1) or the nodes found by hop h (op 3h+1).  Taken from
// the cumulative counts nc[9+h], which are written once per batch, so that a gather may overlap
// the sampling of the next hop on another stream.  Block 0 also leaves the (offset, size)
// snapshot that counter_update writes for a lookup op (operator_impl.cu:85-87).
__device__ __forceinline__ void segment_of(int32_t *nc, int op_id, int &off, int &n)
{
    if (op_id == kOpGatherAll) {
        // every node of the batch in one launch (the runner's choice: one long gather instead of one
        // short one per hop); the snapshot words get the values the last per-hop lookup would leave
        const int hops = nc[LEGION_INTRABATCH_CON * 3 - 1];
        off = 0;
        n = nc[LEGION_INTRABATCH_CON * 3 + hops];
        if (blockIdx.x == 0 && threadIdx.x == 0) {
            const int last = hops > 0 ? nc[LEGION_INTRABATCH_CON * 3 + hops - 1] : 0;
            nc[2] = last;
            nc[3] = n - last;
        }
        return;
    }
    const int h = op_id / LEGION_INTRABATCH_CON;
    off = h > 0 ? nc[LEGION_INTRABATCH_CON * 3 + h - 1] : 0;
    n = nc[LEGION_INTRABATCH_CON * 3 + h] - off;
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        nc[(op_id % LEGION_INTRABATCH_CON) * 2] = off;
        nc[(op_id % LEGION_INTRABATCH_CON) * 2 + 1] = n;
    }
}

// Looks one id up and resolves it to a source row.  `where`: 0 local, 1 peer, 2 host, 3 none.
// A table entry >= 0 is the global cache index; LEGION_CACHEMISS_FLAG (-2) means "row `id` of the
// host table"; an entry <= -3 means "row -(entry + 3) of the host table", for host tables that are
// not laid out in id order (legion_cache_fill_static_rows).  `host_row` is the row to fetch on a miss;
// gidx leaves as the reference's FindFeat would write it.
__device__ __forceinline__ const uint8_t *resolve(const GatherParams &p, int32_t id, int32_t &gidx, int &where,
                                                  int32_t &host_row)
{
    gidx = LEGION_CACHEMISS_FLAG;
    where = 3;
    host_row = id;
    if (id < 0 || id >= p.n_nodes) return nullptr;  // not a node: nothing is read, the output row stays as it is
    if (p.lut != nullptr) gidx = __ldg(&p.lut[id]);
    if (gidx >= 0) {
        int d = gidx / p.capacity;
        int row = gidx - d * p.capacity;
        const uint8_t *base = d <= LEGION_MAX_DEVICE ? p.part[d] : nullptr;
        if (base != nullptr) {
            where = (d == p.ki || d == p.kg) ? 0 : 1;
            return base + (int64_t)row * p.slot_bytes;
        }
        gidx = LEGION_CACHEMISS_FLAG;  // the table names a partition this call was not given: served as a miss
    }
    if (gidx <= -3) host_row = -(gidx + 3);
    gidx = LEGION_CACHEMISS_FLAG;
    if (p.host != nullptr) {
        where = 2;
        return p.host + ((int64_t)host_row % p.n_nodes) * (int64_t)p.row_bytes;
    }
    return nullptr;
}

// Rows served by the host table are not copied by the hit kernels: the warp appends them to the
// batch's miss list (one atomicAdd per warp, ranks by ballot) and clears their source pointer.
// The list holds (position in `ids`, row of the host table), so the miss kernel needs nothing else of the batch
// and may still run while the next batch on the same pipe is being sampled; it empties the list.
__device__ __forceinline__ void defer_misses(int2 *miss_rows, int32_t *miss_count, int row, int32_t id, int where,
                                             const uint8_t *&src, int lane)
{
    unsigned m = __ballot_sync(kFull, where == 2);
    if (m == 0u) return;
    int base = 0;
    if (lane == 0) base = atomicAdd(&miss_count[0], __popc(m));
    base = __shfl_sync(kFull, base, 0);
    if (where == 2) {
        miss_rows[base + __popc(m & ((1u << lane) - 1u))] = make_int2(row, id);
        src = nullptr;
    }
}

// The same in two halves, for a kernel that wants the row copies of the chunk in flight before it needs the
// list position: the first half counts the chunk's misses, asks for their place in the list (the atomic's answer
// travels while the rows do) and clears their source pointers; the second half writes the entries.
struct MissTicket {
    unsigned mask;
    int base;
};
__device__ __forceinline__ MissTicket miss_begin(int32_t *miss_count, int where, const uint8_t *&src, int lane)
{
    MissTicket t;
    t.mask = __ballot_sync(kFull, where == 2);
    t.base = 0;
    if (t.mask != 0u && lane == 0) t.base = atomicAdd(&miss_count[0], __popc(t.mask));
    if (where == 2) src = nullptr;
    return t;
}
__device__ __forceinline__ void miss_finish(int2 *miss_rows, const MissTicket &t, int row, int32_t id, int where, int lane)
{
    if (t.mask == 0u) return;
    const int base = __shfl_sync(kFull, t.base, 0);
    if (where == 2) miss_rows[base + __popc(t.mask & ((1u << lane) - 1u))] = make_int2(row, id);
}

// Hit / miss counters of a CTA, added to the cache's counters once per CTA (three atomics on three words that
// every warp of every gather would otherwise hit).
__device__ __forceinline__ void count_where(int *cta_counts, int where, int lane)
{
    unsigned m0 = __ballot_sync(kFull, where == 0);
    unsigned m1 = __ballot_sync(kFull, where == 1);
    unsigned m2 = __ballot_sync(kFull, where == 2);
    if (lane == 0) {
        if (m0) atomicAdd(&cta_counts[0], __popc(m0));
        if (m1) atomicAdd(&cta_counts[1], __popc(m1));
        if (m2) atomicAdd(&cta_counts[2], __popc(m2));
    }
}

__device__ __forceinline__ void add_stats(unsigned long long *stats, int where, int lane)
{
    unsigned m0 = __ballot_sync(kFull, where == 0);
    unsigned m1 = __ballot_sync(kFull, where == 1);
    unsigned m2 = __ballot_sync(kFull, where == 2);
    if (stats != nullptr && lane == 0) {
        if (m0) atomicAdd(&stats[0], (unsigned long long)__popc(m0));
        if (m1) atomicAdd(&stats[1], (unsigned long long)__popc(m1));
        if (m2) atomicAdd(&stats[2], (unsigned long long)__popc(m2));
    }
}

// The two halves of resolve(), for callers that fetch the table entry of the next chunk early.
__device__ __forceinline__ int32_t lookup_raw(const GatherParams &p, int32_t id)
{
    return (id >= 0 && id < p.n_nodes && p.lut != nullptr) ? __ldg(&p.lut[id]) : LEGION_CACHEMISS_FLAG;
}
__device__ __forceinline__ const uint8_t *decode_raw(const GatherParams &p, int32_t id, int32_t raw, int32_t &gidx,
                                                     int &where, int32_t &host_row)
{
    gidx = LEGION_CACHEMISS_FLAG;
    where = 3;
    host_row = id;
    if (id < 0 || id >= p.n_nodes) return nullptr;  // not a node: nothing is read, the output row stays as it is
    if (raw >= 0) {
        int d = raw / p.capacity;
        int row = raw - d * p.capacity;
        const uint8_t *base = d <= LEGION_MAX_DEVICE ? p.part[d] : nullptr;
        if (base != nullptr) {
            gidx = raw;
            where = (d == p.ki || d == p.kg) ? 0 : 1;
            return base + (int64_t)row * p.slot_bytes;
        }
        // the table names a partition this call was not given: served as a miss
    }
    if (raw <= -3) host_row = -(raw + 3);
    if (p.host != nullptr) {
        where = 2;
        return p.host + ((int64_t)host_row % p.n_nodes) * (int64_t)p.row_bytes;
    }
    return nullptr;
}

// Rows whose size is a multiple of 16 bytes.  VPL = 16-byte vectors per lane per row,
// R = rows copied together (R * VPL * 512 bytes in flight per warp).  A warp looks 32 ids up, one per
// lane, then copies their rows R at a time; while the first rows of a chunk are in flight it already
// fetches the id and the table entry of its next chunk, so that only the first lookup of a warp is
// exposed.
template <int VPL, int R, int RPW = 32>
__global__ void __launch_bounds__(256) gather_vec_kernel(GatherParams p)
{
    // RPW = rows one warp looks up and copies per chunk (32: one per lane; 16 or 8: the upper lanes idle during
    // the lookup, but a warp's life is shorter, so the last wave of CTAs costs less)
    static_assert(RPW == 32 || RPW == 16 || RPW == 8, "rows per warp");
    static_assert(RPW >= R, "a chunk holds at least one round of rows");
    __shared__ int cta_counts[3];
    if (threadIdx.x < 3) cta_counts[threadIdx.x] = 0;
    __syncthreads();
    int off, n;
    segment_of(p.nc, p.op_id, off, n);
    const int lane = threadIdx.x & 31;
    const int n_warps = (gridDim.x * blockDim.x) >> 5;
    const int row_vec = p.row_bytes >> 4;
    int c = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (blockIdx.x * (blockDim.x >> 5) * RPW >= n) return;  // the whole CTA is past the end
    int32_t id = (lane < RPW && c * RPW + lane < n) ? __ldg(&p.ids[off + c * RPW + lane]) : -1;
    int32_t raw = lookup_raw(p, id);
    for (; c * RPW < n; c += n_warps) {
        const int r = c * RPW + lane;
        int32_t gidx, host_row;
        int where;
        const uint8_t *src = decode_raw(p, id, raw, gidx, where, host_row);
        if (lane < RPW && r < n) p.cache_index[off + r] = gidx;
        use_staged(p, off + r, where, src);
        if (p.stats != nullptr) count_where(cta_counts, where, lane);
        const MissTicket ticket = miss_begin(p.miss_count, where, src, lane);
        const int rows_here = min(RPW, n - c * RPW);
        uint8_t *dst_base = p.dst + (int64_t)(off + c * RPW) * p.row_bytes;
        const int rn = (c + n_warps) * RPW + lane;
        id = (lane < RPW && rn < n) ? __ldg(&p.ids[off + rn]) : -1;
        for (int j0 = 0; j0 < rows_here; j0 += R) {
            uint4 v[R][VPL];
            const uint8_t *sp[R];
#pragma unroll
            for (int jj = 0; jj < R; ++jj) {
                sp[jj] = shfl_ptr(src, (j0 + jj) & 31);
                if (j0 + jj >= rows_here) sp[jj] = nullptr;
            }
#pragma unroll
            for (int jj = 0; jj < R; ++jj) {
#pragma unroll
                for (int q = 0; q < VPL; ++q) {
                    int idx = lane + 32 * q;
                    if (sp[jj] != nullptr && idx < row_vec)
                        v[jj][q] = *reinterpret_cast<const uint4 *>(sp[jj] + idx * 16);
                }
            }
            if (j0 == 0) raw = lookup_raw(p, id);
#pragma unroll
            for (int jj = 0; jj < R; ++jj) {
#pragma unroll
                for (int q = 0; q < VPL; ++q) {
                    int idx = lane + 32 * q;
                    if (sp[jj] != nullptr && idx < row_vec)
                        __stcs(reinterpret_cast<uint4 *>(dst_base + (int64_t)(j0 + jj) * p.row_bytes + idx * 16),
                               v[jj][q]);
                }
            }
        }
        miss_finish(p.miss_rows, ticket, off + r, host_row, where, lane);
    }
    __syncthreads();
    if (p.stats != nullptr && threadIdx.x < 3 && cta_counts[threadIdx.x] != 0)
        atomicAdd(&p.stats[threadIdx.x], (unsigned long long)cta_counts[threadIdx.x]);
}

// ---- the same gather with the copy engine of the SM (bulk asynchronous copies) -----------------------
//
// A warp looks 32 ids up, one per lane, as above; then every lane whose row is held in GPU memory issues
// ONE bulk copy global -> shared for its whole row (cp.async.bulk, completion counted in bytes on the
// warp's mbarrier), the warp waits for the barrier, and every lane issues ONE bulk copy shared -> global
// into the output row.  No row data passes through registers, so a warp keeps 32 rows (16 KB for
// 512-byte rows) in flight with a handful of registers, and three CTAs of four warps hold 192 KB of
// reads in flight per SM.  Rows, shared-memory slots and output rows are 16-byte aligned and a multiple
// of 16 bytes long, which is all that the untiled bulk copy asks for; no multicast, no tensor map.
// Every wait is bounded: on a timeout the warp raises DERR_BULK_TIMEOUT, waits once more (again bounded) for
// the copies it issued and leaves.  After that error the pipe's output rows are invalid and the caller must
// stop issuing work on this context (legion_pool_device_error reports it): a copy that is still on its way
// when the CTA retires would land in shared memory that no longer belongs to it.
constexpr int kBulkWarps = 4;
constexpr int kBulkWaitLimit = 1 << 20;

__device__ __forceinline__ uint32_t smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity)
{
    for (int spin = 0; spin < kBulkWaitLimit; ++spin) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}

__global__ void __launch_bounds__(kBulkWarps * 32) gather_bulk_kernel(GatherParams p)
{
    extern __shared__ __align__(128) uint8_t bulk_smem[];          // [warp][32 rows][row_bytes]
    __shared__ __align__(8) unsigned long long bars[kBulkWarps];
    int off, n;
    segment_of(p.nc, p.op_id, off, n);
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int n_warps = (gridDim.x * blockDim.x) >> 5;
    const uint32_t row_bytes = (uint32_t)p.row_bytes;
    uint8_t *my_rows = bulk_smem + (size_t)warp * 32 * row_bytes;
    const uint32_t my_slot = smem_addr(my_rows + (size_t)lane * row_bytes);
    const uint32_t bar = smem_addr(&bars[warp]);
    if (lane == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(bar) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    uint32_t parity = 0;
    bool store_pending = false;
    int c = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (c * 32 < n) {
        int32_t id = (c * 32 + lane < n) ? __ldg(&p.ids[off + c * 32 + lane]) : -1;
        int32_t raw = lookup_raw(p, id);
        for (; c * 32 < n; c += n_warps) {
            const int r = c * 32 + lane;
            int32_t gidx, host_row;
            int where;
            const uint8_t *src = decode_raw(p, id, raw, gidx, where, host_row);
            if (r < n) p.cache_index[off + r] = gidx;
            add_stats(p.stats, where, lane);
            defer_misses(p.miss_rows, p.miss_count, off + r, host_row, where, src, lane);
            const int rn = (c + n_warps) * 32 + lane;
            id = (rn < n) ? __ldg(&p.ids[off + rn]) : -1;
            const unsigned hits = __ballot_sync(kFull, src != nullptr);
            // the previous chunk's stores must have read their rows out of shared memory
            if (store_pending) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            __syncwarp();
            if (hits != 0u) {
                if (lane == 0) {
                    const uint32_t tx = (uint32_t)__popc(hits) * row_bytes;
                    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(tx) : "memory");
                }
                __syncwarp();
                if (src != nullptr)
                    asm volatile(
                        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                        :: "r"(my_slot), "l"(src), "r"(row_bytes), "r"(bar) : "memory");
            }
            raw = lookup_raw(p, id);  // the next chunk's table entries travel while the rows do
            if (hits != 0u) {
                const bool done = mbar_wait(bar, parity);
                parity ^= 1u;
                if (!__all_sync(kFull, done)) {
                    if (lane == 0 && p.err != nullptr) atomicCAS(p.err, DERR_NONE, DERR_BULK_TIMEOUT);
                    mbar_wait(bar, parity ^ 1u);  // one more bounded wait for the copies that are still on their way
                    break;
                }
                if (src != nullptr) {
                    uint8_t *dst = p.dst + (int64_t)(off + r) * p.row_bytes;
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                                 :: "l"(dst), "r"(my_slot), "r"(row_bytes) : "memory");
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    store_pending = true;
                }
            }
        }
    }
    // nothing of this CTA may still be in flight when its shared memory is given back
    if (store_pending) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

// Any row size that is a multiple of 4 bytes (rows of F floats with F odd, ...).
__global__ void __launch_bounds__(256) gather_word_kernel(GatherParams p)
{
    int off, n;
    segment_of(p.nc, p.op_id, off, n);
    const int lane = threadIdx.x & 31;
    const int n_warps = (gridDim.x * blockDim.x) >> 5;
    const int row_words = p.row_bytes >> 2;
    for (int c = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; c * 32 < n; c += n_warps) {
        const int r = c * 32 + lane;
        int32_t id = (r < n) ? __ldg(&p.ids[off + r]) : -1;
        int32_t gidx, host_row;
        int where;
        const uint8_t *src = resolve(p, id, gidx, where, host_row);
        if (r < n) p.cache_index[off + r] = gidx;
        use_staged(p, off + r, where, src);
        add_stats(p.stats, where, lane);
        defer_misses(p.miss_rows, p.miss_count, off + r, host_row, where, src, lane);
        const int rows_here = min(32, n - c * 32);
        uint32_t *dst_base = reinterpret_cast<uint32_t *>(p.dst + (int64_t)(off + c * 32) * p.row_bytes);
        for (int j = 0; j < rows_here; ++j) {
            const uint32_t *sp = reinterpret_cast<const uint32_t *>(shfl_ptr(src, j));
            if (sp == nullptr) continue;
            for (int w = lane; w < row_words; w += 32) __stcs(&dst_base[(int64_t)j * row_words + w], sp[w]);
        }
    }
}

// Compressed cache: a hit row holds feature_len one-byte codes followed by an fp32 scale
// and is expanded to fp32 here; a miss row is a plain fp32 row of the host table.
// x^ = float(code) * scale, one multiplication, so the host replay is exact.
template <int CODEC>
__device__ __forceinline__ float decode_code(uint8_t b)
{
    if (CODEC == LEGION_CODEC_INT8) return (float)(int8_t)b;
    __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
    return __half2float(__half(h));
}

template <int CODEC>
__global__ void __launch_bounds__(256) gather_quant_kernel(GatherParams p)
{
    int off, n;
    segment_of(p.nc, p.op_id, off, n);
    const int lane = threadIdx.x & 31;
    const int n_warps = (gridDim.x * blockDim.x) >> 5;
    const int f = p.feature_len;
    for (int c = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; c * 32 < n; c += n_warps) {
        const int r = c * 32 + lane;
        int32_t id = (r < n) ? __ldg(&p.ids[off + r]) : -1;
        int32_t gidx, host_row;
        int where;
        const uint8_t *src = resolve(p, id, gidx, where, host_row);
        if (r < n) p.cache_index[off + r] = gidx;
        add_stats(p.stats, where, lane);
        defer_misses(p.miss_rows, p.miss_count, off + r, host_row, where, src, lane);
        const int rows_here = min(32, n - c * 32);
        float *dst_base = reinterpret_cast<float *>(p.dst + (int64_t)(off + c * 32) * p.row_bytes);
        if (f <= 128) {
            // up to 128 codes per row: one 4-byte word per lane and row, 8 rows in flight per warp
            constexpr int R = 8;
            const bool mine = lane < (f >> 2);
            for (int j0 = 0; j0 < rows_here; j0 += R) {
                const uint8_t *sp[R];
                uint32_t packed[R];
                float scale[R];
#pragma unroll
                for (int jj = 0; jj < R; ++jj) {
                    sp[jj] = shfl_ptr(src, (j0 + jj) & 31);
                    if (j0 + jj >= rows_here) sp[jj] = nullptr;
                }
#pragma unroll
                for (int jj = 0; jj < R; ++jj) {
                    if (sp[jj] != nullptr && mine) {
                        packed[jj] = *reinterpret_cast<const uint32_t *>(sp[jj] + lane * 4);
                        scale[jj] = *reinterpret_cast<const float *>(sp[jj] + f);
                    }
                }
#pragma unroll
                for (int jj = 0; jj < R; ++jj) {
                    if (sp[jj] != nullptr && mine) {
                        float4 o;
                        o.x = __fmul_rn(decode_code<CODEC>((uint8_t)(packed[jj])), scale[jj]);
                        o.y = __fmul_rn(decode_code<CODEC>((uint8_t)(packed[jj] >> 8)), scale[jj]);
                        o.z = __fmul_rn(decode_code<CODEC>((uint8_t)(packed[jj] >> 16)), scale[jj]);
                        o.w = __fmul_rn(decode_code<CODEC>((uint8_t)(packed[jj] >> 24)), scale[jj]);
                        __stcs(reinterpret_cast<float4 *>(dst_base + (int64_t)(j0 + jj) * f) + lane, o);
                    }
                }
            }
            continue;
        }
        for (int j = 0; j < rows_here; ++j) {
            const uint8_t *sp = shfl_ptr(src, j);
            if (sp == nullptr) continue;  // invalid id, or a miss left to the miss kernel (raw fp32 row)
            float *drow = dst_base + (int64_t)j * f;
            {
                const float scale = *reinterpret_cast<const float *>(sp + f);  // f is a multiple of 4
                const int groups = f >> 2;
                for (int g = lane; g < groups; g += 32) {
                    uint32_t packed = *reinterpret_cast<const uint32_t *>(sp + g * 4);
                    float4 o;
                    o.x = __fmul_rn(decode_code<CODEC>((uint8_t)(packed)), scale);
                    o.y = __fmul_rn(decode_code<CODEC>((uint8_t)(packed >> 8)), scale);
                    o.z = __fmul_rn(decode_code<CODEC>((uint8_t)(packed >> 16)), scale);
                    o.w = __fmul_rn(decode_code<CODEC>((uint8_t)(packed >> 24)), scale);
                    __stcs(reinterpret_cast<float4 *>(drow) + g, o);
                }
            }
        }
    }
}

// Rows that miss the cache: one warp copies `R` rows of the miss list at a time from the pinned host
// table by zero-copy loads (16 bytes per lane, so a 512-byte row is four 128-byte reads on the
// host link).  Runs on its own stream with a grid of its own so that the link has thousands of
// reads in flight while the HBM-bound kernels of the next batch carry on.  The last CTA empties the
// list.  Measured alone on random 512-byte rows: 50.6 GB/s over a 1 GB table (0.91 of a pinned
// cudaMemcpy), 26 GB/s over 48 GB, where address translation of the scattered pages limits the link.
constexpr int kMissCtas = 148;     // CTAs of the host-link fetch (see launch_gather_misses)
constexpr int kMissThreads = 256;

struct MissParams {
    const int2 *miss_rows;
    int32_t *miss_count;
    int32_t *ticket;
    const uint8_t *host;
    int64_t n_nodes;
    uint8_t *dst;
    int32_t row_bytes;
    int32_t host_row_bytes;  // bytes of one row of the host table (compressed host tables: codes + scale, padded)
};

// The list is complete and consumed: the last CTA to finish empties it for the next batch.
__device__ __forceinline__ void miss_list_done(const MissParams &p, int *s_last)
{
    __syncthreads();
    if (threadIdx.x == 0) {
        int t = atomicAdd(p.ticket, 1);
        *s_last = (t == (int)gridDim.x - 1);
    }
    __syncthreads();
    if (*s_last && threadIdx.x == 0) {
        p.miss_count[0] = 0;
        *p.ticket = 0;
    }
}

// Host table stored as compressed rows (feature_len one-byte codes + fp32 scale): the fetch moves
// host_row_bytes per row over the host link instead of 4 * feature_len and decodes into the fp32 output row.
template <int CODEC, int R>
__global__ void __launch_bounds__(1024) gather_miss_quant_kernel(MissParams p)
{
    __shared__ int s_last;
    const int n = p.miss_count[0];
    const int lane = threadIdx.x & 31;
    const int n_warps = (gridDim.x * blockDim.x) >> 5;
    const int2 *list = p.miss_rows;
    const int f = p.row_bytes >> 2;
    const int groups = f >> 2;
    for (int m0 = ((blockIdx.x * blockDim.x + threadIdx.x) >> 5) * R; m0 < n; m0 += n_warps * R) {
        const uint8_t *sp[R];
        float *dp[R];
        float scale[R];
#pragma unroll
        for (int jj = 0; jj < R; ++jj) {
            sp[jj] = nullptr;
            dp[jj] = nullptr;
            if (m0 + jj < n) {
                const int2 e = __ldg(&list[m0 + jj]);
                sp[jj] = p.host + ((int64_t)e.y % p.n_nodes) * (int64_t)p.host_row_bytes;
                dp[jj] = reinterpret_cast<float *>(p.dst + (int64_t)e.x * p.row_bytes);
            }
        }
#pragma unroll
        for (int jj = 0; jj < R; ++jj)
            if (sp[jj] != nullptr) scale[jj] = *reinterpret_cast<const float *>(sp[jj] + f);
        for (int g0 = 0; g0 < groups; g0 += 32) {
            const int g = g0 + lane;
            uint32_t packed[R];
#pragma unroll
            for (int jj = 0; jj < R; ++jj)
                if (sp[jj] != nullptr && g < groups) packed[jj] = *reinterpret_cast<const uint32_t *>(sp[jj] + g * 4);
#pragma unroll
            for (int jj = 0; jj < R; ++jj) {
                if (sp[jj] != nullptr && g < groups) {
                    float4 o;
                    o.x = __fmul_rn(decode_code<CODEC>((uint8_t)(packed[jj])), scale[jj]);
                    o.y = __fmul_rn(decode_code<CODEC>((uint8_t)(packed[jj] >> 8)), scale[jj]);
                    o.z = __fmul_rn(decode_code<CODEC>((uint8_t)(packed[jj] >> 16)), scale[jj]);
                    o.w = __fmul_rn(decode_code<CODEC>((uint8_t)(packed[jj] >> 24)), scale[jj]);
                    __stcs(reinterpret_cast<float4 *>(dp[jj]) + g, o);
                }
            }
        }
    }
    miss_list_done(p, &s_last);
}

template <int R>
__global__ void __launch_bounds__(1024) gather_miss_kernel(MissParams p)
{
    __shared__ int s_last;
    const int n = p.miss_count[0];
    const int lane = threadIdx.x & 31;
    const int n_warps = (gridDim.x * blockDim.x) >> 5;
    const int2 *list = p.miss_rows;
    if ((p.row_bytes & 15) == 0) {
        const int row_vec = p.row_bytes >> 4;
        for (int m0 = ((blockIdx.x * blockDim.x + threadIdx.x) >> 5) * R; m0 < n; m0 += n_warps * R) {
            const uint8_t *sp[R];
            uint8_t *dp[R];
#pragma unroll
            for (int jj = 0; jj < R; ++jj) {
                sp[jj] = nullptr;
                dp[jj] = nullptr;
                if (m0 + jj < n) {
                    const int2 e = __ldg(&list[m0 + jj]);
                    sp[jj] = p.host + ((int64_t)e.y % p.n_nodes) * (int64_t)p.row_bytes;
                    dp[jj] = p.dst + (int64_t)e.x * p.row_bytes;
                }
            }
            for (int q0 = 0; q0 < row_vec; q0 += 32) {
                uint4 v[R];
                const int idx = q0 + lane;
#pragma unroll
                for (int jj = 0; jj < R; ++jj)
                    if (sp[jj] != nullptr && idx < row_vec) v[jj] = *reinterpret_cast<const uint4 *>(sp[jj] + idx * 16);
#pragma unroll
                for (int jj = 0; jj < R; ++jj)
                    if (sp[jj] != nullptr && idx < row_vec) __stcs(reinterpret_cast<uint4 *>(dp[jj] + idx * 16), v[jj]);
            }
        }
    } else {
        const int row_words = p.row_bytes >> 2;
        for (int m = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; m < n; m += n_warps) {
            const int2 e = __ldg(&list[m]);
            const uint32_t *sp = reinterpret_cast<const uint32_t *>(p.host + ((int64_t)e.y % p.n_nodes) * (int64_t)p.row_bytes);
            uint32_t *dp = reinterpret_cast<uint32_t *>(p.dst + (int64_t)e.x * p.row_bytes);
            for (int w = lane; w < row_words; w += 32) __stcs(&dp[w], sp[w]);
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int t = atomicAdd(p.ticket, 1);
        s_last = (t == (int)gridDim.x - 1);
        if (s_last) {  // every CTA has read its count by now
            p.miss_count[0] = 0;
            *p.ticket = 0;
        }
    }
}

// ---- set-associative LRU cache ----------------------------------------------------------------------
// Lookup ("retrieve_and_touch"): `ways` consecutive lanes probe one set; a hit stamps the way
// with the batch clock.  Addressing: set = id % sets (one GPU), slot = set * ways + way.
struct LruParams {
    const int32_t *ids;
    int32_t *nc;
    int32_t op_id;
    int32_t *keys, *stamps;
    int64_t sets;
    int32_t ways;
    const BatchCtl *bctl;  // clock of the batch
    const uint8_t *rows;
    const uint8_t *host;
    int64_t n_nodes;
    uint8_t *dst;
    int64_t *cache_index;
    unsigned long long *stats;
    int32_t row_bytes;
    int2 *miss_rows;
    int32_t *miss_count;
};

template <int VPL, int R>
__global__ void __launch_bounds__(256) gather_lru_kernel(LruParams p)
{
    int off, n;
    segment_of(p.nc, p.op_id, off, n);
    const int lane = threadIdx.x & 31;
    const int n_warps = (gridDim.x * blockDim.x) >> 5;
    const int row_vec = p.row_bytes >> 4;
    const int clock = p.bctl->clock;
    const int ways = p.ways;              // power of two, <= 32
    const int per_pass = 32 / ways;       // ids probed together by one warp
    const int sub = lane / ways, way = lane % ways;
    for (int c = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; c * 32 < n; c += n_warps) {
        const int r = c * 32 + lane;
        const int32_t my_id = (r < n) ? __ldg(&p.ids[off + r]) : -1;
        int64_t my_slot = -1;
        for (int pass = 0; pass < 32; pass += per_pass) {
            const int owner = pass + sub;  // lane whose id this group of `ways` lanes probes
            const int32_t id = __shfl_sync(kFull, my_id, owner);
            int64_t set = id >= 0 ? (int64_t)id % p.sets : 0;
            int32_t key = id >= 0 ? __ldcg(&p.keys[set * ways + way]) : -1;
            unsigned hitmask = __ballot_sync(kFull, id >= 0 && key == id);
            unsigned group = (ways == 32) ? hitmask : ((hitmask >> (sub * ways)) & ((1u << ways) - 1u));
            int hit_way = __ffs(group) - 1;
            if (hit_way == way && id >= 0) p.stamps[set * ways + way] = clock;
            // hand the answer to the owning lane
            int64_t slot = hit_way >= 0 ? set * ways + hit_way : -1;
#pragma unroll 1
            for (int g = 0; g < per_pass; ++g) {
                long long s_g = __shfl_sync(kFull, (long long)slot, g * ways);
                if (lane == pass + g) my_slot = s_g;
            }
        }
        if (r < n) p.cache_index[off + r] = my_slot;
        int where = 3;
        const uint8_t *src = nullptr;
        if (my_id >= 0) {
            if (my_slot >= 0) { where = 0; src = p.rows + my_slot * (int64_t)p.row_bytes; }
            else if (p.host != nullptr) { where = 2; src = p.host + ((int64_t)my_id % p.n_nodes) * (int64_t)p.row_bytes; }
        }
        add_stats(p.stats, where, lane);
        defer_misses(p.miss_rows, p.miss_count, off + r, my_id, where, src, lane);
        const int rows_here = min(32, n - c * 32);
        uint8_t *dst_base = p.dst + (int64_t)(off + c * 32) * p.row_bytes;
        for (int j0 = 0; j0 < rows_here; j0 += R) {
            uint4 v[R][VPL];
            const uint8_t *sp[R];
#pragma unroll
            for (int jj = 0; jj < R; ++jj) {
                sp[jj] = shfl_ptr(src, (j0 + jj) & 31);
                if (j0 + jj >= rows_here) sp[jj] = nullptr;
            }
#pragma unroll
            for (int jj = 0; jj < R; ++jj) {
#pragma unroll
                for (int q = 0; q < VPL; ++q) {
                    int idx = lane + 32 * q;
                    if (sp[jj] != nullptr && idx < row_vec)
                        v[jj][q] = *reinterpret_cast<const uint4 *>(sp[jj] + idx * 16);
                }
            }
#pragma unroll
            for (int jj = 0; jj < R; ++jj) {
#pragma unroll
                for (int q = 0; q < VPL; ++q) {
                    int idx = lane + 32 * q;
                    if (sp[jj] != nullptr && idx < row_vec)
                        __stcs(reinterpret_cast<uint4 *>(dst_base + (int64_t)(j0 + jj) * p.row_bytes + idx * 16),
                               v[jj][q]);
                }
            }
        }
    }
}

// Insertion phase, run once per batch after every gather (two launches):
//  claim : every missed id picks the way of its set with the smallest stamp (empty ways count
//          as -1, ways stamped in this batch are excluded, lowest way on ties) and bids for it
//          with its position in the id list (atomicMin);
//  commit: the lowest bidder writes key and stamp and copies its row from the batch's feature
//          buffer (already gathered) into the slot.
__global__ void lru_claim_kernel(const int32_t *__restrict__ ids, const int64_t *__restrict__ cache_index,
                                 const int32_t *__restrict__ nc, const int32_t *__restrict__ keys,
                                 const int32_t *__restrict__ stamps, int64_t sets, int ways,
                                 const BatchCtl *__restrict__ bctl, unsigned long long *claim,
                                 int64_t *victim /* per row: chosen slot or -1 */)
{
    const int clock = bctl->clock;
    const int n = nc[LEGION_INTRABATCH_CON * 3 + nc[LEGION_INTRABATCH_CON * 3 - 1]];  // all nodes of the batch
    for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < n; r += gridDim.x * blockDim.x) {
        int64_t v = -1;
        int32_t id = ids[r];
        if (id >= 0 && cache_index[r] < 0) {
            int64_t set = (int64_t)id % sets;
            int best = -1, best_stamp = 0;
            for (int w = 0; w < ways; ++w) {
                int32_t key = keys[set * ways + w];
                int32_t st = key == -1 ? -1 : stamps[set * ways + w];
                if (st == clock) continue;
                if (best < 0 || st < best_stamp) { best = w; best_stamp = st; }
            }
            if (best >= 0) {
                v = set * ways + best;
                atomicMin(&claim[v], (unsigned long long)r);
            }
        }
        victim[r] = v;
    }
}

__global__ void lru_commit_kernel(const int32_t *__restrict__ ids, const int32_t *__restrict__ nc, int32_t *keys,
                                  int32_t *stamps, const BatchCtl *__restrict__ bctl,
                                  const unsigned long long *__restrict__ claim,
                                  const int64_t *__restrict__ victim, const uint8_t *__restrict__ features,
                                  uint8_t *rows, int row_bytes, unsigned long long *stats)
{
    const int clock = bctl->clock;
    const int n = nc[LEGION_INTRABATCH_CON * 3 + nc[LEGION_INTRABATCH_CON * 3 - 1]];  // all nodes of the batch
    const int lane = threadIdx.x & 31;
    const int n_warps = (gridDim.x * blockDim.x) >> 5;
    const int row_vec = row_bytes >> 4;
    for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < n; r += n_warps) {
        int64_t v = victim[r];
        if (v < 0) continue;
        if (claim[v] != (unsigned long long)r) continue;  // a lower position won the way
        const uint4 *s = reinterpret_cast<const uint4 *>(features + (int64_t)r * row_bytes);
        uint4 *d = reinterpret_cast<uint4 *>(rows + v * (int64_t)row_bytes);
        for (int q = lane; q < row_vec; q += 32) d[q] = s[q];
        if (lane == 0) {
            keys[v] = ids[r];
            stamps[v] = clock;
            if (stats != nullptr) atomicAdd(&stats[3], 1ull);
        }
    }
}

__global__ void lru_claim_reset_kernel(const int64_t *__restrict__ victim, const int32_t *__restrict__ nc,
                                       unsigned long long *claim)
{
    const int n = nc[LEGION_INTRABATCH_CON * 3 + nc[LEGION_INTRABATCH_CON * 3 - 1]];  // all nodes of the batch
    for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < n; r += gridDim.x * blockDim.x) {
        int64_t v = victim[r];
        if (v >= 0) claim[v] = ~0ull;
    }
}

// ---- launchers ------------------------------------------------------------------------------------------

template <int VPL, int R, int RPW = 32>
static void launch_vec(int grid, cudaStream_t s, const GatherParams &gp)
{
    gather_vec_kernel<VPL, R, RPW><<<grid, 256, 0, s>>>(gp);
}
template <int VPL, int R>
static void launch_lru(int grid, cudaStream_t s, const LruParams &lp)
{
    gather_lru_kernel<VPL, R><<<grid, 256, 0, s>>>(lp);
}

// 0: loads and stores through registers; 1: bulk asynchronous copies through shared memory.  The
// environment variable LEGION_GATHER_ENGINE sets the start value (legion_set_tunable overrides it).
static int gather_engine_from_env()
{
    const char *v = getenv("LEGION_GATHER_ENGINE");
    return (v != nullptr && v[0] == '1' && v[1] == 0) ? 1 : 0;
}
int g_gather_engine = gather_engine_from_env();
int g_gather_cps = 0;  // CTAs per SM of the hit gathers (0 = default); see legion_set_tunable
int g_gather_rows = 0; // rows in flight per warp for 512-byte-class rows (0 = default)

int g_gather_rpw = 0;  // rows per warp and chunk of the 512-byte-class gather (0 = default); see legion_set_tunable

static int segment_grid(const LegionPool *p, int32_t op_id, int64_t *rows_out, int rows_per_warp = 32, int cps_default = 8)
{
    // worst-case rows of this segment: the seeds, or the new nodes of hop (op_id / 3), or all nodes
    int hop = op_id / LEGION_INTRABATCH_CON;  // 0 = seeds
    int64_t rows = p->batch_size;
    int64_t nodes = p->batch_size;
    for (int h = 0; h < hop; ++h) { rows = nodes * p->fanout[h]; nodes += rows; }
    if (op_id == kOpGatherAll) rows = p->max_nodes;
    if (rows_out) *rows_out = rows;
    int64_t chunks = (rows + rows_per_warp - 1) / rows_per_warp;
    int64_t g64 = (chunks + 7) / 8;
    int cap = p->sm_count * (g_gather_cps > 0 ? g_gather_cps : cps_default) * (32 / rows_per_warp);
    return (int)(g64 < 1 ? 1 : (g64 > cap ? cap : g64));
}

// Lookup + gather of every row that is served from GPU memory; rows served by the host table
// are listed for launch_gather_misses.
int launch_gather_hits(cudaStream_t s, LegionPool *p, LegionCache *c, int32_t op_id)
{
    const int pipe = p->pipe;
    const int grid = segment_grid(p, op_id, nullptr);
    const int row_bytes = p->row_bytes_out;

    if (c != nullptr && c->kind == 1) {
        LG_ARG(c->row_bytes == row_bytes && row_bytes % 16 == 0, "lru cache rows must be a multiple of 16 bytes");
        LruParams lp;
        lp.ids = p->ids[pipe];
        lp.nc = p->pub_nc[pipe % p->slots];  // the hand-off slot's counters (the pipe's own unless it samples ahead)
        lp.op_id = op_id;
        lp.keys = c->keys;
        lp.stamps = c->stamps;
        lp.sets = c->sets;
        lp.ways = c->ways;
        lp.bctl = p->bctl[pipe];
        lp.rows = (const uint8_t *)c->rows;
        lp.host = (const uint8_t *)c->host_table;
        lp.n_nodes = c->n_nodes;
        lp.dst = (uint8_t *)p->features[pipe];
        lp.cache_index = p->cache_index[pipe];
        lp.stats = c->stats;
        lp.row_bytes = row_bytes;
        lp.miss_rows = p->miss_rows[pipe];
        lp.miss_count = p->miss_count[pipe];
        int vpl = (row_bytes / 16 + 31) / 32;
        LG_ARG(vpl >= 1 && vpl <= 4, "row size above 2048 bytes is not supported by the lru gather");
        switch (vpl) {
        case 1: launch_lru<1, 4>(grid, s, lp); break;
        case 2: launch_lru<2, 2>(grid, s, lp); break;
        case 3: launch_lru<3, 2>(grid, s, lp); break;
        default: launch_lru<4, 2>(grid, s, lp); break;
        }
        LG_LAUNCH_CHECK();
        return LEGION_OK;
    }

    GatherParams gp;
    gp.ids = p->ids[pipe];
    gp.nc = p->pub_nc[pipe % p->slots];  // the hand-off slot's counters (the pipe's own unless it samples ahead)
    gp.op_id = op_id;
    gp.lut = c ? c->lut : nullptr;
    gp.capacity = c ? (c->capacity > 0 ? c->capacity : 1) : 1;
    gp.kg = c ? c->kg : 1;
    gp.ki = c ? c->ki : 0;
    for (int k = 0; k <= LEGION_MAX_DEVICE; ++k) gp.part[k] = c ? (const uint8_t *)c->part[k] : nullptr;
    gp.host = c ? (const uint8_t *)c->host_table : nullptr;
    gp.n_nodes = c ? c->n_nodes : 1;
    gp.dst = (uint8_t *)p->features[pipe];
    gp.cache_index = reinterpret_cast<int32_t *>(p->cache_index[pipe]);
    gp.stats = c ? c->stats : nullptr;
    gp.row_bytes = row_bytes;
    gp.slot_bytes = c ? c->slot_bytes : row_bytes;
    gp.feature_len = row_bytes / 4;
    gp.miss_rows = p->miss_rows[pipe];
    gp.miss_count = p->miss_count[pipe];
    gp.err = p->ctl[pipe] + CTL_ERROR;
    // staged seed rows are only meaningful for a launch that starts at the seeds, over uncompressed rows
    const bool staged = p->stage_rows != nullptr && (op_id == kOpGatherAll || op_id == 1) && c != nullptr &&
                        c->codec == LEGION_CODEC_RAW && g_gather_engine == 0;
    gp.stage_rows = staged ? p->stage_rows : nullptr;
    gp.stage_pos = staged ? p->stage_pos : nullptr;
    gp.stage_base = staged ? p->stage_base : 0;
    gp.stage_n = staged ? p->stage_n : 0;

    // the bulk-copy engine has only ever read this GPU's own memory: a clique of more than one GPU keeps the register path
    if (g_gather_engine == 1 && gp.kg == 1 && (c == nullptr || c->codec == LEGION_CODEC_RAW) && row_bytes % 16 == 0 &&
        row_bytes <= 1024 && gp.slot_bytes == row_bytes) {
        // 32 rows per warp in shared memory: 64 KB per CTA for 512-byte rows, three CTAs per SM
        const size_t smem = (size_t)kBulkWarps * 32 * row_bytes;
        static bool attr_set[64] = { false };
        if (p->dev_id >= 0 && p->dev_id < 64 && !attr_set[p->dev_id]) {
            LG_CUDA(cudaFuncSetAttribute(gather_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 1024));
            attr_set[p->dev_id] = true;
        }
        int64_t rows = 0;
        segment_grid(p, op_id, &rows);
        int64_t want = (rows + 32 * kBulkWarps - 1) / (32 * kBulkWarps);
        int per_sm = (int)(200 * 1024 / (smem + 1024));
        if (per_sm < 1) per_sm = 1;
        if (g_gather_cps > 0 && g_gather_cps < per_sm) per_sm = g_gather_cps;
        int64_t cap = (int64_t)p->sm_count * per_sm;
        int bgrid = (int)(want < 1 ? 1 : (want > cap ? cap : want));
        gather_bulk_kernel<<<bgrid, kBulkWarps * 32, smem, s>>>(gp);
        LG_LAUNCH_CHECK();
        return LEGION_OK;
    }

    if (c != nullptr && c->codec != LEGION_CODEC_RAW) {
        LG_ARG(gp.feature_len % 4 == 0, "compressed rows need a feature length that is a multiple of 4");
        if (c->codec == LEGION_CODEC_INT8) gather_quant_kernel<LEGION_CODEC_INT8><<<grid, 256, 0, s>>>(gp);
        else gather_quant_kernel<LEGION_CODEC_E4M3><<<grid, 256, 0, s>>>(gp);
        LG_LAUNCH_CHECK();
        return LEGION_OK;
    }
    if (row_bytes % 16 == 0 && row_bytes <= 2048) {
        int vpl = (row_bytes / 16 + 31) / 32;
        switch (vpl) {
        case 1:
            // 8 rows (4 KB) in flight per warp measured best on 512-byte rows (2: 0.47-0.55 of the copy
            // peak, 4: 0.55-0.57, 8: 0.58-0.61, 16: 0.52-0.55, over 2-8 CTAs per SM)
            // The gather over all nodes of a batch runs beside the sampling kernels of the other pipes.  With two
            // CTAs per SM (each warp then copies two or three chunks, the next chunk's lookups in flight) it
            // leaves a third of the register file to them: the launch alone is as fast as with eight (46.1 against
            // 45.7 us at 2 x 10^5 rows), the batch is 3% shorter with the whole table cached (70.1 against 72.4 us).
            if (g_gather_rpw == 16) launch_vec<1, 8, 16>(segment_grid(p, op_id, nullptr, 16), s, gp);
            else if (g_gather_rpw == 8) launch_vec<1, 8, 8>(segment_grid(p, op_id, nullptr, 8), s, gp);
            else if (g_gather_rows == 4) launch_vec<1, 4>(grid, s, gp);
            else if (g_gather_rows == 16) launch_vec<1, 16>(grid, s, gp);
            else if (g_gather_rows == 2) launch_vec<1, 2>(grid, s, gp);
            else launch_vec<1, 8>(op_id == kOpGatherAll ? segment_grid(p, op_id, nullptr, 32, 2) : grid, s, gp);
            break;
        case 2: launch_vec<2, 2>(grid, s, gp); break;
        case 3: launch_vec<3, 2>(grid, s, gp); break;
        default: launch_vec<4, 2>(grid, s, gp); break;
        }
    } else {
        LG_ARG(row_bytes % 4 == 0, "row size must be a multiple of 4 bytes");
        gather_word_kernel<<<grid, 256, 0, s>>>(gp);
    }
    LG_LAUNCH_CHECK();
    return LEGION_OK;
}

int g_miss_ctas = 0;     // 0 = default; see legion_set_tunable
int g_miss_threads = 0;  // 0 = default
int g_miss_rows = 0;     // rows a warp of the fetch keeps in flight (0 = default, 4)

// The rows the hit kernels listed so far, fetched from the pinned host table; empties the list.
// No-op without a host table.
int launch_gather_misses(cudaStream_t s, LegionPool *p, LegionCache *c)
{
    if (c == nullptr || c->host_table == nullptr) return LEGION_OK;
    const int pipe = p->pipe;
    MissParams mp;
    mp.miss_rows = p->miss_rows[pipe];
    mp.miss_count = p->miss_count[pipe];
    mp.ticket = p->miss_count[pipe] + 4;
    mp.host = (const uint8_t *)c->host_table;
    mp.n_nodes = c->n_nodes;
    mp.dst = (uint8_t *)p->features[pipe];
    mp.row_bytes = p->row_bytes_out;
    mp.host_row_bytes = c->host_codec != LEGION_CODEC_RAW ? c->slot_bytes : p->row_bytes_out;

    // A static cache behind seed staging leaves a few thousand scattered rows per batch, which arrive at the
    // scattered-page rate of the link whatever is in flight, while every row in flight slows the kernels beside
    // the fetch: one row per warp and four warps per CTA measured best (6.5 k batches/s against 6.1 k with four
    // rows per warp and eight warps).  An LRU cache misses tens of thousands of rows per batch: its fetch
    // keeps the wider shape.
    const bool many = c->kind == 1;
    int64_t g64 = (p->max_nodes + 31) / 32;
    int cap = g_miss_ctas > 0 ? g_miss_ctas : kMissCtas;
    int threads = g_miss_threads > 0 ? g_miss_threads : (many ? kMissThreads : 128);
    const int rows = g_miss_rows > 0 ? g_miss_rows : (many ? 4 : 1);
    int grid = (int)(g64 < 1 ? 1 : (g64 > cap ? cap : g64));
    if (c->host_codec == LEGION_CODEC_INT8) gather_miss_quant_kernel<LEGION_CODEC_INT8, 8><<<grid, threads, 0, s>>>(mp);
    else if (c->host_codec == LEGION_CODEC_E4M3) gather_miss_quant_kernel<LEGION_CODEC_E4M3, 8><<<grid, threads, 0, s>>>(mp);
    else if (rows == 1) gather_miss_kernel<1><<<grid, threads, 0, s>>>(mp);
    else if (rows == 2) gather_miss_kernel<2><<<grid, threads, 0, s>>>(mp);
    else if (rows == 8) gather_miss_kernel<8><<<grid, threads, 0, s>>>(mp);
    else gather_miss_kernel<4><<<grid, threads, 0, s>>>(mp);
    LG_LAUNCH_CHECK();
    return LEGION_OK;
}

int launch_gather(cudaStream_t s, LegionPool *p, LegionCache *c, int32_t op_id)
{
    int rc = launch_gather_hits(s, p, c, op_id);
    if (rc != LEGION_OK) return rc;
    return launch_gather_misses(s, p, c);
}

int launch_lru_insert(cudaStream_t s, LegionPool *p, LegionCache *c)
{
    if (c == nullptr || c->kind != 1) return LEGION_OK;
    const int pipe = p->pipe;
    const int cap = p->sm_count * 8;
    int64_t g_thread = (p->max_nodes + 255) / 256;
    int64_t g_warp = (p->max_nodes + 7) / 8;
    int grid_t = (int)(g_thread > cap ? cap : g_thread);
    int grid_w = (int)(g_warp > cap ? cap : g_warp);
    unsigned long long *claim = reinterpret_cast<unsigned long long *>(c->claim);
    lru_claim_kernel<<<grid_t, 256, 0, s>>>(p->ids[pipe], p->cache_index[pipe], p->node_counter[pipe], c->keys, c->stamps,
                                            c->sets, c->ways, p->bctl[pipe], claim, p->lru_victim[pipe]);
    LG_LAUNCH_CHECK();
    lru_commit_kernel<<<grid_w, 256, 0, s>>>(p->ids[pipe], p->node_counter[pipe], c->keys, c->stamps, p->bctl[pipe], claim,
                                             p->lru_victim[pipe], (const uint8_t *)p->features[pipe],
                                             (uint8_t *)c->rows, c->row_bytes, c->stats);
    LG_LAUNCH_CHECK();
    lru_claim_reset_kernel<<<grid_t, 256, 0, s>>>(p->lru_victim[pipe], p->node_counter[pipe], claim);
    LG_LAUNCH_CHECK();
    return LEGION_OK;
}

}  // namespace legion

// ---- gather without any allocation ---------------------------------------------------------------------
// legion_gather_rows_noalloc: the lookup + gather of one list of node ids (cached rows from the
// clique's partitions, the others from the pinned host table) for callers that must not allocate
// device memory when they call into this library: a trainer-side process whose framework allocator
// already owns the GPU's memory, or a serving loop that cannot afford the device-wide
// synchronisation, the fragmentation or the failure of a cudaMalloc in the middle of a step.  The
// entry points above take their scratch (cache_index, the miss list and its counters, the segment
// words the kernels read) from a LegionPool, which allocates; this one keeps the same scratch in a
// fixed array inside the library image.  Every GPU that loads the library holds that array
// (256 B + 12 B per row of LEGION_NOALLOC_MAX_ROWS, about 3 MB) until the process exits.
static __device__ __align__(256) unsigned char g_noalloc_scratch[256 + 12 * (size_t)LEGION_NOALLOC_MAX_ROWS];

namespace legion {

// byte offsets inside the array
constexpr size_t kNaCounter = 0;     // 16 int32: the node_counter words the gather kernels read
constexpr size_t kNaMissCount = 64;  // 8 int32: [0] entries of the miss list, [4] ticket
constexpr size_t kNaMissRows = 256;  // int2[LEGION_NOALLOC_MAX_ROWS]
constexpr size_t kNaCacheIndex = 256 + 8 * (size_t)LEGION_NOALLOC_MAX_ROWS;  // int32[LEGION_NOALLOC_MAX_ROWS]

// The array is shared by every call and keeps what the last call left: the words that must start
// from a known value are rewritten here at the start of each call.
__global__ void noalloc_setup_kernel(int32_t *nc, int32_t *miss_count, int32_t n_rows)
{
    const int t = threadIdx.x;
    if (t < 16) nc[t] = 0;
    if (t < 8) miss_count[t] = 0;
    __syncthreads();
    if (t == 0) {
        nc[LEGION_INTRABATCH_CON * 3 - 1] = 0;   // no hops: one segment
        nc[LEGION_INTRABATCH_CON * 3] = n_rows;  // rows [0, n_rows)
    }
}

}  // namespace legion

// In host code the name g_noalloc_scratch is only a stand-in for the device array: its device
// address is asked for once per device, with that device current, and kept here.
static void *g_noalloc_ptr[64] = { nullptr };
static cudaError_t noalloc_scratch_of(int dev_id, unsigned char **out)
{
    if (g_noalloc_ptr[dev_id] == nullptr) {
        void *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess) return e;
        g_noalloc_ptr[dev_id] = p;
    }
    *out = (unsigned char *)g_noalloc_ptr[dev_id];
    return cudaSuccess;
}

extern "C" int legion_gather_rows_noalloc(void *stream, int32_t dev_id, const int32_t *ids_dev, int64_t n_rows,
                                          const int32_t *lut_dev, int32_t capacity, int32_t kg, int32_t ki,
                                          const void *const *partitions, const void *host_table, int64_t n_nodes,
                                          int32_t row_bytes, void *out_dev)
{
    using namespace legion;
    LG_ARG(dev_id >= 0 && dev_id < 64, "dev_id out of range");
    LG_ARG(n_rows >= 0 && (n_rows == 0 || (ids_dev != nullptr && out_dev != nullptr)), "NULL pointer");
    if (n_rows > LEGION_NOALLOC_MAX_ROWS) {
        set_error("legion_gather_rows_noalloc: %lld rows are above the built-in scratch of %d rows; split the list or "
                  "use legion_feature_cache_lookup with a LegionPool",
                  (long long)n_rows, LEGION_NOALLOC_MAX_ROWS);
        return LEGION_E_LIMIT;
    }
    LG_ARG(row_bytes > 0 && row_bytes % 4 == 0, "row_bytes must be a positive multiple of 4");
    LG_ARG(kg >= 1 && kg <= LEGION_MAX_DEVICE && ki >= 0 && ki < kg, "bad clique size or member index");
    LG_ARG(lut_dev == nullptr || (capacity > 0 && partitions != nullptr), "a lookup table needs partitions");
    LG_ARG(n_nodes > 0, "n_nodes must be positive");
    LG_CUDA(cudaSetDevice(dev_id));
    unsigned char *scratch = nullptr;
    LG_CUDA(noalloc_scratch_of(dev_id, &scratch));
    if (n_rows == 0) return LEGION_OK;
    cudaStream_t s = (cudaStream_t)stream;
    int32_t *nc = reinterpret_cast<int32_t *>(scratch + kNaCounter);
    int32_t *miss_count = reinterpret_cast<int32_t *>(scratch + kNaMissCount);
    noalloc_setup_kernel<<<1, 32, 0, s>>>(nc, miss_count, (int32_t)n_rows);
    LG_LAUNCH_CHECK();

    GatherParams gp;
    gp.ids = ids_dev;
    gp.nc = nc;
    gp.op_id = 1;
    gp.lut = lut_dev;
    gp.capacity = capacity > 0 ? capacity : 1;
    gp.kg = kg;
    gp.ki = ki;
    for (int k = 0; k <= LEGION_MAX_DEVICE; ++k)
        gp.part[k] = (lut_dev != nullptr && k < kg) ? (const uint8_t *)partitions[k] : nullptr;
    gp.host = (const uint8_t *)host_table;
    gp.n_nodes = n_nodes;
    gp.dst = (uint8_t *)out_dev;
    gp.cache_index = reinterpret_cast<int32_t *>(scratch + kNaCacheIndex);
    gp.stats = nullptr;
    gp.err = nullptr;
    gp.stage_rows = nullptr;
    gp.stage_pos = nullptr;
    gp.stage_base = gp.stage_n = 0;
    gp.row_bytes = row_bytes;
    gp.slot_bytes = row_bytes;
    gp.feature_len = row_bytes / 4;
    gp.miss_rows = reinterpret_cast<int2 *>(scratch + kNaMissRows);
    gp.miss_count = miss_count;
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev_id);
    if (sms <= 0) sms = 148;
    int64_t g64 = ((n_rows + 31) / 32 + 7) / 8;
    int grid = (int)(g64 < 1 ? 1 : (g64 > (int64_t)sms * 8 ? (int64_t)sms * 8 : g64));
    if (row_bytes % 16 == 0 && row_bytes <= 2048) {
        int vpl = (row_bytes / 16 + 31) / 32;
        switch (vpl) {
        case 1: launch_vec<1, 8>(grid, s, gp); break;  // the shape the pool-based path launches
        case 2: launch_vec<2, 2>(grid, s, gp); break;
        case 3: launch_vec<3, 2>(grid, s, gp); break;
        default: launch_vec<4, 2>(grid, s, gp); break;
        }
    } else {
        gather_word_kernel<<<grid, 256, 0, s>>>(gp);
    }
    LG_LAUNCH_CHECK();
    if (host_table != nullptr) {
        MissParams mp;
        mp.miss_rows = gp.miss_rows;
        mp.miss_count = miss_count;
        mp.ticket = miss_count + 4;
        mp.host = (const uint8_t *)host_table;
        mp.n_nodes = n_nodes;
        mp.dst = (uint8_t *)out_dev;
        mp.row_bytes = row_bytes;
        mp.host_row_bytes = row_bytes;
        int64_t m64 = (n_rows + 31) / 32;
        int mgrid = (int)(m64 < 1 ? 1 : (m64 > (int64_t)sms * 2 ? (int64_t)sms * 2 : m64));
        gather_miss_kernel<4><<<mgrid, 256, 0, s>>>(mp);
        LG_LAUNCH_CHECK();
    }
    return LEGION_OK;
}

// Launch-shape knobs for measurements.  "miss_ctas": CTAs of the host-link fetch (0 = one per SM).
extern "C" int legion_set_tunable(const char *name, int32_t value)
{
    using namespace legion;
    LG_ARG(name != nullptr, "name is NULL");
    if (strcmp(name, "miss_ctas") == 0) {
        LG_ARG(value >= 0 && value <= 4096, "miss_ctas out of range");
        g_miss_ctas = value;
        return LEGION_OK;
    }
    if (strcmp(name, "miss_threads") == 0) {
        LG_ARG(value == 0 || (value >= 32 && value <= 1024 && value % 32 == 0), "miss_threads must be a multiple of 32 up to 1024");
        g_miss_threads = value;
        return LEGION_OK;
    }
    if (strcmp(name, "miss_rows") == 0) {
        LG_ARG(value == 0 || value == 1 || value == 2 || value == 4 || value == 8, "miss_rows must be 0, 1, 2, 4 or 8");
        g_miss_rows = value;
        return LEGION_OK;
    }
    if (strcmp(name, "map_front_shift") == 0) {
        LG_ARG(value >= -1 && value <= 30, "map_front_shift must be -1 (automatic) or 0..30");
        g_map_front_shift = value;  // pools created afterwards
        return LEGION_OK;
    }
    if (strcmp(name, "pdl") == 0) {
        LG_ARG(value == 0 || value == 1, "pdl must be 0 or 1");
        g_pdl = value;  // takes effect for runners created (graphs captured) afterwards
        return LEGION_OK;
    }
    if (strcmp(name, "gather_engine") == 0) {
        LG_ARG(value == 0 || value == 1, "gather_engine must be 0 (registers) or 1 (bulk copies)");
        g_gather_engine = value;
        return LEGION_OK;
    }
    if (strcmp(name, "gather_ctas_per_sm") == 0) {
        LG_ARG(value >= 0 && value <= 16, "gather_ctas_per_sm out of range");
        g_gather_cps = value;
        return LEGION_OK;
    }
    if (strcmp(name, "gather_rows_per_warp") == 0) {
        LG_ARG(value == 0 || value == 8 || value == 16 || value == 32, "gather_rows_per_warp must be 0, 8, 16 or 32");
        g_gather_rpw = value == 32 ? 0 : value;
        return LEGION_OK;
    }
    if (strcmp(name, "gather_rows_in_flight") == 0) {
        LG_ARG(value == 0 || value == 2 || value == 4 || value == 8 || value == 16, "gather_rows_in_flight must be 0, 2, 4, 8 or 16");
        g_gather_rows = value;
        return LEGION_OK;
    }
    set_error("legion_set_tunable: unknown name %s", name);
    return LEGION_E_ARG;
}
