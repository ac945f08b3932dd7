// Seed batch generation, neighbour sampling, per-hop dedup and relabel.
//
// One hop is four launches on one stream, with every size kept on the device:
//   hop_count   : per input node degree, CSR start and its edge offset inside a 1024-node tile;
//                 the last CTA to finish turns the tile sums into tile offsets (no host sync);
//                 over the seeds it can also take the seed slice itself (batch_generate's work)
//   hop_sample  : one warp per input node draws the neighbours (Philox4x32-10 counter RNG),
//                 writes the edges at their final positions and enters every neighbour into the
//                 batch-local id map with atomicMin(first edge index)
//   hop_flag    : marks the edge that reached a new node first, ranks the marks per tile
//   hop_finish  : gives new nodes their local ids in order of first appearance and writes the
//                 local source id of every edge; the last CTA advances the counters
// The edge order (input after input, slot after slot) and the node order (first appearance in
// that edge order) do not depend on scheduling, so a host replay reproduces them bit for bit.
//
// Replaces batch_generate / random_sample / construct_graph / counter_update / ClearPosMap of
// sampling_server/src/engine/operator_impl.cu:28-91,178-317,598-604: the O(N) bitmap and
// position_map become a batch-local open-addressing map that stays in L2, the fixed <<<16,512>>>
// grid becomes a grid sized from the SM count, and the blocking counter read-backs disappear.
#include "common.cuh"
#include <cstdlib>

namespace legion {

static constexpr unsigned kFull = 0xFFFFFFFFu;

// Programmatic dependent launch.  A kernel launched with the attribute may be scheduled while its
// predecessor in the stream is still running; it must not touch the predecessor's results before
// pdl_wait() returns (all prerequisite grids complete, their writes visible).  pdl_trigger() lets the
// successor of THIS kernel be scheduled as soon as every CTA of this kernel has started.  Both are
// no-ops for a kernel launched the ordinary way.  The point: a hop is four 8-20 us kernels, and the
// drain / launch / ramp-up between two of them costs as much as a quarter of one.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ uint32_t mix32(uint32_t h)
{
    h ^= h >> 16; h *= 0x85EBCA6Bu; h ^= h >> 13; h *= 0xC2B2AE35u; h ^= h >> 16;
    return h;
}

// Enters `key` and lowers its value to `cand`; returns the slot.  Keys never change once
// written during a batch, so a stale read can only show "empty", which the CAS then corrects.
// The front region is tried first (kFrontProbes slots from the key's home slot).  Slots never empty
// during a batch, so every thread that carries the same key sees the same first usable slot there, or
// finds all of them taken by other keys and moves on to the back region, like every other thread
// with that key.
__device__ __forceinline__ int32_t map_insert_min(MapSlot *map, MapDims dims, int32_t key, int32_t cand,
                                                  int32_t *ctl)
{
    const uint32_t h = mix32((uint32_t)key);
    uint32_t s = h & dims.front_mask;
    for (int probe = 0; probe < kFrontProbes; ++probe) {
        int32_t k = __ldcg(&map[s].key);
        if (k == kEmptyKey) {
            int32_t old = atomicCAS(&map[s].key, kEmptyKey, key);
            k = (old == kEmptyKey) ? key : old;
        }
        if (k == key) {
            atomicMin(&map[s].val, cand);
            return (int32_t)s;
        }
        s = (s + 1) & dims.front_mask;
    }
    if (ctl[CTL_BACK_DIRTY] == 0) ctl[CTL_BACK_DIRTY] = 1;
    MapSlot *back = map + dims.front_mask + 1;
    s = mix32(h ^ 0x9E3779B9u) & dims.back_mask;
    for (uint32_t probe = 0; probe <= dims.back_mask; ++probe) {
        int32_t k = __ldcg(&back[s].key);
        if (k == kEmptyKey) {
            int32_t old = atomicCAS(&back[s].key, kEmptyKey, key);
            k = (old == kEmptyKey) ? key : old;
        }
        if (k == key) {
            atomicMin(&back[s].val, cand);
            return (int32_t)(dims.front_mask + 1 + s);
        }
        s = (s + 1) & dims.back_mask;
    }
    atomicCAS(&ctl[CTL_ERROR], DERR_NONE, DERR_MAP_FULL);
    return 0;
}

__device__ __forceinline__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                              uint32_t k0, uint32_t k1, uint32_t &o0, uint32_t &o1)
{
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
        uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
        uint32_t n0 = hi1 ^ c1 ^ k0;
        uint32_t n2 = hi0 ^ c3 ^ k1;
        c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    o0 = c0; o1 = c1;
}

// one bounded draw in [0, n): 64 random bits times n, high half
__device__ __forceinline__ uint32_t draw_below(uint32_t input_index, uint32_t lane, uint32_t round,
                                               uint32_t hop, uint32_t batch_id, uint32_t k0, uint32_t k1,
                                               uint32_t n)
{
    uint32_t w0, w1;
    philox4x32_10(input_index, round * 32u + lane, hop, batch_id, k0, k1, w0, w1);
    unsigned long long r64 = ((unsigned long long)w1 << 32) | w0;
    return (uint32_t)__umul64hi(r64, (unsigned long long)n);
}

// m distinct values of [0, n) in lanes 0..m-1 (m <= 32 < n).  All 32 lanes take part; lanes
// >= m hold a dummy that can never compare equal.  A lane keeps its draw unless a lane that
// already holds the value, or a lower lane that drew it in the same round, exists.
__device__ __forceinline__ uint32_t draw_distinct(int m, uint32_t n, uint32_t input_index, uint32_t hop,
                                                  uint32_t batch_id, uint32_t k0, uint32_t k1,
                                                  int max_rounds, int lane)
{
    bool kept = lane >= m;
    uint32_t x = 0x80000000u | (uint32_t)lane;
    for (int r = 0; r < max_rounds; ++r) {
        unsigned keptmask = __ballot_sync(kFull, kept);
        if (keptmask == kFull) break;
        if (!kept) x = draw_below(input_index, (uint32_t)lane, (uint32_t)r, hop, batch_id, k0, k1, n);
        unsigned peers = __match_any_sync(kFull, x);
        if (!kept) kept = ((peers & keptmask) == 0u) && ((__ffs(peers) - 1) == lane);
    }
    // Lanes still without a value after max_rounds take the next free value, in lane order.
    unsigned keptmask = __ballot_sync(kFull, kept);
    for (int guard = 0; guard < 32 && keptmask != kFull; ++guard) {
        int l = __ffs(~keptmask) - 1;
        uint32_t cand = __shfl_sync(kFull, x, l);
        for (int it = 0; it < 64; ++it) {
            unsigned clash = __ballot_sync(kFull, kept && lane < m && x == cand);
            if (!clash) break;
            cand = (cand + 1u) % n;
        }
        if (lane == l) { x = cand; kept = true; }
        keptmask = __ballot_sync(kFull, kept);
    }
    return x;
}

// exclusive scan over the CTA (kScanThreads threads); smem holds 8 ints
__device__ __forceinline__ int block_excl_scan(int x, int *total, int *smem)
{
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int incl = x;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        int t = __shfl_up_sync(kFull, incl, d);
        if (lane >= d) incl += t;
    }
    if (lane == 31) smem[warp] = incl;
    __syncthreads();
    int wo = 0, tot = 0;
#pragma unroll
    for (int w = 0; w < kScanThreads / 32; ++w) {
        int s = smem[w];
        if (w < warp) wo += s;
        tot += s;
    }
    __syncthreads();
    *total = tot;
    return wo + incl - x;
}

// The CTA that takes the last ticket turns tile sums into exclusive tile offsets and
// returns the grand total through *out_total (valid in thread 0 of that CTA only).
__device__ __forceinline__ bool last_cta_scan(int32_t *ticket, const int32_t *tile_sum, int32_t *tile_off,
                                              int n_tiles, int *smem, int *s_flag, int *out_total)
{
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        int t = atomicAdd(ticket, 1);
        *s_flag = (t == (int)gridDim.x - 1);
    }
    __syncthreads();
    if (!*s_flag) return false;
    __threadfence();
    int running = 0;
    for (int c0 = 0; c0 < n_tiles; c0 += kScanThreads) {
        int idx = c0 + threadIdx.x;
        int x = idx < n_tiles ? __ldcg(&tile_sum[idx]) : 0;
        int tot;
        int ex = block_excl_scan(x, &tot, smem);
        if (idx < n_tiles) tile_off[idx] = running + ex;
        running += tot;
    }
    if (threadIdx.x == 0) {
        *ticket = 0;
        *out_total = running;
    }
    return true;
}

// literal restatement of counter_update (operator_impl.cu:58-91), executed by one thread
__device__ __forceinline__ void counter_update(int32_t *nc, int32_t *ec, int op_id, int size, int hop_num)
{
    const int C = LEGION_INTRABATCH_CON;
    if (op_id == 0) {
        nc[0] = 0;
        nc[1] = size;
        nc[C * 3] = size;
        nc[C * 3 - 1] = hop_num;
    } else if (op_id % C == 0) {
        nc[0] = nc[0] + nc[1];
        nc[1] = nc[C * 2];
        nc[C * 2] = 0;
        nc[C * 2 + 1] = nc[0] + nc[1];
        ec[0] = ec[0] + ec[1];
        ec[1] = ec[2];
        ec[2] = 0;
        nc[C * 3 + op_id / C] = nc[0] + nc[1];
        ec[C * 3 + op_id / C] = ec[1];
        ec[C * 4 + op_id / C] = ec[0];
    } else {
        nc[(op_id % C) * 2] = nc[0];
        nc[(op_id % C) * 2 + 1] = nc[1];
    }
}

// ---- batch start -----------------------------------------------------------------------------

// First kernel of every batch: empties the id map, zeroes the counters and stores the batch's
// parameters, the only values of the batch that are passed by value.  The front region of the map is
// always cleared; the back region only if the last batch on this pipe put anything there.
__global__ void map_clear_kernel(uint4 *slots2, int64_t n_pairs, int32_t *ctl, int32_t *nc, int32_t *ec,
                                 BatchCtl *bctl, BatchCtl value, int64_t back_pairs)
{
    __shared__ int s_last;
    const bool back_dirty = ctl[CTL_BACK_DIRTY] != 0;  // final since the end of the last batch's sampling
    if (blockIdx.x == 0 && threadIdx.x == 32) *bctl = value;
    const uint4 empty = make_uint4((uint32_t)kEmptyKey, (uint32_t)kEmptyVal, (uint32_t)kEmptyKey,
                                   (uint32_t)kEmptyVal);
    const int64_t total = n_pairs + (back_dirty ? back_pairs : 0);
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x)
        slots2[i] = empty;
    if (blockIdx.x == 0 && threadIdx.x < 16) {
        // the error word is sticky; the dirty flag and its ticket are read by every CTA of this kernel
        if (threadIdx.x != CTL_ERROR && threadIdx.x != CTL_BAD_IDS && threadIdx.x != CTL_BACK_DIRTY && threadIdx.x != CTL_TICKET_D)
            ctl[threadIdx.x] = 0;
        nc[threadIdx.x] = 0;  // cudaMemsetAsync of both counters, operator_impl.cu:158-159
        ec[threadIdx.x] = 0;
    }
    // the last CTA to get here lowers the flag: every CTA has read it by then, and nothing enters the
    // map before the next kernel
    __syncthreads();
    if (threadIdx.x == 0) {
        int t = atomicAdd(&ctl[CTL_TICKET_D], 1);
        s_last = (t == (int)gridDim.x - 1);
    }
    __syncthreads();
    if (s_last && threadIdx.x == 0) {
        ctl[CTL_BACK_DIRTY] = 0;
        ctl[CTL_TICKET_D] = 0;
    }
}

__global__ void batch_generate_kernel(const BatchCtl *__restrict__ b, int32_t *ids, int32_t *labels, MapSlot *map,
                                      MapDims mask, int32_t *ctl, int32_t *nc, int32_t *ec)
{
    pdl_wait();
    pdl_trigger();
    const int32_t *__restrict__ all_ids = b->all_ids;
    const int32_t *__restrict__ all_labels = b->all_labels;
    const int32_t total_cap = b->total_cap, size = b->size, hop_num = b->hop_num;
    const int64_t first = b->first;
    int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < size) {
        int64_t pos = first + idx;
        if (pos >= total_cap) {  // operator_impl.cu:41-43
            ids[idx] = -1;
            labels[idx] = -1;
        } else {
            int32_t id = all_ids[pos % total_cap];
            if (id >= b->n_nodes) {  // not a node of this graph: skipped like an overrun slot, and reported
                id = -1;
                ctl[CTL_BAD_IDS] = 1;
            }
            ids[idx] = id;
            labels[idx] = all_labels[pos % total_cap];
            if (id >= 0) map_insert_min(map, mask, id, idx, ctl);
        }
    }
    if (idx == 0) {
        counter_update(nc, ec, 0, size, hop_num);
        ctl[CTL_N_NODES] = size;
        ctl[CTL_E_TOTAL] = 0;
    }
}

// ---- one hop -----------------------------------------------------------------------------------

// FIRST: the hop over the seeds also does the work of batch_generate_kernel (seed slice, labels, seeds
// into the id map, counter words of op 0), which saves one launch per batch.
template <bool FIRST>
__global__ void __launch_bounds__(kScanThreads)
hop_count_kernel(const int64_t *__restrict__ indptr, int32_t *ids, int32_t fanout,
                 NodeRec *rec, int32_t *tile_sum, int32_t *tile_off, int32_t *ctl, int64_t max_edges,
                 const BatchCtl *__restrict__ b, int32_t *labels, MapSlot *map, MapDims mask, int32_t *nc, int32_t *ec)
{
    pdl_wait();
    pdl_trigger();
    // the seeds are few (one batch): one item per thread and 256-node tiles give that launch 4 x the CTAs
    constexpr int IPT = FIRST ? 1 : 4;
    constexpr int TILE = kScanThreads * IPT;
    __shared__ int smem[kScanThreads / 32];
    __shared__ int s_flag;
    const int n = FIRST ? b->size : ctl[CTL_N_NODES];
    const int n_limit = b->n_nodes;
    const int n_tiles = (n + TILE - 1) / TILE;
    if (FIRST && blockIdx.x == 0 && threadIdx.x == 0) {
        counter_update(nc, ec, 0, n, b->hop_num);
        ctl[CTL_N_NODES] = n;
        ctl[CTL_E_TOTAL] = 0;
    }
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const int base = tile * TILE + threadIdx.x * IPT;
        int32_t v[4];
        if (FIRST) {
            const int32_t total_cap = b->total_cap;
            const int64_t first = b->first;
#pragma unroll
            for (int j = 0; j < IPT; ++j) {
                v[j] = -1;
                const int idx = base + j;
                if (idx < n) {
                    const int64_t pos = first + idx;
                    int32_t lab = -1;
                    if (pos < total_cap) {  // operator_impl.cu:41-43
                        v[j] = b->all_ids[pos % total_cap];
                        lab = b->all_labels[pos % total_cap];
                        if (v[j] >= n_limit) {  // not a node of this graph: skipped like an overrun slot, and reported
                            v[j] = -1;
                            ctl[CTL_BAD_IDS] = 1;
                        }
                    }
                    ids[idx] = v[j];
                    labels[idx] = lab;
                    if (v[j] >= 0 && pos < total_cap) map_insert_min(map, mask, v[j], idx, ctl);
                }
            }
        } else {
            int4 v4 = *reinterpret_cast<const int4 *>(ids + base);  // ids is padded to a whole tile
            v[0] = v4.x; v[1] = v4.y; v[2] = v4.z; v[3] = v4.w;
        }
        int64_t start[4];
        int32_t deg[4], cnt[4];
#pragma unroll
        for (int j = 0; j < IPT; ++j) {
            start[j] = 0; deg[j] = 0; cnt[j] = 0;
            if (base + j < n && v[j] >= 0) {
                if (v[j] < n_limit) {
                    int64_t s = indptr[v[j]];
                    int64_t e = indptr[v[j] + 1];
                    start[j] = s;
                    deg[j] = (int32_t)(e - s);
                    cnt[j] = min(deg[j], fanout);
                } else {  // a neighbour id that the topology itself got wrong is never followed
                    ctl[CTL_BAD_IDS] = 1;
                }
            }
        }
        int tsum = 0;
#pragma unroll
        for (int j = 0; j < IPT; ++j) tsum += cnt[j];
        int total;
        int ex = block_excl_scan(tsum, &total, smem);
#pragma unroll
        for (int j = 0; j < IPT; ++j) {
            if (base + j < n) {
                NodeRec r;
                r.start = start[j];
                r.loff = ex;
                r.deg = deg[j];
                *reinterpret_cast<int4 *>(&rec[base + j]) = *reinterpret_cast<int4 *>(&r);
            }
            ex += cnt[j];
        }
        if (threadIdx.x == 0) tile_sum[tile] = total;
    }
    int grand;
    if (last_cta_scan(&ctl[CTL_TICKET_A], tile_sum, tile_off, n_tiles, smem, &s_flag, &grand)) {
        if (threadIdx.x == 0) {
            ctl[CTL_E_HOP] = grand;
            const int e_total = FIRST ? 0 : ctl[CTL_E_TOTAL];
            if ((int64_t)e_total + grand > max_edges) atomicCAS(&ctl[CTL_ERROR], DERR_NONE, DERR_EDGE_OVERFLOW);
        }
    }
}

__global__ void __launch_bounds__(256)
hop_sample_kernel(const int32_t *__restrict__ indices, const NodeRec *__restrict__ rec,
                  const int32_t *__restrict__ tile_off, int32_t fanout, uint32_t hop,
                  const BatchCtl *__restrict__ b, int32_t *src_global, int32_t *agg_dst,
                  int32_t *eslot, MapSlot *map, MapDims mask, int32_t *ctl, int tile_shift,
                  const int32_t *nc, uint8_t *edge_cnt)
{
    pdl_wait();
    pdl_trigger();
    if (ctl[CTL_ERROR] != DERR_NONE) return;
    const uint32_t batch_id = b->global_batch, k0 = b->k0, k1 = b->k1;
    const int max_rounds = b->max_rounds;
    const int n = ctl[CTL_N_NODES];
    const int e_base = ctl[CTL_E_TOTAL];
    const int lane = threadIdx.x & 31;
    const int n_warps = (gridDim.x * blockDim.x) >> 5;
    const uint32_t k = (uint32_t)fanout;
    for (int i = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; i < n; i += n_warps) {
        int4 raw = __ldg(reinterpret_cast<const int4 *>(&rec[i]));
        NodeRec r = *reinterpret_cast<NodeRec *>(&raw);
        const uint32_t deg = (uint32_t)r.deg;
        if (lane == 0) {
            // this hop's per-destination edge counts start behind those of the hops before it, whose destinations
            // were the nodes known when each began (node_counter words 9 .. 9 + hop - 1; summed here, by one lane,
            // rather than held in a register of every thread for the whole kernel)
            int cnt_at = i;
            for (uint32_t h = 0; h < hop; ++h) cnt_at += __ldg(&nc[LEGION_INTRABATCH_CON * 3 + h]);
            edge_cnt[cnt_at] = (uint8_t)min(deg, k);
        }
        if (deg == 0) continue;
        const int eh0 = __ldg(&tile_off[i >> tile_shift]) + r.loff;  // tile of the counting kernel that ran before
        int out_slot = -1;   // slot of this lane's first edge, second edge in out_slot2
        int out_slot2 = -1;
        int64_t pos = 0, pos2 = 0;
        if (deg <= k) {
            if ((uint32_t)lane < deg) { out_slot = lane; pos = lane; }
        } else if (deg >= 2 * k) {
            uint32_t x = draw_distinct((int)k, deg, (uint32_t)i, hop, batch_id, k0, k1, max_rounds, lane);
            if ((uint32_t)lane < k) { out_slot = lane; pos = x; }
        } else {
            const int m = (int)(deg - k);
            uint32_t x = draw_distinct(m, deg, (uint32_t)i, hop, batch_id, k0, k1, max_rounds, lane);
            uint32_t mylo = (lane < m && x < 32u) ? (1u << x) : 0u;
            uint32_t myhi = (lane < m && x >= 32u) ? (1u << (x - 32u)) : 0u;
            uint32_t exlo = __reduce_or_sync(kFull, mylo);
            uint32_t exhi = __reduce_or_sync(kFull, myhi);
            uint32_t validlo = deg >= 32u ? 0xFFFFFFFFu : ((1u << deg) - 1u);
            uint32_t validhi = deg <= 32u ? 0u : (deg >= 64u ? 0xFFFFFFFFu : ((1u << (deg - 32u)) - 1u));
            uint32_t keeplo = ~exlo & validlo;
            uint32_t keephi = ~exhi & validhi;
            uint32_t below = (1u << lane) - 1u;
            if ((keeplo >> lane) & 1u) { out_slot = __popc(keeplo & below); pos = lane; }
            if ((keephi >> lane) & 1u) { out_slot2 = __popc(keeplo) + __popc(keephi & below); pos2 = lane + 32; }
        }
        if (out_slot >= 0) {
            int32_t u = __ldg(&indices[r.start + pos]);
            int eh = eh0 + out_slot;
            src_global[e_base + eh] = u;
            agg_dst[e_base + eh] = i;
            eslot[eh] = map_insert_min(map, mask, u, kNewBase + eh, ctl);
        }
        if (out_slot2 >= 0) {
            int32_t u = __ldg(&indices[r.start + pos2]);
            int eh = eh0 + out_slot2;
            src_global[e_base + eh] = u;
            agg_dst[e_base + eh] = i;
            eslot[eh] = map_insert_min(map, mask, u, kNewBase + eh, ctl);
        }
    }
}

__global__ void __launch_bounds__(kScanThreads)
hop_flag_kernel(const int32_t *__restrict__ eslot, const MapSlot *map, int32_t *erank, int32_t *tile_sum,
                int32_t *tile_off, int32_t *ctl, int64_t max_nodes)
{
    pdl_wait();
    pdl_trigger();
    __shared__ int smem[kScanThreads / 32];
    __shared__ int s_flag;
    const int n_edges = ctl[CTL_E_HOP];
    const int n_tiles = (n_edges + kTile - 1) / kTile;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const int base = tile * kTile + threadIdx.x * 4;
        int4 s4 = *reinterpret_cast<const int4 *>(eslot + base);  // eslot is padded to a whole tile
        int32_t s[4] = { s4.x, s4.y, s4.z, s4.w };
        int f[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            f[j] = 0;
            if (base + j < n_edges) f[j] = (__ldcg(&map[s[j]].val) == kNewBase + base + j) ? 1 : 0;
        }
        int total;
        int ex = block_excl_scan(f[0] + f[1] + f[2] + f[3], &total, smem);
        int4 out;
        out.x = f[0] ? ex : -1; ex += f[0];
        out.y = f[1] ? ex : -1; ex += f[1];
        out.z = f[2] ? ex : -1; ex += f[2];
        out.w = f[3] ? ex : -1;
        *reinterpret_cast<int4 *>(erank + base) = out;  // erank is padded to a whole tile
        if (threadIdx.x == 0) tile_sum[tile] = total;
    }
    int grand;
    if (last_cta_scan(&ctl[CTL_TICKET_B], tile_sum, tile_off, n_tiles, smem, &s_flag, &grand)) {
        if (threadIdx.x == 0) {
            ctl[CTL_C_HOP] = grand;
            if ((int64_t)ctl[CTL_N_NODES] + grand > max_nodes) atomicCAS(&ctl[CTL_ERROR], DERR_NONE, DERR_NODE_OVERFLOW);
        }
    }
}

// New nodes get their local ids (order of first appearance: rank of the flagged edge) and every edge of
// the hop is relabelled, in one pass.  The local id of a node whose first edge is fe is
// n0 + tile_off[fe / tile] + erank[fe], which every edge can compute for itself once the flags are
// scanned; the map entry is rewritten to that id by the first edge, and an edge that reads the entry
// after the rewrite finds the same number.  The last CTA advances the counters.
__global__ void hop_finish_kernel(const int32_t *__restrict__ erank, const int32_t *__restrict__ tile_off,
                                  const int32_t *__restrict__ eslot, const int32_t *__restrict__ src_global,
                                  int32_t *ids, MapSlot *map, int32_t *agg_src, int32_t *ctl, int32_t *nc, int32_t *ec,
                                  int op_id, const BatchCtl *__restrict__ b, int last_hop)
{
    pdl_wait();
    pdl_trigger();
    __shared__ int s_flag;
    const int n_edges = ctl[CTL_E_HOP];
    const int n0 = ctl[CTL_N_NODES];
    const int e_base = ctl[CTL_E_TOTAL];
    const int c_hop = ctl[CTL_C_HOP];
    const bool ok = ctl[CTL_ERROR] == DERR_NONE;
    if (ok) {
        for (int eh = blockIdx.x * blockDim.x + threadIdx.x; eh < n_edges; eh += gridDim.x * blockDim.x) {
            const int slot = eslot[eh];
            const int r = erank[eh];
            int local;
            if (r >= 0) {
                local = n0 + tile_off[eh >> 10] + r;
                ids[local] = src_global[e_base + eh];
                map[slot].val = local;
            } else {
                local = __ldcg(&map[slot].val);
                if (local >= kNewBase) {
                    const int fe = local - kNewBase;
                    local = n0 + tile_off[fe >> 10] + erank[fe];
                }
            }
            agg_src[e_base + eh] = local;
        }
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        int t = atomicAdd(&ctl[CTL_TICKET_C], 1);
        s_flag = (t == (int)gridDim.x - 1);
    }
    __syncthreads();
    if (s_flag && threadIdx.x == 0) {
        // every other CTA has read ctl by now
        int c = ok ? c_hop : 0;
        int e = ok ? n_edges : 0;
        nc[LEGION_INTRABATCH_CON * 2] += c;  // operator_impl.cu:281
        ec[2] += e;                          // operator_impl.cu:282
        counter_update(nc, ec, op_id, 0, 0);
        ctl[CTL_N_NODES] = n0 + c;
        ctl[CTL_E_TOTAL] = e_base + e;
        ctl[CTL_E_HOP] = 0;
        ctl[CTL_C_HOP] = 0;
        ctl[CTL_TICKET_C] = 0;
    }
    // After the last hop both counter arrays also go to page-locked host memory (one posted store per thread of
    // a warp): the host learns the sizes of the batch without a copy-engine transfer queued behind other batches'
    // exports.  s_flag is the same for every thread of the CTA.
    int32_t *host_mirror = last_hop ? b->mirror : nullptr;
    if (s_flag && host_mirror != nullptr) {
        __syncthreads();
        if (threadIdx.x < 32) {
            host_mirror[threadIdx.x] = threadIdx.x < 16 ? nc[threadIdx.x] : ec[threadIdx.x - 16];
            __threadfence_system();
        }
    }
}

// ---- launchers -----------------------------------------------------------------------------------

// 1: the kernels of a batch after its first are launched as programmatic dependents (legion_set_tunable
// "pdl"; start value from the environment variable LEGION_PDL)
static int pdl_from_env()
{
    const char *v = getenv("LEGION_PDL");
    return (v != nullptr && v[0] == '1' && v[1] == 0) ? 1 : 0;
}
int g_pdl = pdl_from_env();
// front region of the id map = worst-case slots >> this; -1: sized by legion_pool_create's own rule
// (legion_set_tunable "map_front_shift")
int g_map_front_shift = -1;

template <typename... KArgs, typename... Args>
static cudaError_t launch_dep(void (*kernel)(KArgs...), int grid, int block, cudaStream_t s, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3((unsigned)block);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = g_pdl ? at : nullptr;
    cfg.numAttrs = g_pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

static inline int grid_for(int64_t items, int per_cta, int cap)
{
    int64_t g = (items + per_cta - 1) / per_cta;
    if (g < 1) g = 1;
    if (g > cap) g = cap;
    return (int)g;
}

const void *map_clear_kernel_address() { return (const void *)map_clear_kernel; }

BatchCtl make_batch_ctl(const LegionPool *p, const LegionCache *c, const int32_t *all_ids, const int32_t *all_labels,
                        int32_t total_cap, int64_t first, int32_t size, int64_t n_nodes)
{
    BatchCtl v;
    v.all_ids = all_ids;
    v.all_labels = all_labels;
    v.first = first;
    v.total_cap = total_cap;
    v.size = size;
    v.hop_num = p->hop_num;
    v.global_batch = p->global_batch;
    v.k0 = (uint32_t)p->rng_seed;
    v.k1 = (uint32_t)(p->rng_seed >> 32);
    v.max_rounds = p->max_rounds;
    v.clock = (c != nullptr && c->kind == 1) ? c->clock : 0;
    v.n_nodes = (n_nodes > 0 && n_nodes < 0x7FFFFFFF) ? (int32_t)n_nodes : 0x7FFFFFFF;
    // two mirrors per pipe when batches are sampled ahead of the hand-off: the next batch on the pipe may finish its
    // sampling before the host has read the counters of the one before
    v.mirror = p->h_stage[p->pipe] + 2 * (size_t)p->batch_size + 32 +
               (p->slots < p->pipes ? 32 * (p->mirror_flip[p->pipe] & 1) : 0);
    return v;
}

// defer_seeds: only the first kernel (map, counters, batch parameters) is issued; the seed slice is then
// taken by the first hop (launch_sample_hop with seeds_pending), one launch fewer per batch.
int launch_batch_generate(cudaStream_t s, LegionPool *p, const BatchCtl &v, bool defer_seeds)
{
    const int pipe = p->pipe;
    const int64_t n_pairs = ((int64_t)p->map_front_mask + 1) / 2;
    const int64_t back_pairs = ((int64_t)p->map_mask + 1) / 2;
    // sized for the front region; when the back region has to be cleared too, the CTAs loop longer
    map_clear_kernel<<<grid_for(n_pairs, 256 * 4, p->sm_count * 8), 256, 0, s>>>(
        reinterpret_cast<uint4 *>(p->map[pipe]), n_pairs, p->ctl[pipe], p->node_counter[pipe], p->edge_counter[pipe],
        p->bctl[pipe], v, back_pairs);
    LG_LAUNCH_CHECK();
    if (defer_seeds) return LEGION_OK;
    LG_CUDA(launch_dep(batch_generate_kernel, grid_for(p->batch_size, 256, 1 << 20), 256, s, p->bctl[pipe], p->ids[pipe],
                       p->labels[pipe], p->map[pipe], MapDims{ p->map_front_mask, p->map_mask }, p->ctl[pipe], p->node_counter[pipe],
                       p->edge_counter[pipe]));
    return LEGION_OK;
}

int launch_sample_hop(cudaStream_t s, LegionPool *p, const LegionGraph *g, int32_t fanout, int32_t hop,
                      int32_t op_id, bool seeds_pending)
{
    const int pipe = p->pipe;
    const int cap = p->sm_count * 8;
    // worst-case sizes of this hop: inputs = all nodes so far, edges = inputs * fanout
    int64_t inputs = p->batch_size;
    for (int h = 0; h < hop; ++h) inputs += inputs * p->fanout[h];
    int64_t edges = inputs * fanout;
    int32_t *ctl = p->ctl[pipe];
    if (seeds_pending) {
        LG_ARG(hop == 0, "only the first hop can take the seed slice");
        LG_CUDA(launch_dep(hop_count_kernel<true>, grid_for(inputs, kScanThreads, cap), kScanThreads, s, g->indptr,
                           p->ids[pipe], fanout, p->node_rec[pipe], p->tile_sum[pipe], p->tile_off[pipe], ctl, p->max_edges,
                           p->bctl[pipe], p->labels[pipe], p->map[pipe], MapDims{ p->map_front_mask, p->map_mask }, p->node_counter[pipe],
                           p->edge_counter[pipe]));
    } else {
        LG_CUDA(launch_dep(hop_count_kernel<false>, grid_for(inputs, kTile, cap), kScanThreads, s, g->indptr, p->ids[pipe],
                           fanout, p->node_rec[pipe], p->tile_sum[pipe], p->tile_off[pipe], ctl, p->max_edges, p->bctl[pipe],
                           p->labels[pipe], p->map[pipe], MapDims{ p->map_front_mask, p->map_mask }, p->node_counter[pipe], p->edge_counter[pipe]));
    }
    LG_CUDA(launch_dep(hop_sample_kernel, grid_for(inputs, 8, cap), 256, s, g->indices, p->node_rec[pipe], p->tile_off[pipe],
                       fanout, (uint32_t)hop, p->bctl[pipe], p->src_global[pipe], p->agg_dst[pipe], p->eslot[pipe],
                       p->map[pipe], MapDims{ p->map_front_mask, p->map_mask }, ctl, seeds_pending ? 8 : 10,
                       p->node_counter[pipe], p->edge_cnt[pipe]));
    static_assert(kScanThreads == 256 && kTile == 1024, "tile shifts above assume 256-thread scans over 1024-item tiles");
    int32_t *tile_sum2 = p->tile_sum[pipe] + p->input_tiles;
    int32_t *tile_off2 = p->tile_off[pipe] + p->input_tiles;
    LG_CUDA(launch_dep(hop_flag_kernel, grid_for(edges, kTile, cap), kScanThreads, s, p->eslot[pipe], p->map[pipe],
                       p->erank[pipe], tile_sum2, tile_off2, ctl, p->max_nodes));
    LG_CUDA(launch_dep(hop_finish_kernel, grid_for(edges, 256 * 4, cap), 256, s, p->erank[pipe], tile_off2, p->eslot[pipe],
                       p->src_global[pipe], p->ids[pipe], p->map[pipe], p->agg_src[pipe], ctl, p->node_counter[pipe],
                       p->edge_counter[pipe], op_id, p->bctl[pipe], hop + 1 == p->hop_num ? 1 : 0));
    return LEGION_OK;
}

// ---- hand-off of a batch that was sampled ahead ------------------------------------------------------------------
// A pool with fewer hand-off slots than pipes samples into private buffers; when the batch's turn comes, its
// block structure (ids, labels, both edge lists, both counter arrays: ~3 MB for a paper100M-shaped batch) is
// copied into the slot that the consumer reads (the buffers of engine/ipc_service.cu:163-169).  Sizes are read
// from the counters on the device.
__global__ void __launch_bounds__(256)
publish_kernel(const int32_t *__restrict__ ids, const int32_t *__restrict__ labels, const int32_t *__restrict__ src,
               const int32_t *__restrict__ dst, const int32_t *__restrict__ nc, const int32_t *__restrict__ ec,
               int32_t *o_ids, int32_t *o_labels, int32_t *o_src, int32_t *o_dst, int32_t *o_nc, int32_t *o_ec)
{
    const int hops = nc[LEGION_INTRABATCH_CON * 3 - 1];
    const int n = nc[LEGION_INTRABATCH_CON * 3 + hops];
    const int n_lab = nc[LEGION_INTRABATCH_CON * 3];
    const int e = ec[0] + ec[1];
    const int tid = blockIdx.x * blockDim.x + threadIdx.x, step = gridDim.x * blockDim.x;
    // every array is padded to whole 1024-element tiles, so whole 16-byte vectors may be copied
    for (int i = tid; i * 4 < n; i += step) reinterpret_cast<int4 *>(o_ids)[i] = reinterpret_cast<const int4 *>(ids)[i];
    for (int i = tid; i * 4 < e; i += step) {
        reinterpret_cast<int4 *>(o_src)[i] = reinterpret_cast<const int4 *>(src)[i];
        reinterpret_cast<int4 *>(o_dst)[i] = reinterpret_cast<const int4 *>(dst)[i];
    }
    for (int i = tid; i < n_lab; i += step) o_labels[i] = labels[i];
    if (blockIdx.x == 0 && threadIdx.x < 16) {
        o_nc[threadIdx.x] = nc[threadIdx.x];
        o_ec[threadIdx.x] = ec[threadIdx.x];
    }
}

int launch_publish(cudaStream_t s, LegionPool *p)
{
    if (p->slots == p->pipes) return LEGION_OK;  // the pipe's buffers are the hand-off buffers
    const int pipe = p->pipe, slot = pipe % p->slots;
    publish_kernel<<<p->sm_count * 2, 256, 0, s>>>(p->ids[pipe], p->labels[pipe], p->agg_src[pipe], p->agg_dst[pipe],
                                                   p->node_counter[pipe], p->edge_counter[pipe], p->pub_ids[slot],
                                                   p->pub_labels[slot], p->pub_agg_src[slot], p->pub_agg_dst[slot],
                                                   p->pub_nc[slot], p->pub_ec[slot]);
    LG_LAUNCH_CHECK();
    return LEGION_OK;
}

}  // namespace legion
