/*
 * legion_oracle.c -- CPU restatement of the Legion sampling-server hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker for the CUDA library; it is
 * never linked into, imported by or called from the product.  Only tests, the smoke
 * check and the CPU-baseline leg of the benchmark may load it.
 *
 * Parity status: the reference keeps no golden vectors or known-answer tests for this
 * path and its own implementation is CUDA-only and does not compile without an
 * un-vendored dependency, so the structural parts below are pinned only by the
 * reference's self-consistency rules (gathered rows are bit copies of the source rows,
 * the counter layout the trainer parses).  "parity unpinned" applies to: the sampler's
 * random stream (redefined here as Philox4x32-10, pinned against the published
 * Random123 known-answer vectors) and to the bit-packing compression of the missing
 * IBP library (replaced by int8 / fp8 per-row absmax quantisation defined here).
 *
 * Every function cites the reference file:line (paths relative to the reference's
 * root) whose behaviour it restates.
 *
 * Build: gcc -O2 -fopenmp -shared -fPIC legion_oracle.c -o liblegion_oracle.so
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <math.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_MAX_FANOUT 32
#define ORC_MAX_HOPS 3
#define ORC_INTRABATCH_CON 3 /* sampling_server/src/include/system_config.cuh:48 */
#define ORC_CACHEMISS_FLAG (-2) /* system_config.cuh:56 */

/* ------------------------------------------------------------------------------------
 * Philox4x32-10 (Salmon et al., SC'11; Random123).  The reference seeds nothing
 * (thrust::minstd_rand with the default seed, operator_impl.cu:244-246); the counter
 * RNG replaces it so that a host replay is possible.
 * ---------------------------------------------------------------------------------- */
void orc_philox4x32_10(const uint32_t ctr[4], const uint32_t key[2], uint32_t out[4])
{
    uint32_t c0 = ctr[0], c1 = ctr[1], c2 = ctr[2], c3 = ctr[3];
    uint32_t k0 = key[0], k1 = key[1];
    for (int r = 0; r < 10; ++r) {
        uint64_t p0 = (uint64_t)0xD2511F53u * c0;
        uint64_t p1 = (uint64_t)0xCD9E8D57u * c2;
        uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0;
        uint32_t n1 = (uint32_t)p1;
        uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1;
        uint32_t n3 = (uint32_t)p0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

/* One bounded draw in [0, n): 64 random bits times n, high half. */
static inline uint32_t orc_draw(uint32_t input_index, uint32_t lane, uint32_t round,
                                uint32_t hop, uint32_t batch_id, uint64_t seed, uint32_t n)
{
    uint32_t ctr[4] = { input_index, round * 32u + lane, hop, batch_id };
    uint32_t key[2] = { (uint32_t)seed, (uint32_t)(seed >> 32) };
    uint32_t w[4];
    orc_philox4x32_10(ctr, key, w);
    uint64_t r64 = ((uint64_t)w[1] << 32) | w[0];
    return (uint32_t)(((unsigned __int128)r64 * (unsigned __int128)n) >> 64);
}

/*
 * m distinct values from [0, n), m <= 32 < n, as a lock-step replay of one warp:
 * in every round all lanes that still need a value draw one; a lane keeps its value
 * unless a lane that already held that value, or a lower lane that drew it in the same
 * round, exists.  The procedure only depends on the equality pattern of the draws, so
 * the resulting set is uniform over the m-subsets.  After max_rounds rounds the
 * remaining lanes are settled in lane order by stepping to the next free value.
 * Replaces the reference's <=10 rounds of __match_any_sync rejection that lets
 * duplicates survive (operator_impl.cu:247-258).
 */
static void orc_draw_distinct(uint32_t m, uint32_t n, uint32_t input_index, uint32_t hop,
                              uint32_t batch_id, uint64_t seed, int max_rounds, uint32_t x[32])
{
    int kept[32];
    for (uint32_t l = 0; l < m; ++l) kept[l] = 0;
    uint32_t pending = m;
    if (max_rounds < 1) max_rounds = 1; /* every lane draws at least once */
    for (int r = 0; r < max_rounds && pending; ++r) {
        int pre[32];
        for (uint32_t l = 0; l < m; ++l) {
            pre[l] = kept[l];
            if (!kept[l]) x[l] = orc_draw(input_index, l, (uint32_t)r, hop, batch_id, seed, n);
        }
        for (uint32_t l = 0; l < m; ++l) {
            if (pre[l]) continue;
            int ok = 1;
            for (uint32_t j = 0; j < m && ok; ++j) {
                if (j == l || x[j] != x[l]) continue;
                if (pre[j] || j < l) ok = 0;
            }
            if (ok) { kept[l] = 1; --pending; }
        }
    }
    for (uint32_t l = 0; l < m && pending; ++l) {
        if (kept[l]) continue;
        uint32_t cand = x[l];
        for (;;) {
            int clash = 0;
            for (uint32_t j = 0; j < m; ++j)
                if (kept[j] && x[j] == cand) { clash = 1; break; }
            if (!clash) break;
            cand = (cand + 1u) % n;
        }
        x[l] = cand; kept[l] = 1; --pending;
    }
}

/*
 * One hop of neighbour sampling for every node found so far (the reference samples all
 * of sampled_ids[0 .. nc[0]+nc[1]) again on every hop, operator_impl.cu:205-213).
 * deg <= fanout keeps the whole adjacency list in CSR order (operator_impl.cu:241-242);
 * otherwise `fanout` distinct positions are drawn: directly when deg >= 2*fanout, and by
 * drawing the deg-fanout positions to leave out when deg < 2*fanout (survivors in CSR
 * order).  Edges are laid out input after input, without gaps (the reference appends them
 * in atomic arrival order, operator_impl.cu:272-296; the order is fixed here so that blocks
 * can be compared bit for bit).  src = sampled neighbour (global id), dst = index of the
 * input node in `ids`, which is its local id (operator_impl.cu:274-275,304-317).
 * Returns the number of edges written.  ids < 0 produce nothing (operator_impl.cu:222).
 */
int64_t orc_sample_hop(const int64_t *indptr, const int32_t *indices, const int32_t *ids,
                       int32_t n_inputs, int32_t fanout, int32_t hop, uint32_t batch_id,
                       uint64_t seed, int32_t max_rounds, int32_t *src_global,
                       int32_t *dst_local)
{
    int64_t e = 0;
    if (fanout > ORC_MAX_FANOUT) return -1; /* operator_impl.cu:504 */
    for (int32_t i = 0; i < n_inputs; ++i) {
        int32_t v = ids[i];
        if (v < 0) continue;
        int64_t start = indptr[v];
        int64_t deg64 = indptr[v + 1] - start;
        uint32_t deg = (uint32_t)deg64;
        uint32_t k = (uint32_t)fanout;
        if (deg <= k) {
            for (uint32_t j = 0; j < deg; ++j) {
                src_global[e] = indices[start + j];
                dst_local[e] = i;
                ++e;
            }
        } else if (deg >= 2 * k) {
            uint32_t x[32];
            orc_draw_distinct(k, deg, (uint32_t)i, (uint32_t)hop, batch_id, seed, max_rounds, x);
            for (uint32_t j = 0; j < k; ++j) {
                src_global[e] = indices[start + x[j]];
                dst_local[e] = i;
                ++e;
            }
        } else {
            uint32_t x[32];
            uint32_t m = deg - k;
            uint64_t excl = 0;
            orc_draw_distinct(m, deg, (uint32_t)i, (uint32_t)hop, batch_id, seed, max_rounds, x);
            for (uint32_t j = 0; j < m; ++j) excl |= (uint64_t)1 << x[j];
            for (uint32_t p = 0; p < deg; ++p) {
                if ((excl >> p) & 1u) continue;
                src_global[e] = indices[start + p];
                dst_local[e] = i;
                ++e;
            }
        }
    }
    return e;
}

/* ------------------------------------------------------------------------------------
 * Batch-local id map (stands for accessed_map + position_map of the reference,
 * operator_impl.cu:45-50,265-271,289-290; O(batch) instead of O(N)).
 * ---------------------------------------------------------------------------------- */
typedef struct {
    int32_t *keys;
    int32_t *vals;
    uint32_t mask;
} orc_map;

static uint32_t orc_mix(uint32_t h)
{
    h ^= h >> 16; h *= 0x85EBCA6Bu; h ^= h >> 13; h *= 0xC2B2AE35u; h ^= h >> 16;
    return h;
}

static int orc_map_init(orc_map *m, int64_t max_items)
{
    uint32_t cap = 16;
    while ((int64_t)cap < max_items * 2) cap <<= 1;
    m->keys = (int32_t *)malloc(sizeof(int32_t) * cap);
    m->vals = (int32_t *)malloc(sizeof(int32_t) * cap);
    if (!m->keys || !m->vals) return -1;
    memset(m->keys, 0xFF, sizeof(int32_t) * cap);
    m->mask = cap - 1;
    return 0;
}

static void orc_map_free(orc_map *m) { free(m->keys); free(m->vals); }

/* returns the value stored for key, inserting (key -> val_if_new) when absent */
static inline int32_t orc_map_get_or_put(orc_map *m, int32_t key, int32_t val_if_new, int *was_new)
{
    uint32_t s = orc_mix((uint32_t)key) & m->mask;
    for (;;) {
        int32_t k = m->keys[s];
        if (k == key) { *was_new = 0; return m->vals[s]; }
        if (k == -1) { m->keys[s] = key; m->vals[s] = val_if_new; *was_new = 1; return val_if_new; }
        s = (s + 1) & m->mask;
    }
}

/*
 * Literal restatement of the 1-thread bookkeeping kernel, operator_impl.cu:58-91.
 */
void orc_counter_update(int32_t *nc, int32_t *ec, int32_t op_id, int32_t size, int32_t hop_num)
{
    const int C = ORC_INTRABATCH_CON;
    if (op_id == 0) {
        nc[0] = 0;
        nc[1] = size;
        nc[C * 3 + (op_id / C)] = nc[0] + nc[1];
        nc[C * 3 - 1] = hop_num;
    } else if (op_id > 0 && op_id % C == 0) {
        nc[0] = nc[0] + nc[1];
        nc[1] = nc[C * 2];
        nc[C * 2] = 0;
        nc[C * 2 + 1] = nc[0] + nc[1];
        ec[0] = ec[0] + ec[1];
        ec[1] = ec[2];
        ec[2] = 0;
        nc[C * 3 + (op_id / C)] = nc[0] + nc[1];
        ec[C * 3 + (op_id / C)] = ec[1];
        ec[C * 4 + (op_id / C)] = ec[0];
    } else if (op_id % C > 0) {
        nc[(op_id % C) * 2] = nc[0];
        nc[(op_id % C) * 2 + 1] = nc[1];
    }
}

/*
 * One whole mini-batch: BatchGenerate -> (RandomSample -> construct_graph)*hops, with
 * the operator order of GPURunner (server.cu:218-228,342-351) and the counter trace it
 * produces.  Seeds are the slice [batch_size*iter, +size) of this GPU's seed list, the
 * tail batch being shortened (operator_impl.cu:162).  New nodes are appended to `ids` in
 * order of first appearance in the hop's edge list; local ids are positions in `ids`
 * (operator_impl.cu:285-291,304-317).  Outputs have the layout the trainer reads
 * (training_backend/ipc_cuda_kernel.cu:194-240).
 * Returns the total node count, or <0 on error.
 */
int64_t orc_run_batch(const int64_t *indptr, const int32_t *indices,
                      const int32_t *all_ids, const int32_t *all_labels, int32_t total_cap,
                      int32_t batch_size, int32_t iter, int32_t hop_num, const int32_t *fanout,
                      uint32_t batch_id, uint64_t seed, int32_t max_rounds,
                      int32_t *ids, int32_t *labels, int32_t *agg_src, int32_t *agg_dst,
                      int32_t *src_global_scratch, int32_t *node_counter, int32_t *edge_counter)
{
    if (hop_num > ORC_MAX_HOPS) return -1;
    memset(node_counter, 0, 16 * sizeof(int32_t)); /* operator_impl.cu:158-159 */
    memset(edge_counter, 0, 16 * sizeof(int32_t));
    int64_t first = (int64_t)batch_size * iter;
    int32_t size = ((int64_t)batch_size * (iter + 1) >= total_cap) ? (int32_t)(total_cap - first)
                                                                  : batch_size;
    if (size < 0) size = 0;
    int64_t bound = size;
    {
        int64_t cur = size;
        for (int h = 0; h < hop_num; ++h) { cur = cur + cur * fanout[h]; }
        bound = cur;
    }
    orc_map map;
    if (orc_map_init(&map, bound + 1) != 0) return -2;
    for (int32_t i = 0; i < size; ++i) { /* batch_generate, operator_impl.cu:28-56 */
        int32_t sid = all_ids[(first + i) % total_cap];
        int was_new;
        ids[i] = sid;
        labels[i] = all_labels[(first + i) % total_cap];
        orc_map_get_or_put(&map, sid, i, &was_new);
    }
    orc_counter_update(node_counter, edge_counter, 0, size, hop_num);
    orc_counter_update(node_counter, edge_counter, 1, 0, 0); /* op1: gather of the seeds */
    int32_t n_nodes = size;
    int64_t e_base = 0;
    for (int h = 0; h < hop_num; ++h) {
        int32_t op_id = ORC_INTRABATCH_CON * (h + 1);
        int32_t n_inputs = node_counter[0] + node_counter[1];
        int64_t e_h = orc_sample_hop(indptr, indices, ids, n_inputs, fanout[h], h, batch_id, seed,
                                     max_rounds, src_global_scratch + e_base, agg_dst + e_base);
        if (e_h < 0) { orc_map_free(&map); return -3; }
        int32_t n_before = n_nodes;
        for (int64_t e = 0; e < e_h; ++e) {
            int was_new;
            int32_t u = src_global_scratch[e_base + e];
            int32_t loc = orc_map_get_or_put(&map, u, n_nodes, &was_new);
            if (was_new) ids[n_nodes++] = u;
            agg_src[e_base + e] = loc;
        }
        node_counter[ORC_INTRABATCH_CON * 2] += n_nodes - n_before; /* operator_impl.cu:281 */
        edge_counter[2] += (int32_t)e_h;                              /* operator_impl.cu:282 */
        orc_counter_update(node_counter, edge_counter, op_id, 0, 0);
        orc_counter_update(node_counter, edge_counter, op_id + 1, 0, 0);
        e_base += e_h;
    }
    orc_map_free(&map);
    return n_nodes;
}

/* ------------------------------------------------------------------------------------
 * Static cache placement and lookup.
 * ---------------------------------------------------------------------------------- */

/* Descending-degree order, ties by ascending id.  Stands for the hotness order QF of
 * CandidateSelection (cache.cu:405-440: sort_by_key descending); degree replaces the
 * presampled hotness as the sort key. */
typedef struct { int64_t deg; int32_t id; } orc_deg_id;
static int orc_cmp_deg(const void *a, const void *b)
{
    const orc_deg_id *x = (const orc_deg_id *)a, *y = (const orc_deg_id *)b;
    if (x->deg != y->deg) return (x->deg > y->deg) ? -1 : 1;
    return (x->id < y->id) ? -1 : (x->id > y->id);
}
int orc_degree_order(const int64_t *indptr, int32_t n, int32_t *order)
{
    orc_deg_id *t = (orc_deg_id *)malloc(sizeof(orc_deg_id) * (size_t)n);
    if (!t) return -1;
    for (int32_t i = 0; i < n; ++i) { t[i].deg = indptr[i + 1] - indptr[i]; t[i].id = i; }
    qsort(t, (size_t)n, sizeof(orc_deg_id), orc_cmp_deg);
    for (int32_t i = 0; i < n; ++i) order[i] = t[i].id;
    free(t);
    return 0;
}

/* Interleaved placement of the first capacity*kg ranked nodes: rank t lives on GPU t % kg
 * at row t / kg, global index (t % kg) * capacity + t / kg (cache_impl.cuh:104-109);
 * every other node maps to CACHEMISS_FLAG.  `lut` has one entry per node and stands for
 * the bcht lookup (cache.cu:157-192). */
void orc_static_cache_lut(const int32_t *order, int32_t n, int32_t capacity, int32_t kg, int32_t *lut)
{
    for (int32_t i = 0; i < n; ++i) lut[i] = ORC_CACHEMISS_FLAG;
    int64_t cached = (int64_t)capacity * kg;
    if (cached > n) cached = n;
    for (int64_t t = 0; t < cached; ++t)
        lut[order[t]] = (int32_t)((t % kg) * (int64_t)capacity + t / kg);
}

/* Rows held by GPU ki: row s <- host row order[s*kg + ki] (FeatFillUp, cache_impl.cuh:183-188).
 * Rows past the end of the ranking stay untouched. */
void orc_static_cache_fill(const int32_t *order, int32_t n, int32_t capacity, int32_t kg, int32_t ki,
                           const uint8_t *host_table, int64_t row_bytes, uint8_t *cache_rows)
{
    for (int64_t s = 0; s < capacity; ++s) {
        int64_t t = s * kg + ki;
        if (t >= n) break;
        memcpy(cache_rows + s * row_bytes, host_table + (int64_t)order[t] * row_bytes, (size_t)row_bytes);
    }
}

/* FindFeat: cache_index[r] = lut[id] (cache.cu:157-192,314-338); ids < 0 are misses. */
void orc_find_feat(const int32_t *ids, int64_t n, const int32_t *lut, int32_t *cache_index)
{
    for (int64_t r = 0; r < n; ++r) cache_index[r] = ids[r] < 0 ? ORC_CACHEMISS_FLAG : lut[ids[r]];
}

/* The gather (multiGPU_feat_cache_lookup, cache_impl.cuh:239-303): row r comes from
 * partition gidx / capacity at row gidx % capacity when gidx >= 0, else from the host
 * table at (id % total_nodes); rows with id < 0 are left untouched.  Rows are copied as
 * opaque bytes. */
void orc_gather(const int32_t *ids, const int32_t *cache_index, int64_t n, int32_t capacity,
                const uint8_t *const *parts, const uint8_t *host_table, int64_t total_nodes,
                int64_t row_bytes, uint8_t *dst)
{
    for (int64_t r = 0; r < n; ++r) {
        int32_t g = cache_index[r];
        if (g < 0) {
            int32_t id = ids[r];
            if (id >= 0)
                memcpy(dst + r * row_bytes, host_table + ((int64_t)id % total_nodes) * row_bytes,
                       (size_t)row_bytes);
        } else {
            memcpy(dst + r * row_bytes, parts[g / capacity] + (int64_t)(g % capacity) * row_bytes,
                   (size_t)row_bytes);
        }
    }
}

/* ------------------------------------------------------------------------------------
 * Compressed rows: int8 / fp8(e4m3) with one fp32 scale per row.  This replaces the
 * lossless bit-packing of the absent IBP library (compress_cache_kernel.cuh:584-693
 * shows the call sites only).  Every step is a single IEEE operation so that host and
 * device agree bit for bit.
 *   int8 : inv = 127 / absmax ; q = rint(x * inv) clamped to +-127 ; scale = absmax / 127
 *   e4m3 : inv = 448 / absmax ; q = e4m3(x * inv) (nearest even, saturating) ; scale = absmax / 448
 *   x^ = float(q) * scale.   absmax == 0 -> q = 0, scale = 0.
 * A stored row is row_q = F code bytes followed by the 4-byte scale, padded to 16 bytes.
 * ---------------------------------------------------------------------------------- */
static float orc_absmax(const float *x, int32_t f)
{
    float a = 0.0f;
    for (int32_t i = 0; i < f; ++i) { float v = fabsf(x[i]); if (v > a) a = v; }
    return a;
}

int64_t orc_quant_row_bytes(int32_t f) { return ((int64_t)f + 4 + 15) / 16 * 16; }

void orc_quant_int8_row(const float *x, int32_t f, uint8_t *row)
{
    float a = orc_absmax(x, f);
    float inv = a > 0.0f ? 127.0f / a : 0.0f;
    float scale = a / 127.0f;
    volatile float prod;
    for (int32_t i = 0; i < f; ++i) {
        prod = x[i] * inv;
        float r = nearbyintf(prod);
        if (r > 127.0f) r = 127.0f;
        if (r < -127.0f) r = -127.0f;
        ((int8_t *)row)[i] = (int8_t)(int)r;
    }
    memcpy(row + f, &scale, 4);
    for (int64_t i = f + 4; i < orc_quant_row_bytes(f); ++i) row[i] = 0;
}

void orc_dequant_int8_row(const uint8_t *row, int32_t f, float *out)
{
    float scale;
    memcpy(&scale, row + f, 4);
    for (int32_t i = 0; i < f; ++i) out[i] = (float)((const int8_t *)row)[i] * scale;
}

/* e4m3 (1-4-3, bias 7, no infinities, max 448) decode */
float orc_e4m3_to_float(uint8_t b)
{
    int s = b >> 7, e = (b >> 3) & 15, m = b & 7;
    float v;
    if (e == 15 && m == 7) v = NAN;
    else if (e == 0) v = ldexpf((float)m, -9);
    else v = ldexpf((float)(8 + m), e - 10);
    return s ? -v : v;
}

/* fp32 -> e4m3, round to nearest even, saturating to +-448, NaN -> 0x7f */
uint8_t orc_float_to_e4m3(float x)
{
    uint32_t u;
    memcpy(&u, &x, 4);
    uint8_t sign = (uint8_t)((u >> 24) & 0x80);
    float a = fabsf(x);
    if (a != a) return (uint8_t)(sign | 0x7F);
    if (a >= 448.0f) {
        /* values above 448 (incl. the tie 464 and infinity) saturate to 448 */
        return (uint8_t)(sign | 0x7E);
    }
    if (a < ldexpf(1.0f, -10)) {
        /* below half of the smallest subnormal 2^-9: the tie 2^-10 goes to even (0) */
        return sign;
    }
    int e;
    (void)frexpf(a, &e); /* a = f * 2^e, f in [0.5,1) -> unbiased exponent e-1 */
    int ue = e - 1;
    if (ue < -6) ue = -6; /* subnormal range shares the exponent of the smallest normal */
    /* quantum = 2^(ue-3); q = a / quantum rounded to nearest even */
    float q = ldexpf(a, 3 - ue);
    float r = nearbyintf(q); /* default rounding mode: nearest even */
    int qi = (int)r;
    if (ue == -6 && qi < 8) return (uint8_t)(sign | qi); /* subnormal */
    if (qi == 16) { qi = 8; ue += 1; }
    int be = ue + 7;
    if (be > 15 || (be == 15 && qi - 8 > 6)) return (uint8_t)(sign | 0x7E);
    return (uint8_t)(sign | (be << 3) | (qi - 8));
}

void orc_quant_e4m3_row(const float *x, int32_t f, uint8_t *row)
{
    float a = orc_absmax(x, f);
    float inv = a > 0.0f ? 448.0f / a : 0.0f;
    float scale = a / 448.0f;
    volatile float prod;
    for (int32_t i = 0; i < f; ++i) {
        prod = x[i] * inv;
        row[i] = orc_float_to_e4m3(prod);
    }
    memcpy(row + f, &scale, 4);
    for (int64_t i = f + 4; i < orc_quant_row_bytes(f); ++i) row[i] = 0;
}

void orc_dequant_e4m3_row(const uint8_t *row, int32_t f, float *out)
{
    float scale;
    memcpy(&scale, row + f, 4);
    for (int32_t i = 0; i < f; ++i) out[i] = orc_e4m3_to_float(row[i]) * scale;
}

/* Gather over a compressed cache: hits are dequantised from the partition's packed rows,
 * misses are raw fp32 rows of the host table.  codec: 1 = int8, 2 = e4m3. */
void orc_gather_quant(const int32_t *ids, const int32_t *cache_index, int64_t n, int32_t capacity,
                      const uint8_t *const *parts, const float *host_table, int64_t total_nodes,
                      int32_t f, int32_t codec, float *dst)
{
    int64_t rq = orc_quant_row_bytes(f);
    for (int64_t r = 0; r < n; ++r) {
        int32_t g = cache_index[r];
        if (g < 0) {
            int32_t id = ids[r];
            if (id >= 0)
                memcpy(dst + r * f, host_table + ((int64_t)id % total_nodes) * f, sizeof(float) * (size_t)f);
        } else {
            const uint8_t *row = parts[g / capacity] + (int64_t)(g % capacity) * rq;
            if (codec == 1) orc_dequant_int8_row(row, f, dst + r * f);
            else orc_dequant_e4m3_row(row, f, dst + r * f);
        }
    }
}

/* ------------------------------------------------------------------------------------
 * Set-associative cache with LRU replacement.  Addressing is the reference's
 * (static_cache_kernel.cuh:6-29): gpu = (key % sets) / (sets / gpus), set = key % (sets / gpus);
 * value = gpu * sets * ways + slot where slot = set * ways + way.  The reference keeps
 * only the skeleton of the dynamic cache (cache_helper.cuh:47-66 reduceMinSync, unused
 * lru_counter in static_cache_kernel.cuh:235, the retrieve_and_touch / transfer calls in
 * comp_cache/tests/test_cache.cu:57-58); the replacement rule is defined here:
 *   - lookup ("retrieve_and_touch"): a hit sets the way's stamp to the batch clock;
 *   - after the gather, every missed id asks for the way of its set with the smallest
 *     stamp (lowest way on ties; empty ways carry stamp -1); ways stamped in the current
 *     batch are never evicted; when several missed ids pick the same way the one that
 *     appears first in the id list wins, the others are not inserted in this batch.
 * State per gpu partition: keys[sets_per_gpu*ways] (-1 empty), stamps[...].
 * ---------------------------------------------------------------------------------- */
void orc_lru_lookup(int32_t *keys, int32_t *stamps, int64_t sets, int32_t ways, int32_t clock,
                    const int32_t *ids, int64_t n, int64_t *cache_index)
{
    for (int64_t r = 0; r < n; ++r) {
        int32_t id = ids[r];
        cache_index[r] = -1; /* static_retrieve_kernel: cache_index[i] = -1 */
        if (id < 0) continue;
        int64_t set = (int64_t)id % sets;
        for (int32_t w = 0; w < ways; ++w) {
            if (keys[set * ways + w] == id) {
                cache_index[r] = set * ways + w;
                stamps[set * ways + w] = clock;
                break;
            }
        }
    }
}

/* returns the number of rows inserted; inserted_slot[r] = slot or -1 */
int64_t orc_lru_insert(int32_t *keys, int32_t *stamps, int64_t sets, int32_t ways, int32_t clock,
                       const int32_t *ids, const int64_t *cache_index, int64_t n,
                       int64_t *inserted_slot)
{
    int64_t count = 0;
    int64_t nslots = sets * ways;
    int64_t *claim = (int64_t *)malloc(sizeof(int64_t) * (size_t)nslots);
    for (int64_t s = 0; s < nslots; ++s) claim[s] = INT64_MAX;
    /* phase 1: every missed id picks its victim from the state before any insertion */
    for (int64_t r = 0; r < n; ++r) {
        inserted_slot[r] = -1;
        if (cache_index[r] >= 0 || ids[r] < 0) continue;
        int64_t set = (int64_t)ids[r] % sets;
        int32_t best = -1, best_stamp = 0;
        for (int32_t w = 0; w < ways; ++w) {
            int32_t st = keys[set * ways + w] == -1 ? -1 : stamps[set * ways + w];
            if (st == clock) continue;
            if (best < 0 || st < best_stamp) { best = w; best_stamp = st; }
        }
        if (best < 0) continue;
        int64_t slot = set * ways + best;
        if (r < claim[slot]) claim[slot] = r;
        inserted_slot[r] = slot;
    }
    /* phase 2: the first claimant wins */
    for (int64_t r = 0; r < n; ++r) {
        int64_t slot = inserted_slot[r];
        if (slot < 0) continue;
        if (claim[slot] != r) { inserted_slot[r] = -1; continue; }
        keys[slot] = ids[r];
        stamps[slot] = clock;
        ++count;
    }
    free(claim);
    return count;
}

/* ------------------------------------------------------------------------------------
 * Step / mode arithmetic of the IPC environment (engine/ipc_service.cu:60-131,213-253).
 * ---------------------------------------------------------------------------------- */
void orc_coordinate(const int32_t *train_num, const int32_t *valid_num, const int32_t *test_num,
                    int32_t parts, int32_t raw_batch, int32_t *steps /*[3]*/,
                    int32_t *valid_bs /*[parts]*/, int32_t *test_bs /*[parts]*/)
{
    int32_t min_train = 1000000000, max_valid = 0, max_test = 0;
    for (int32_t i = 0; i < parts; ++i) {
        if (train_num[i] < min_train) min_train = train_num[i];
        if (valid_num[i] > max_valid) max_valid = valid_num[i];
        if (test_num[i] > max_test) max_test = test_num[i];
    }
    steps[0] = (min_train - 1) / raw_batch;
    steps[1] = (max_valid - 1) / 512 + 1;
    steps[2] = (max_test - 1) / 512 + 1;
    for (int32_t i = 0; i < parts; ++i) {
        valid_bs[i] = (valid_num[i] - 1) / steps[1] + 1;
        test_bs[i] = (test_num[i] - 1) / steps[2] + 1;
    }
}

void orc_mode_of_batch(int32_t global_batch, int32_t train_step, int32_t valid_step, int32_t test_step,
                       int32_t epochs, int32_t *mode, int32_t *local_batch)
{
    if (global_batch < (train_step + valid_step) * epochs) {
        int32_t eb = global_batch % (train_step + valid_step);
        if (eb < train_step) { *mode = 0; *local_batch = eb; }
        else { *mode = 1; *local_batch = eb - train_step; }
    } else {
        *mode = 2;
        *local_batch = (global_batch - (train_step + valid_step) * epochs) % test_step;
    }
}

/* ------------------------------------------------------------------------------------
 * Timed CPU baseline: the DGL CPU pipeline of training_backend/dgl_graphsage.py:189-204
 * (NeighborSampler -> to_block per hop -> feature and label index-select), restated with
 * the functions above and run over many batches with one batch per OpenMP thread.
 * features_out is one scratch area of `threads * max_nodes * row_bytes` bytes.
 * Returns the number of nodes gathered in total (a checksum that keeps the work alive).
 * ---------------------------------------------------------------------------------- */
int orc_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

int64_t orc_cpu_pipeline(const int64_t *indptr, const int32_t *indices,
                         const int32_t *all_ids, const int32_t *all_labels, int32_t total_cap,
                         int32_t batch_size, int32_t first_iter, int32_t n_batches, int32_t hop_num,
                         const int32_t *fanout, uint64_t seed, const uint8_t *host_table,
                         int64_t total_nodes, int64_t row_bytes, int64_t max_nodes, int64_t max_edges,
                         int32_t threads, uint8_t *features_out, int32_t *scratch /* threads*(max_nodes + 3*max_edges + batch) */)
{
    int64_t total = 0;
    int64_t per_thread = max_nodes + 3 * max_edges + batch_size;
#ifdef _OPENMP
    if (threads > 0) omp_set_num_threads(threads);
#endif
#pragma omp parallel for schedule(dynamic, 1) reduction(+ : total)
    for (int32_t b = 0; b < n_batches; ++b) {
        int tid = 0;
#ifdef _OPENMP
        tid = omp_get_thread_num();
#endif
        int32_t *base = scratch + per_thread * tid;
        int32_t *ids = base;
        int32_t *agg_src = ids + max_nodes;
        int32_t *agg_dst = agg_src + max_edges;
        int32_t *src_g = agg_dst + max_edges;
        int32_t *labels = src_g + max_edges;
        int32_t nc[16], ec[16];
        /* the list is walked round and round: batch numbers past its end start over */
        const int32_t whole = (total_cap - 1) / batch_size > 0 ? (total_cap - 1) / batch_size : 1;
        int64_t nn = orc_run_batch(indptr, indices, all_ids, all_labels, total_cap, batch_size,
                                   (first_iter + b) % whole, hop_num, fanout, (uint32_t)(first_iter + b), seed, 64,
                                   ids, labels, agg_src, agg_dst, src_g, nc, ec);
        if (nn < 0) continue;
        uint8_t *out = features_out + (int64_t)tid * max_nodes * row_bytes;
        for (int64_t r = 0; r < nn; ++r)
            memcpy(out + r * row_bytes, host_table + ((int64_t)ids[r] % total_nodes) * row_bytes,
                   (size_t)row_bytes);
        total += nn;
    }
    return total;
}

/* ------------------------------------------------------------------------------------
 * The same timed CPU baseline with a sampler written for a CPU, not a replay of the GPU's
 * lock-step algorithm: what a CPU library does for training_backend/dgl_graphsage.py:189-204
 * (uniform neighbour sampling without replacement, to_block relabelling, index-select).
 * Per hop the inputs are all nodes found so far, as above.  Picks: the whole list when
 * deg <= fanout, else Floyd's algorithm (fanout draws, distinct by construction) with a
 * splitmix64 stream per (batch, hop, input).  Relabelling: one open-addressing map per thread,
 * sized once and emptied through the list of touched slots.  NOT bit-comparable with the GPU
 * path (another random stream); it exists to be timed.  Returns the nodes gathered.
 * ---------------------------------------------------------------------------------- */
static inline uint64_t orc_splitmix(uint64_t *s)
{
    uint64_t z = (*s += 0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

int64_t orc_cpu_pipeline_native(const int64_t *indptr, const int32_t *indices,
                                const int32_t *all_ids, const int32_t *all_labels, int32_t total_cap,
                                int32_t batch_size, int32_t first_iter, int32_t n_batches, int32_t hop_num,
                                const int32_t *fanout, uint64_t seed, const uint8_t *host_table,
                                int64_t total_nodes, int64_t row_bytes, int64_t max_nodes, int64_t max_edges,
                                int32_t threads, uint8_t *features_out,
                                int32_t *scratch /* threads * (max_nodes + 2*max_edges + batch + 3*map_slots) */,
                                int64_t map_slots /* power of two >= 2 * max_nodes */)
{
    int64_t total = 0;
    const int64_t per_thread = max_nodes + 2 * max_edges + batch_size + 3 * map_slots;
#ifdef _OPENMP
    if (threads > 0) omp_set_num_threads(threads);
#endif
#pragma omp parallel reduction(+ : total)
    {
        int tid = 0;
#ifdef _OPENMP
        tid = omp_get_thread_num();
#endif
        int32_t *base = scratch + per_thread * tid;
        int32_t *ids = base;
        int32_t *agg_src = ids + max_nodes;
        int32_t *agg_dst = agg_src + max_edges;
        int32_t *labels = agg_dst + max_edges;
        int32_t *mkey = labels + batch_size;
        int32_t *mval = mkey + map_slots;
        int32_t *touched = mval + map_slots;
        const uint32_t mask = (uint32_t)(map_slots - 1);
        for (int64_t i = 0; i < map_slots; ++i) mkey[i] = -1;
        uint8_t *out = features_out + (int64_t)tid * max_nodes * row_bytes;
#pragma omp for schedule(dynamic, 1)
        for (int32_t b = 0; b < n_batches; ++b) {
            /* the list is walked round and round: batch numbers past its end start over */
            const int32_t whole = (total_cap - 1) / batch_size > 0 ? (total_cap - 1) / batch_size : 1;
            const int64_t first = (int64_t)batch_size * ((first_iter + b) % whole);
            int64_t size = first + batch_size >= total_cap ? total_cap - first : batch_size;
            if (size <= 0) continue;
            int64_t n_nodes = 0, n_edges = 0, n_touched = 0;
            for (int64_t i = 0; i < size; ++i) {
                const int32_t v = all_ids[first + i];
                labels[i] = all_labels[first + i];
                uint32_t s = orc_mix((uint32_t)v) & mask;
                while (mkey[s] != -1 && mkey[s] != v) s = (s + 1) & mask;
                if (mkey[s] == -1) { mkey[s] = v; mval[s] = (int32_t)n_nodes; touched[n_touched++] = (int32_t)s; }
                ids[n_nodes++] = v;
            }
            for (int32_t h = 0; h < hop_num; ++h) {
                const int64_t n_in = n_nodes;
                const int32_t k = fanout[h];
                for (int64_t i = 0; i < n_in; ++i) {
                    const int32_t v = ids[i];
                    if (v < 0) continue;
                    const int64_t s0 = indptr[v];
                    const int64_t deg = indptr[v + 1] - s0;
                    int32_t pick[ORC_MAX_FANOUT];
                    int32_t m = 0;
                    if (deg <= k) {
                        for (int64_t j = 0; j < deg; ++j) pick[m++] = (int32_t)j;
                    } else {
                        uint64_t st = seed ^ ((uint64_t)(first_iter + b) << 40) ^ ((uint64_t)h << 34) ^ (uint64_t)i;
                        for (int64_t j = deg - k; j < deg; ++j) {  /* Floyd: k distinct values of [0, deg) */
                            int32_t t = (int32_t)(orc_splitmix(&st) % (uint64_t)(j + 1));
                            int dup = 0;
                            for (int32_t q = 0; q < m; ++q) if (pick[q] == t) { dup = 1; break; }
                            pick[m++] = dup ? (int32_t)j : t;
                        }
                    }
                    for (int32_t q = 0; q < m; ++q) {
                        const int32_t u = indices[s0 + pick[q]];
                        uint32_t s = orc_mix((uint32_t)u) & mask;
                        while (mkey[s] != -1 && mkey[s] != u) s = (s + 1) & mask;
                        if (mkey[s] == -1) {
                            mkey[s] = u; mval[s] = (int32_t)n_nodes; touched[n_touched++] = (int32_t)s;
                            ids[n_nodes++] = u;
                        }
                        agg_src[n_edges] = mval[s];
                        agg_dst[n_edges] = (int32_t)i;
                        ++n_edges;
                    }
                }
            }
            for (int64_t r = 0; r < n_nodes; ++r)
                memcpy(out + r * row_bytes, host_table + ((int64_t)ids[r] % total_nodes) * row_bytes, (size_t)row_bytes);
            for (int64_t t = 0; t < n_touched; ++t) mkey[touched[t]] = -1;
            total += n_nodes;
        }
    }
    return total;
}
