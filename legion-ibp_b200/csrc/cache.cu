// Feature-cache construction: ranking, placement over the clique, fill (with optional
// int8 / fp8 encoding), and the state of the set-associative LRU cache.
//
// Replaces UnifiedCache::CandidateSelection / FillUp and their kernels
// (sampling_server/src/cache/cache.cu:354-447,559-656; cache/cache_impl.cuh:72-109,183-188) and
// StaticCache::init_cache (comp_cache/static_cache.cu:20-114).  The bucketed cuckoo table of
// the reference (include/hashmap/bcht.hpp) becomes a direct table with one int32 per node:
// one 4-byte read per lookup instead of up to three 128-byte bucket probes.
#include "common.cuh"

#include <cub/device/device_radix_sort.cuh>
#include <cub/device/device_scan.cuh>
#include <cuda_fp8.h>

namespace legion {

static constexpr unsigned kFull = 0xFFFFFFFFu;

__global__ void fill_i32_kernel(int32_t *a, int64_t n, int32_t v)
{
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        a[i] = v;
}

__global__ void fill_u64_kernel(unsigned long long *a, int64_t n, unsigned long long v)
{
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        a[i] = v;
}

__global__ void degree_keys_kernel(const int64_t *__restrict__ indptr, int64_t n, uint32_t *deg, int32_t *id)
{
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        deg[i] = (uint32_t)(indptr[i + 1] - indptr[i]);
        id[i] = (int32_t)i;
    }
}

// nodes that are not cached: remember where their row sits in a host table that is not in id order
__global__ void encode_host_rows_kernel(int32_t *lut, const int32_t *__restrict__ row_of, int64_t n)
{
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        if (lut[i] < 0) lut[i] = -(row_of[i] + 3);
}

__global__ void iota_kernel(int32_t *id, int64_t n)
{
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        id[i] = (int32_t)i;
}

// HotnessMeasure (cache/cache_impl.cuh:190-198): one count per node of the batch
__global__ void hotness_kernel(const int32_t *__restrict__ ids, const int32_t *__restrict__ nc, uint32_t *counts)
{
    const int n = nc[LEGION_INTRABATCH_CON * 3 + nc[LEGION_INTRABATCH_CON * 3 - 1]];
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        int32_t v = ids[i];
        if (v >= 0) atomicAdd(&counts[v], 1u);
    }
}

// rank t -> GPU t % kg, row t / kg (InitPair, cache_impl.cuh:104-109)
__global__ void static_place_kernel(const int32_t *__restrict__ order, int64_t n_cached, int32_t capacity, int32_t kg,
                                    int32_t *lut)
{
    for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < n_cached; t += (int64_t)gridDim.x * blockDim.x)
        lut[order[t]] = (int32_t)((t % kg) * (int64_t)capacity + t / kg);
}

__device__ __forceinline__ float warp_max(float v)
{
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v = fmaxf(v, __shfl_xor_sync(kFull, v, d));
    return v;
}

// Rank held by row s of a GPU's private replica region: the ranks that the striping gives to the
// other kg-1 members, in rank order (s = 0 is the hottest row this GPU does not hold itself).
__host__ __device__ __forceinline__ int64_t replica_rank(int64_t s, int32_t kg, int32_t ki)
{
    const int64_t round = s / (kg - 1);
    const int32_t j = (int32_t)(s - round * (kg - 1));
    return round * kg + j + (j >= ki ? 1 : 0);
}

__global__ void replica_place_kernel(const int32_t *__restrict__ order, int64_t n_ranked, int64_t n_rows, int32_t capacity,
                                     int32_t kg, int32_t ki, int32_t *lut)
{
    for (int64_t s = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; s < n_rows; s += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = replica_rank(s, kg, ki);
        if (t < n_ranked) lut[order[t]] = (int32_t)((int64_t)kg * capacity + s);
    }
}

// One warp per cached row: row s of GPU ki <- host row order[s*kg + ki] (FeatFillUp, cache_impl.cuh:183-188);
// with REPLICA, row s of the replica region <- host row order[replica_rank(s)].
// CODEC 0 copies bytes; 1 / 2 store feature_len codes + one fp32 scale, zero padded to slot_bytes.
template <int CODEC, bool REPLICA = false>
__global__ void __launch_bounds__(256)
static_fill_kernel(const int32_t *__restrict__ order, int64_t n_order, int32_t capacity, int32_t kg, int32_t ki,
                   const uint8_t *__restrict__ host, const int32_t *__restrict__ row_of, int32_t row_bytes, uint8_t *part,
                   int32_t slot_bytes)
{
    const int lane = threadIdx.x & 31;
    const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t s = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; s < capacity; s += n_warps) {
        int64_t t = REPLICA ? replica_rank(s, kg, ki) : s * kg + ki;
        if (t >= n_order) break;
        const int32_t node = order != nullptr ? order[t] : (int32_t)t;  // no order: row t of the table
        const uint8_t *src = host + (int64_t)(row_of != nullptr ? row_of[node] : node) * row_bytes;
        uint8_t *dst = part + s * (int64_t)slot_bytes;
        if (CODEC == LEGION_CODEC_RAW) {
            if ((row_bytes & 15) == 0) {
                for (int q = lane; q < (row_bytes >> 4); q += 32)
                    reinterpret_cast<uint4 *>(dst)[q] = reinterpret_cast<const uint4 *>(src)[q];
            } else {
                for (int q = lane; q < (row_bytes >> 2); q += 32)
                    reinterpret_cast<uint32_t *>(dst)[q] = reinterpret_cast<const uint32_t *>(src)[q];
            }
        } else {
            const int f = row_bytes >> 2;
            const float *x = reinterpret_cast<const float *>(src);
            float a = 0.0f;
            for (int i = lane; i < f; i += 32) a = fmaxf(a, fabsf(x[i]));
            a = warp_max(a);
            const float top = (CODEC == LEGION_CODEC_INT8) ? 127.0f : 448.0f;
            const float inv = a > 0.0f ? __fdiv_rn(top, a) : 0.0f;
            const float scale = __fdiv_rn(a, top);
            for (int i = lane; i < f; i += 32) {
                float prod = __fmul_rn(x[i], inv);
                uint8_t code;
                if (CODEC == LEGION_CODEC_INT8) {
                    int q = __float2int_rn(prod);
                    q = max(-127, min(127, q));
                    code = (uint8_t)(int8_t)q;
                } else {
                    code = (uint8_t)__nv_cvt_float_to_fp8(prod, __NV_SATFINITE, __NV_E4M3);
                }
                dst[i] = code;
            }
            if (lane == 0) *reinterpret_cast<float *>(dst + f) = scale;
            for (int i = f + 4 + lane; i < slot_bytes; i += 32) dst[i] = 0;
        }
    }
}

// weight of the node at every rank: its degree (indptr given) or its presampled access count
__global__ void ranked_weight_kernel(const int32_t *__restrict__ order, const int64_t *__restrict__ indptr,
                                     const uint32_t *__restrict__ counts, int64_t n, double *w)
{
    for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < n; t += (int64_t)gridDim.x * blockDim.x) {
        const int32_t v = order[t];
        w[t] = indptr != nullptr ? (double)(indptr[v + 1] - indptr[v]) : (double)counts[v];
    }
}

__global__ void pick_kernel(const double *__restrict__ cum, const int64_t *__restrict__ at, int n_at, double *out)
{
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n_at) out[i] = at[i] > 0 ? cum[at[i] - 1] : 0.0;
}

static int grid_stride(int64_t n, int sm_count)
{
    int64_t g = (n + 255) / 256;
    int64_t cap = (int64_t)sm_count * 16;
    if (g > cap) g = cap;
    if (g < 1) g = 1;
    return (int)g;
}

static int sm_count_of(int dev)
{
    int n = 148;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    return n > 0 ? n : 148;
}

int launch_hotness(cudaStream_t s, LegionPool *p, uint32_t *counts)
{
    int64_t g = (p->max_nodes + 255) / 256;
    int cap = p->sm_count * 8;
    hotness_kernel<<<(int)(g > cap ? cap : g), 256, 0, s>>>(p->ids[p->pipe], p->node_counter[p->pipe], counts);
    LG_LAUNCH_CHECK();
    return LEGION_OK;
}

}  // namespace legion

using namespace legion;

extern "C" int legion_cache_create(LegionCache **out, int32_t dev_id, int64_t n_nodes, int32_t row_bytes,
                                   int32_t kg, int32_t ki, int32_t capacity, int32_t codec)
{
    LG_ARG(out != nullptr, "out is NULL");
    LG_ARG(n_nodes > 0 && n_nodes < (1ll << 31), "n_nodes must fit int32");
    LG_ARG(row_bytes > 0 && row_bytes % 4 == 0, "row_bytes must be a positive multiple of 4");
    LG_ARG(kg >= 1 && kg <= LEGION_MAX_DEVICE && ki >= 0 && ki < kg, "bad clique size or member index");
    LG_ARG(capacity >= 0 && (int64_t)capacity * kg < (1ll << 31), "capacity * kg must fit int32");
    LG_ARG(codec >= LEGION_CODEC_RAW && codec <= LEGION_CODEC_E4M3, "unknown codec");
    if (codec != LEGION_CODEC_RAW) LG_ARG((row_bytes / 4) % 4 == 0, "compressed rows need feature_len % 4 == 0");
    LG_CUDA(cudaSetDevice(dev_id));
    LegionCache *c = new LegionCache();
    memset(c, 0, sizeof(*c));
    c->dev_id = dev_id;
    c->n_nodes = n_nodes;
    c->row_bytes = row_bytes;
    c->codec = codec;
    c->kind = 0;
    c->kg = kg;
    c->ki = ki;
    c->capacity = capacity;
    c->slot_bytes = codec == LEGION_CODEC_RAW ? row_bytes : (row_bytes / 4 + 4 + 15) / 16 * 16;
    cudaError_t e = cudaMalloc(&c->lut, sizeof(int32_t) * n_nodes);
    if (e == cudaSuccess && capacity > 0) {
        // a partition that peers will read is allocated as shareable memory so that other processes
        // can map it; when that is not available it falls back to cudaMalloc (+ legacy IPC handles)
        if (kg > 1 && vmm_alloc(dev_id, (int64_t)capacity * c->slot_bytes, &c->own_block) == LEGION_OK)
            c->part[ki] = c->own_block.ptr;
        else
            e = cudaMalloc(&c->part[ki], (int64_t)capacity * c->slot_bytes);
    }
    if (e == cudaSuccess) e = cudaMalloc(&c->stats, sizeof(unsigned long long) * 4);
    if (e != cudaSuccess) {
        set_error("legion_cache_create: cudaMalloc failed: %s", cudaGetErrorString(e));
        cudaFree(c->lut); cudaFree(c->stats);
        if (c->own_block.ptr) vmm_free(&c->own_block); else cudaFree(c->part[ki]);
        delete c;
        return LEGION_E_NOMEM;
    }
    int sms = sm_count_of(dev_id);
    fill_i32_kernel<<<grid_stride(n_nodes, sms), 256>>>(c->lut, n_nodes, LEGION_CACHEMISS_FLAG);
    LG_LAUNCH_CHECK();
    LG_CUDA(cudaMemset(c->stats, 0, sizeof(unsigned long long) * 4));
    LG_CUDA(cudaDeviceSynchronize());
    *out = c;
    return LEGION_OK;
}

// ids 0..n-1 sorted by descending 32-bit key, ties by ascending id (LSD radix sort is stable)
static int order_by_key_desc(int32_t dev_id, uint32_t *keys_in, int64_t n_nodes, int32_t *order_dev, cudaStream_t s,
                             const int64_t *indptr_for_degree)
{
    uint32_t *deg_out = nullptr;
    int32_t *id_in = nullptr;
    void *tmp = nullptr;
    size_t tmp_bytes = 0;
    int rc = LEGION_OK;
    cudaError_t e = cudaMalloc(&deg_out, sizeof(uint32_t) * n_nodes);
    if (e == cudaSuccess) e = cudaMalloc(&id_in, sizeof(int32_t) * n_nodes);
    if (e == cudaSuccess)
        e = cub::DeviceRadixSort::SortPairsDescending(nullptr, tmp_bytes, keys_in, deg_out, id_in, order_dev,
                                                      (int)n_nodes, 0, 32, s);
    if (e == cudaSuccess) e = cudaMalloc(&tmp, tmp_bytes > 0 ? tmp_bytes : 1);
    if (e == cudaSuccess) {
        if (indptr_for_degree != nullptr)
            degree_keys_kernel<<<grid_stride(n_nodes, sm_count_of(dev_id)), 256, 0, s>>>(indptr_for_degree, n_nodes, keys_in, id_in);
        else
            iota_kernel<<<grid_stride(n_nodes, sm_count_of(dev_id)), 256, 0, s>>>(id_in, n_nodes);
        e = cudaGetLastError();
    }
    if (e == cudaSuccess)
        e = cub::DeviceRadixSort::SortPairsDescending(tmp, tmp_bytes, keys_in, deg_out, id_in, order_dev, (int)n_nodes,
                                                      0, 32, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) {
        set_error("node ranking failed: %s", cudaGetErrorString(e));
        rc = LEGION_E_CUDA;
    }
    cudaFree(deg_out); cudaFree(id_in); cudaFree(tmp);
    return rc;
}

extern "C" int legion_cache_degree_order(int32_t dev_id, const int64_t *indptr, int64_t n_nodes,
                                         int32_t *order_dev, void *stream)
{
    LG_ARG(indptr != nullptr && order_dev != nullptr, "NULL pointer");
    LG_ARG(n_nodes > 0 && n_nodes < (1ll << 31), "n_nodes must fit int32");
    LG_CUDA(cudaSetDevice(dev_id));
    uint32_t *keys = nullptr;
    if (cudaMalloc(&keys, sizeof(uint32_t) * n_nodes) != cudaSuccess) {
        set_error("legion_cache_degree_order: out of memory");
        return LEGION_E_NOMEM;
    }
    int rc = order_by_key_desc(dev_id, keys, n_nodes, order_dev, (cudaStream_t)stream, indptr);
    cudaFree(keys);
    return rc;
}

// CandidateSelection (cache/cache.cu:354-447): nodes ranked by how often the presampling epoch
// touched them, most often first (thrust::sort_by_key with greater<>, cache.cu:419); ties, which the
// reference leaves to the sort, go by ascending id.  counts_dev: one uint32 per node, as filled by
// legion_runner_presample.
extern "C" int legion_cache_hotness_order(int32_t dev_id, const uint32_t *counts_dev, int64_t n_nodes,
                                          int32_t *order_dev, void *stream)
{
    LG_ARG(counts_dev != nullptr && order_dev != nullptr, "NULL pointer");
    LG_ARG(n_nodes > 0 && n_nodes < (1ll << 31), "n_nodes must fit int32");
    LG_CUDA(cudaSetDevice(dev_id));
    uint32_t *keys = nullptr;
    if (cudaMalloc(&keys, sizeof(uint32_t) * n_nodes) != cudaSuccess) {
        set_error("legion_cache_hotness_order: out of memory");
        return LEGION_E_NOMEM;
    }
    cudaError_t e = cudaMemcpyAsync(keys, counts_dev, sizeof(uint32_t) * n_nodes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream);
    int rc = e == cudaSuccess ? order_by_key_desc(dev_id, keys, n_nodes, order_dev, (cudaStream_t)stream, nullptr) : LEGION_E_CUDA;
    cudaFree(keys);
    return rc;
}

extern "C" int legion_cache_fill_static_rows(LegionCache *c, const int32_t *order_dev, int64_t n_order,
                                             const void *host_table, const int32_t *row_of_id_dev, void *stream)
{
    LG_ARG(c != nullptr && c->kind == 0, "not a static cache");
    LG_ARG(order_dev != nullptr && n_order >= 0 && n_order <= c->n_nodes, "bad order");
    LG_CUDA(cudaSetDevice(c->dev_id));
    cudaStream_t s = (cudaStream_t)stream;
    c->host_table = host_table;
    int sms = sm_count_of(c->dev_id);
    int64_t n_cached = (int64_t)c->capacity * c->kg;
    if (n_cached > n_order) n_cached = n_order;
    if (c->part[c->kg] != nullptr) {  // a refill drops the replicas of the previous ranking
        LG_CUDA(cudaStreamSynchronize(s));
        cudaFree(c->part[c->kg]);
        c->part[c->kg] = nullptr;
        c->replica_rows = 0;
    }
    fill_i32_kernel<<<grid_stride(c->n_nodes, sms), 256, 0, s>>>(c->lut, c->n_nodes, LEGION_CACHEMISS_FLAG);
    LG_LAUNCH_CHECK();
    if (n_cached > 0) {
        static_place_kernel<<<grid_stride(n_cached, sms), 256, 0, s>>>(order_dev, n_cached, c->capacity, c->kg, c->lut);
        LG_LAUNCH_CHECK();
        if (host_table == nullptr && c->fill_by_caller) {  // legion_cache_place_static: the caller writes the rows
            LG_CUDA(cudaStreamSynchronize(s));
            c->fill_gen += 1;
            return LEGION_OK;
        }
        LG_ARG(host_table != nullptr, "host_table is NULL");
        int64_t warps = c->capacity;
        int64_t g = (warps + 7) / 8;
        int grid = (int)(g > (int64_t)sms * 16 ? (int64_t)sms * 16 : (g < 1 ? 1 : g));
        uint8_t *part = (uint8_t *)c->part[c->ki];
        const uint8_t *host = (const uint8_t *)host_table;
        if (c->host_codec != LEGION_CODEC_RAW)  // rows of the host table are cache slots already: copy them
            static_fill_kernel<LEGION_CODEC_RAW><<<grid, 256, 0, s>>>(order_dev, n_cached, c->capacity, c->kg, c->ki,
                                                                     host, row_of_id_dev, c->slot_bytes, part, c->slot_bytes);
        else if (c->codec == LEGION_CODEC_RAW)
            static_fill_kernel<LEGION_CODEC_RAW><<<grid, 256, 0, s>>>(order_dev, n_cached, c->capacity, c->kg, c->ki,
                                                                     host, row_of_id_dev, c->row_bytes, part, c->slot_bytes);
        else if (c->codec == LEGION_CODEC_INT8)
            static_fill_kernel<LEGION_CODEC_INT8><<<grid, 256, 0, s>>>(order_dev, n_cached, c->capacity, c->kg, c->ki,
                                                                      host, row_of_id_dev, c->row_bytes, part, c->slot_bytes);
        else
            static_fill_kernel<LEGION_CODEC_E4M3><<<grid, 256, 0, s>>>(order_dev, n_cached, c->capacity, c->kg, c->ki,
                                                                      host, row_of_id_dev, c->row_bytes, part, c->slot_bytes);
        LG_LAUNCH_CHECK();
    }
    if (row_of_id_dev != nullptr) {
        encode_host_rows_kernel<<<grid_stride(c->n_nodes, sms), 256, 0, s>>>(c->lut, row_of_id_dev, c->n_nodes);
        LG_LAUNCH_CHECK();
    }
    LG_CUDA(cudaStreamSynchronize(s));
    c->fill_gen += 1;
    return LEGION_OK;
}

extern "C" int legion_cache_add_replicas(LegionCache *c, const int32_t *order_dev, int64_t n_order, int64_t n_rows,
                                         const int32_t *row_of_id_dev, void *stream)
{
    LG_ARG(c != nullptr && c->kind == 0, "not a static cache");
    LG_ARG(c->kg > 1, "a clique of one GPU has nothing to replicate");
    LG_ARG(c->host_table != nullptr, "fill the cache first (legion_cache_fill_static)");
    LG_ARG(c->part[c->kg] == nullptr, "the cache already holds replicas; refill it first");
    LG_ARG(order_dev != nullptr && n_order >= 0 && n_order <= c->n_nodes, "bad order");
    LG_ARG(n_rows >= 0 && n_rows <= c->capacity, "replica rows must not exceed the capacity of a partition");
    LG_ARG(((int64_t)c->kg + 1) * c->capacity < (1ll << 31), "capacity * (kg + 1) must fit int32");
    LG_CUDA(cudaSetDevice(c->dev_id));
    cudaStream_t s = (cudaStream_t)stream;
    // only ranks that the striping placed can be replicated
    int64_t n_ranked = (int64_t)c->capacity * c->kg;
    if (n_ranked > n_order) n_ranked = n_order;
    while (n_rows > 0 && replica_rank(n_rows - 1, c->kg, c->ki) >= n_ranked) --n_rows;
    if (n_rows == 0) return LEGION_OK;
    void *rep = nullptr;
    if (cudaMalloc(&rep, n_rows * (int64_t)c->slot_bytes) != cudaSuccess) {
        cudaGetLastError();
        set_error("legion_cache_add_replicas: out of device memory for %lld rows", (long long)n_rows);
        return LEGION_E_NOMEM;
    }
    int sms = sm_count_of(c->dev_id);
    int64_t g = (n_rows + 7) / 8;
    int grid = (int)(g > (int64_t)sms * 16 ? (int64_t)sms * 16 : (g < 1 ? 1 : g));
    const uint8_t *host = (const uint8_t *)c->host_table;
    if (c->host_codec != LEGION_CODEC_RAW)
        static_fill_kernel<LEGION_CODEC_RAW, true><<<grid, 256, 0, s>>>(order_dev, n_ranked, (int32_t)n_rows, c->kg, c->ki, host,
                                                                         row_of_id_dev, c->slot_bytes, (uint8_t *)rep, c->slot_bytes);
    else if (c->codec == LEGION_CODEC_RAW)
        static_fill_kernel<LEGION_CODEC_RAW, true><<<grid, 256, 0, s>>>(order_dev, n_ranked, (int32_t)n_rows, c->kg, c->ki, host,
                                                                         row_of_id_dev, c->row_bytes, (uint8_t *)rep, c->slot_bytes);
    else if (c->codec == LEGION_CODEC_INT8)
        static_fill_kernel<LEGION_CODEC_INT8, true><<<grid, 256, 0, s>>>(order_dev, n_ranked, (int32_t)n_rows, c->kg, c->ki, host,
                                                                          row_of_id_dev, c->row_bytes, (uint8_t *)rep, c->slot_bytes);
    else
        static_fill_kernel<LEGION_CODEC_E4M3, true><<<grid, 256, 0, s>>>(order_dev, n_ranked, (int32_t)n_rows, c->kg, c->ki, host,
                                                                          row_of_id_dev, c->row_bytes, (uint8_t *)rep, c->slot_bytes);
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) {
        replica_place_kernel<<<grid_stride(n_rows, sms), 256, 0, s>>>(order_dev, n_ranked, n_rows, c->capacity, c->kg, c->ki, c->lut);
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) {
        set_error("legion_cache_add_replicas: %s", cudaGetErrorString(e));
        cudaFree(rep);
        return LEGION_E_CUDA;
    }
    c->part[c->kg] = rep;
    c->replica_rows = (int32_t)n_rows;
    c->fill_gen += 1;
    return LEGION_OK;
}

// Placement only (InitPair + Insert, cache/cache_impl.cuh:104-109, cache/cache.cu:74-112, without FeatFillUp):
// builds the lookup table for `order`; the caller then writes the rows of this GPU's partition itself
// (row s of legion_cache_partition holds node order[s * kg + ki]).  For tables that exist nowhere as a
// whole, e.g. a table larger than host memory whose stripes are loaded or generated GPU by GPU.
extern "C" int legion_cache_place_static(LegionCache *c, const int32_t *order_dev, int64_t n_order, void *stream)
{
    LG_ARG(c != nullptr && c->kind == 0, "not a static cache");
    LG_ARG(c->codec == LEGION_CODEC_RAW, "rows written by the caller must be uncompressed");
    c->fill_by_caller = 1;
    int rc = legion_cache_fill_static_rows(c, order_dev, n_order, nullptr, nullptr, stream);
    c->fill_by_caller = 0;
    return rc;
}

extern "C" int legion_cache_fill_static(LegionCache *c, const int32_t *order_dev, int64_t n_order,
                                        const void *host_table, void *stream)
{
    return legion_cache_fill_static_rows(c, order_dev, n_order, host_table, nullptr, stream);
}

// Splits one GPU's row budget into its stripe of the clique's cache and private copies of hot rows
// held by peers (legion_cache_add_replicas).  mass(x) = share of all row accesses that go to the x
// hottest nodes, estimated from the weights in rank order (degree, or presampled counts).  With R
// replica rows and S = budget - R stripe rows per GPU the clique holds C = min(n, S * world) nodes; the
// T = R * world / (world - 1) hottest of them are local on every GPU, the others with probability
// 1 / world; the plan minimises
//   host * (1 - mass(C)) + peer * (mass(C) - mass(T)) * (world - 1) / world + local * (the rest).
// R = 0 is the reference's plan (striping only, cache/cache_impl.cuh:104-109).
extern "C" int legion_cache_plan(int32_t dev_id, const int32_t *order_dev, const int64_t *indptr_dev,
                                 const uint32_t *counts_dev, int64_t n_nodes, int64_t budget_rows, int32_t world,
                                 const double cost_local_peer_host[3], int64_t *stripe_rows, int64_t *replica_rows,
                                 void *stream)
{
    LG_ARG(order_dev != nullptr && (indptr_dev != nullptr || counts_dev != nullptr), "NULL pointer");
    LG_ARG(stripe_rows != nullptr && replica_rows != nullptr, "NULL result pointer");
    LG_ARG(n_nodes > 0 && n_nodes < (1ll << 31) && world >= 1 && world <= LEGION_MAX_DEVICE, "bad size");
    if (budget_rows < 0) budget_rows = 0;
    if (budget_rows > n_nodes) budget_rows = n_nodes;
    *stripe_rows = budget_rows;
    *replica_rows = 0;
    if (world == 1 || budget_rows == 0) return LEGION_OK;
    const double c_local = cost_local_peer_host ? cost_local_peer_host[0] : 0.16;
    const double c_peer = cost_local_peer_host ? cost_local_peer_host[1] : 1.0;
    const double c_host = cost_local_peer_host ? cost_local_peer_host[2] : 15.0;
    constexpr int kSteps = 64;
    const int64_t full = (n_nodes + world - 1) / world;
    int64_t cand_r[kSteps + 1], cand_s[kSteps + 1], at[2 * (kSteps + 1) + 1];
    for (int i = 0; i <= kSteps; ++i) {
        int64_t r = budget_rows / 2 * i / kSteps;
        int64_t stripe = budget_rows - r < full ? budget_rows - r : full;
        if (r > stripe) r = stripe;
        int64_t covered = stripe * world < n_nodes ? stripe * world : n_nodes;
        int64_t local_top = r * world / (world - 1);
        if (local_top > covered) local_top = covered;
        cand_r[i] = r;
        cand_s[i] = stripe;
        at[2 * i] = covered;
        at[2 * i + 1] = local_top;
    }
    at[2 * (kSteps + 1)] = n_nodes;
    const int n_at = 2 * (kSteps + 1) + 1;

    LG_CUDA(cudaSetDevice(dev_id));
    cudaStream_t s = (cudaStream_t)stream;
    double *w = nullptr, *d_out = nullptr;
    int64_t *d_at = nullptr;
    void *tmp = nullptr;
    size_t tmp_bytes = 0;
    double h_out[2 * (kSteps + 1) + 1];
    cudaError_t e = cudaMalloc(&w, sizeof(double) * n_nodes);
    if (e == cudaSuccess) e = cudaMalloc(&d_out, sizeof(double) * n_at);
    if (e == cudaSuccess) e = cudaMalloc(&d_at, sizeof(int64_t) * n_at);
    if (e == cudaSuccess) e = cub::DeviceScan::InclusiveSum(nullptr, tmp_bytes, w, w, (int)n_nodes, s);
    if (e == cudaSuccess) e = cudaMalloc(&tmp, tmp_bytes > 0 ? tmp_bytes : 1);
    if (e == cudaSuccess) {
        ranked_weight_kernel<<<grid_stride(n_nodes, sm_count_of(dev_id)), 256, 0, s>>>(order_dev, indptr_dev, counts_dev, n_nodes, w);
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cub::DeviceScan::InclusiveSum(tmp, tmp_bytes, w, w, (int)n_nodes, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(d_at, at, sizeof(int64_t) * n_at, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) {
        pick_kernel<<<(n_at + 127) / 128, 128, 0, s>>>(w, d_at, n_at, d_out);
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaMemcpyAsync(h_out, d_out, sizeof(double) * n_at, cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    cudaFree(w); cudaFree(d_out); cudaFree(d_at); cudaFree(tmp);
    if (e != cudaSuccess) {
        cudaGetLastError();
        set_error("legion_cache_plan: %s", cudaGetErrorString(e));
        return e == cudaErrorMemoryAllocation ? LEGION_E_NOMEM : LEGION_E_CUDA;
    }
    const double total = h_out[n_at - 1];
    int best = 0;
    double best_cost = 0.0;
    for (int i = 0; i <= kSteps; ++i) {
        const double m_c = total > 0.0 ? h_out[2 * i] / total : 0.0;
        const double m_t = total > 0.0 ? h_out[2 * i + 1] / total : 0.0;
        const double t = c_host * (1.0 - m_c) + c_peer * (m_c - m_t) * (world - 1) / world +
                         c_local * (m_t + (m_c - m_t) / world);
        if (i == 0 || t < best_cost - 1e-12) {
            best_cost = t;
            best = i;
        }
    }
    int64_t stripe = cand_s[best], r = cand_r[best];
    if (stripe == full) {  // memory left over once the stripes cover the table goes to replicas
        int64_t spare = budget_rows - stripe < stripe ? budget_rows - stripe : stripe;
        if (spare > r) r = spare;
    }
    *stripe_rows = stripe;
    *replica_rows = r;
    return LEGION_OK;
}

extern "C" int legion_cache_set_host_codec(LegionCache *c, int32_t codec)
{
    LG_ARG(c != nullptr && c->kind == 0, "not a static cache");
    LG_ARG(codec == LEGION_CODEC_RAW || codec == c->codec, "a compressed host table needs a cache of the same codec");
    c->host_codec = codec;
    return LEGION_OK;
}

extern "C" int legion_quantize_table(int32_t dev_id, int32_t codec, const void *rows, int64_t n_rows, int32_t feature_len,
                                     void *out_rows, void *stream)
{
    LG_ARG(codec == LEGION_CODEC_INT8 || codec == LEGION_CODEC_E4M3, "codec must be INT8 or E4M3");
    LG_ARG(rows != nullptr && out_rows != nullptr && n_rows >= 0 && n_rows < (1ll << 31), "bad rows");
    LG_ARG(feature_len > 0 && feature_len % 4 == 0, "compressed rows need feature_len % 4 == 0");
    if (n_rows == 0) return LEGION_OK;
    LG_CUDA(cudaSetDevice(dev_id));
    cudaStream_t s = (cudaStream_t)stream;
    const int sms = sm_count_of(dev_id);
    const int32_t slot = (feature_len + 4 + 15) / 16 * 16;
    int64_t g = (n_rows + 7) / 8;
    int grid = (int)(g > (int64_t)sms * 16 ? (int64_t)sms * 16 : g);
    if (codec == LEGION_CODEC_INT8)
        static_fill_kernel<LEGION_CODEC_INT8><<<grid, 256, 0, s>>>(nullptr, n_rows, (int32_t)n_rows, 1, 0, (const uint8_t *)rows,
                                                                  nullptr, feature_len * 4, (uint8_t *)out_rows, slot);
    else
        static_fill_kernel<LEGION_CODEC_E4M3><<<grid, 256, 0, s>>>(nullptr, n_rows, (int32_t)n_rows, 1, 0, (const uint8_t *)rows,
                                                                  nullptr, feature_len * 4, (uint8_t *)out_rows, slot);
    LG_LAUNCH_CHECK();
    LG_CUDA(cudaStreamSynchronize(s));
    return LEGION_OK;
}

extern "C" int legion_cache_set_host_table(LegionCache *c, const void *host_table)
{
    LG_ARG(c != nullptr, "cache is NULL");
    c->host_table = host_table;
    return LEGION_OK;
}

extern "C" int legion_cache_partition(LegionCache *c, void **ptr, int64_t *bytes)
{
    LG_ARG(c != nullptr && c->kind == 0, "not a static cache");
    if (ptr) *ptr = c->part[c->ki];
    if (bytes) *bytes = (int64_t)c->capacity * c->slot_bytes;
    return LEGION_OK;
}

extern "C" int legion_cache_set_peer(LegionCache *c, int32_t k, const void *partition_ptr)
{
    LG_ARG(c != nullptr && c->kind == 0, "not a static cache");
    LG_ARG(k >= 0 && k < c->kg && k != c->ki, "k must name another member of the clique");
    c->part[k] = const_cast<void *>(partition_ptr);
    return LEGION_OK;
}

extern "C" int legion_cache_lut(LegionCache *c, int32_t **lut_dev)
{
    LG_ARG(c != nullptr && c->kind == 0 && lut_dev != nullptr, "not a static cache");
    LG_ARG(c->part[c->kg] == nullptr, "the lookup table of a cache with replicas is only usable through the cache handle");
    LG_ARG(c->codec == LEGION_CODEC_RAW, "the lookup table of a compressed cache is only usable through the cache handle");
    *lut_dev = c->lut;
    return LEGION_OK;
}

extern "C" int legion_cache_create_lru(LegionCache **out, int32_t dev_id, int64_t n_nodes, int32_t row_bytes,
                                       int64_t sets, int32_t ways)
{
    LG_ARG(out != nullptr, "out is NULL");
    LG_ARG(n_nodes > 0 && n_nodes < (1ll << 31), "n_nodes must fit int32");
    LG_ARG(row_bytes > 0 && row_bytes % 16 == 0 && row_bytes <= 2048, "row_bytes must be a multiple of 16, at most 2048");
    LG_ARG(sets > 0, "sets must be positive");
    LG_ARG(ways >= 1 && ways <= 32 && (ways & (ways - 1)) == 0, "ways must be a power of two, at most 32");
    LG_CUDA(cudaSetDevice(dev_id));
    LegionCache *c = new LegionCache();
    memset(c, 0, sizeof(*c));
    c->dev_id = dev_id;
    c->n_nodes = n_nodes;
    c->row_bytes = row_bytes;
    c->slot_bytes = row_bytes;
    c->kind = 1;
    c->kg = 1;
    c->sets = sets;
    c->ways = ways;
    c->clock = 1;
    int64_t slots = sets * ways;
    cudaError_t e = cudaMalloc(&c->keys, sizeof(int32_t) * slots);
    if (e == cudaSuccess) e = cudaMalloc(&c->stamps, sizeof(int32_t) * slots);
    if (e == cudaSuccess) e = cudaMalloc(&c->claim, sizeof(int64_t) * slots);
    if (e == cudaSuccess) e = cudaMalloc(&c->rows, slots * (int64_t)row_bytes);
    if (e == cudaSuccess) e = cudaMalloc(&c->stats, sizeof(unsigned long long) * 4);
    if (e != cudaSuccess) {
        set_error("legion_cache_create_lru: cudaMalloc failed: %s", cudaGetErrorString(e));
        cudaFree(c->keys); cudaFree(c->stamps); cudaFree(c->claim); cudaFree(c->rows); cudaFree(c->stats);
        delete c;
        return LEGION_E_NOMEM;
    }
    int sms = sm_count_of(dev_id);
    fill_i32_kernel<<<grid_stride(slots, sms), 256>>>(c->keys, slots, -1);
    LG_LAUNCH_CHECK();
    fill_i32_kernel<<<grid_stride(slots, sms), 256>>>(c->stamps, slots, 0);
    LG_LAUNCH_CHECK();
    fill_u64_kernel<<<grid_stride(slots, sms), 256>>>(reinterpret_cast<unsigned long long *>(c->claim), slots, ~0ull);
    LG_LAUNCH_CHECK();
    LG_CUDA(cudaMemset(c->stats, 0, sizeof(unsigned long long) * 4));
    LG_CUDA(cudaDeviceSynchronize());
    *out = c;
    return LEGION_OK;
}

extern "C" int legion_cache_lru_state(LegionCache *c, int32_t **keys_dev, int32_t **stamps_dev, void **rows_dev)
{
    LG_ARG(c != nullptr && c->kind == 1, "not an lru cache");
    if (keys_dev) *keys_dev = c->keys;
    if (stamps_dev) *stamps_dev = c->stamps;
    if (rows_dev) *rows_dev = c->rows;
    return LEGION_OK;
}

extern "C" int legion_cache_lru_clock(LegionCache *c, int32_t *clock)
{
    LG_ARG(c != nullptr && c->kind == 1 && clock != nullptr, "not an lru cache");
    *clock = c->clock;
    return LEGION_OK;
}

extern "C" int legion_cache_stats(LegionCache *c, int64_t stats[4], void *stream)
{
    LG_ARG(c != nullptr && stats != nullptr, "NULL pointer");
    LG_CUDA(cudaSetDevice(c->dev_id));
    unsigned long long h[4];
    LG_CUDA(cudaMemcpyAsync(h, c->stats, sizeof(h), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    LG_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    for (int i = 0; i < 4; ++i) stats[i] = (int64_t)h[i];
    return LEGION_OK;
}

extern "C" int legion_cache_destroy(LegionCache *c)
{
    if (c == nullptr) return LEGION_OK;
    cudaSetDevice(c->dev_id);
    if (c->kind == 0) {
        cudaDeviceSynchronize();
        cudaFree(c->lut);
        if (c->own_block.ptr) vmm_free(&c->own_block); else cudaFree(c->part[c->ki]);
        cudaFree(c->part[c->kg]);
        for (int k = 0; k < LEGION_MAX_DEVICE; ++k)
            if (c->peer_block[k].ptr) vmm_free(&c->peer_block[k]);
    } else {
        cudaFree(c->keys); cudaFree(c->stamps); cudaFree(c->claim); cudaFree(c->rows);
    }
    cudaFree(c->stats);
    delete c;
    return LEGION_OK;
}
