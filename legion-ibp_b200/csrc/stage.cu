// Seed-row staging: the rows of a seed list's uncached nodes, kept in page-locked host memory in list
// order, so that the uncached seed rows of one batch are ONE contiguous block that the copy engine
// brings to the device while the batch is still being sampled.
//
// Why: on this platform a kernel that reads pinned host memory by zero-copy loads slows the HBM-bound
// kernels that run beside it by 2.4-3.6x for as long as it runs (measured: a gather of cached rows at
// 5.5 TB/s alone drops to ~1.5 TB/s beside a fetch that moves 12-37 GB/s, whatever the fetch's launch
// shape, plain loads or bulk copies), so fetch time and device time add up instead of overlapping.  A
// copy-engine transfer does not.  Seeds are about 60% of the rows that miss a degree-ordered cache (they
// are random training nodes, not hubs), and the seed list of a mode is known for the whole run
// (engine/operator_impl.cu:28-56 slices it batch by batch), so their rows can be laid out ahead of time.
// Rows of sampled neighbours that miss still come by zero-copy loads (cache/cache_impl.cuh:283-286 is
// the reference's miss path for every row).
#include "common.cuh"

#include <cub/device/device_scan.cuh>

namespace legion {

// flags[q] = 1 when list entry q is a node whose row only the host table holds
__global__ void stage_flag_kernel(const int32_t *__restrict__ ids, int32_t count, const int32_t *__restrict__ lut,
                                  int64_t n_nodes, int32_t *flags)
{
    for (int q = blockIdx.x * blockDim.x + threadIdx.x; q <= count; q += gridDim.x * blockDim.x) {
        int f = 0;
        if (q < count) {
            const int32_t id = ids[q];
            if (id >= 0 && id < n_nodes) f = (lut == nullptr || lut[id] < 0) ? 1 : 0;
        }
        flags[q] = f;
    }
}

// one warp per list entry: host table row -> its slot of the staging array (both reached by zero-copy)
__global__ void __launch_bounds__(256)
stage_copy_kernel(const int32_t *__restrict__ ids, int32_t count, const int32_t *__restrict__ lut,
                  const int32_t *__restrict__ pos, const uint8_t *__restrict__ host, int64_t n_nodes, int32_t row_bytes,
                  uint8_t *rows_out)
{
    const int lane = threadIdx.x & 31;
    const int n_warps = (gridDim.x * blockDim.x) >> 5;
    for (int q = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; q < count; q += n_warps) {
        if (pos[q + 1] == pos[q]) continue;
        const int32_t id = ids[q];
        const int32_t raw = lut != nullptr ? lut[id] : LEGION_CACHEMISS_FLAG;
        const int64_t host_row = raw <= -3 ? (int64_t)(-(raw + 3)) : (int64_t)id;
        const uint8_t *src = host + (host_row % n_nodes) * (int64_t)row_bytes;
        uint8_t *dst = rows_out + (int64_t)pos[q] * row_bytes;
        if ((row_bytes & 15) == 0) {
            for (int v = lane; v < (row_bytes >> 4); v += 32)
                reinterpret_cast<uint4 *>(dst)[v] = reinterpret_cast<const uint4 *>(src)[v];
        } else {
            for (int v = lane; v < (row_bytes >> 2); v += 32)
                reinterpret_cast<uint32_t *>(dst)[v] = reinterpret_cast<const uint32_t *>(src)[v];
        }
    }
}

void stage_free(SeedStage *st)
{
    if (st == nullptr) return;
    cudaFree(st->pos_dev);
    cudaFree(st->own_ids_dev);
    if (st->rows_host) cudaFreeHost(st->rows_host);
    delete[] st->pos;
    delete[] st->host_copy;
    memset(st, 0, sizeof(*st));
}

// Builds the staging of one list for one static cache of uncompressed rows.  ids_dev: the list on the
// device (count entries).  The cache must be filled (and its replicas added) before.
int stage_build(LegionCache *c, const int32_t *ids_dev, int32_t count, int sm_count, SeedStage *st)
{
    LG_ARG(c != nullptr && c->kind == 0 && c->codec == LEGION_CODEC_RAW && c->host_codec == LEGION_CODEC_RAW,
           "seed staging needs a static cache of uncompressed rows");
    LG_ARG(c->host_table != nullptr, "seed staging needs a host table (fill the cache first)");
    LG_ARG(ids_dev != nullptr && count > 0, "empty seed list");
    LG_CUDA(cudaSetDevice(c->dev_id));
    st->count = count;
    st->ids_dev = ids_dev;
    st->fill_gen = c->fill_gen;
    st->cache = c;
    int32_t *flags = nullptr;
    void *tmp = nullptr;
    size_t tmp_bytes = 0;
    const int grid = (int)((count + 256) / 256 < (int64_t)sm_count * 8 ? (count + 256) / 256 : (int64_t)sm_count * 8);
    cudaError_t e = cudaMalloc(&flags, sizeof(int32_t) * ((size_t)count + 1));
    if (e == cudaSuccess) e = cudaMalloc(&st->pos_dev, sizeof(int32_t) * ((size_t)count + 1));
    if (e == cudaSuccess) e = cub::DeviceScan::ExclusiveSum(nullptr, tmp_bytes, flags, st->pos_dev, count + 1);
    if (e == cudaSuccess) e = cudaMalloc(&tmp, tmp_bytes > 0 ? tmp_bytes : 1);
    if (e == cudaSuccess) {
        stage_flag_kernel<<<grid, 256>>>(ids_dev, count, c->lut, c->n_nodes, flags);
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cub::DeviceScan::ExclusiveSum(tmp, tmp_bytes, flags, st->pos_dev, count + 1);
    if (e == cudaSuccess) {
        st->pos = new int32_t[(size_t)count + 1];
        e = cudaMemcpy(st->pos, st->pos_dev, sizeof(int32_t) * ((size_t)count + 1), cudaMemcpyDeviceToHost);
    }
    cudaFree(flags);
    cudaFree(tmp);
    if (e == cudaSuccess) {
        const int64_t rows = st->pos[count];
        st->rows = rows;
        if (rows > 0) {
            e = cudaHostAlloc(reinterpret_cast<void **>(&st->rows_host), (size_t)rows * c->row_bytes, cudaHostAllocMapped);
            if (e == cudaSuccess) {
                const int64_t want = ((int64_t)count + 7) / 8;
                const int cgrid = (int)(want < (int64_t)sm_count * 8 ? want : (int64_t)sm_count * 8);
                stage_copy_kernel<<<cgrid, 256>>>(ids_dev, count, c->lut, st->pos_dev, (const uint8_t *)c->host_table, c->n_nodes,
                                                  c->row_bytes, st->rows_host);
                e = cudaGetLastError();
            }
            if (e == cudaSuccess) e = cudaDeviceSynchronize();
        }
    }
    if (e != cudaSuccess) {
        cudaGetLastError();
        set_error("seed staging: %s", cudaGetErrorString(e));
        stage_free(st);
        return e == cudaErrorMemoryAllocation ? LEGION_E_NOMEM : LEGION_E_CUDA;
    }
    st->valid = 1;
    return LEGION_OK;
}

}  // namespace legion
