// Legion-format datasets and the meta_config line: what StorageManagement reads at start-up
// (sampling_server/src/storage/storage_management.cu:33-279, storage_management_impl.cuh:48-196;
// file list in dataset/README.md:4-10; the line itself is written by legion_server.py:45-46).
//
//   <dir>/edge_src      int64  CSR offsets, node_num + 1 entries
//   <dir>/edge_dst      int32  CSR neighbour ids, edge_num entries
//   <feat dir>/features float32 node_num x float_feature_len, row-major
//   <dir>/labels        int32  one per node
//   <dir>/trainingset, validationset, testingset   int32 node ids
//   <dir>/partition     int32  owner GPU per node (optional; without it seeds are split id % ngpu)
//
// Topology and features land in mapped pinned host memory (cudaHostAlloc) so that kernels can
// read them in place, exactly where the reference keeps them; with pin == 0 plain host memory is
// used, which lets the loader run (and be tested) on machines without a GPU.
#include "common.cuh"

#include <errno.h>
#include <fcntl.h>
#include <string.h>
#include <sys/stat.h>
#include <unistd.h>

#include <string>
#include <vector>

struct LegionDataset {
    LegionMetaConfig meta;
    int32_t pinned;
    int64_t *indptr;
    int32_t *indices;
    float *features;
    std::vector<int32_t> labels, sets[3], partition;
    bool has_partition;
};

using namespace legion;

static int read_whole(const std::string &path, void *dst, int64_t want_bytes, bool exact, int64_t *got)
{
    int fd = open(path.c_str(), O_RDONLY);
    if (fd < 0) {
        set_error("cannot open file: %s (%s)", path.c_str(), strerror(errno));  // storage_management_impl.cuh:51-53
        return LEGION_E_SYS;
    }
    struct stat st;
    if (fstat(fd, &st) != 0) {
        close(fd);
        set_error("cannot stat %s", path.c_str());
        return LEGION_E_SYS;
    }
    if ((exact && st.st_size != want_bytes) || st.st_size < want_bytes) {
        close(fd);
        set_error("%s holds %lld bytes, %lld expected from meta_config", path.c_str(), (long long)st.st_size,
                  (long long)want_bytes);
        return LEGION_E_ARG;
    }
    int64_t done = 0;
    while (done < want_bytes) {
        ssize_t r = read(fd, (char *)dst + done, (size_t)((want_bytes - done) > (1ll << 30) ? (1ll << 30) : (want_bytes - done)));
        if (r <= 0) {
            close(fd);
            set_error("short read on %s", path.c_str());
            return LEGION_E_SYS;
        }
        done += r;
    }
    close(fd);
    if (got) *got = done;
    return LEGION_OK;
}

static void *host_alloc(int64_t bytes, int pinned)
{
    void *p = nullptr;
    if (bytes <= 0) bytes = 8;
    if (pinned) {
        if (cudaHostAlloc(&p, (size_t)bytes, cudaHostAllocMapped) != cudaSuccess) return nullptr;  // storage_management.cu:114-115,171
    } else {
        p = malloc((size_t)bytes);
    }
    return p;
}

static void host_free(void *p, int pinned)
{
    if (p == nullptr) return;
    if (pinned) cudaFreeHost(p); else free(p);
}

// ReadMetaFIle, in-memory mode (storage_management.cu:33-68): one line,
// "path batch nodes edges feature_dim ntrain nvalid ntest cache_bytes epochs [feature_path]".
extern "C" int legion_meta_config_read(const char *file, LegionMetaConfig *out)
{
    LG_ARG(file != nullptr && out != nullptr, "NULL pointer");
    FILE *f = fopen(file, "r");
    if (!f) {
        set_error("unable to open meta config file %s", file);
        return LEGION_E_SYS;
    }
    memset(out, 0, sizeof(*out));
    long long nodes = 0, edges = 0, cache = 0;
    int n = fscanf(f, "%511s %d %lld %lld %d %d %d %d %lld %d %511s", out->dataset_path, &out->raw_batch_size, &nodes, &edges,
                   &out->float_feature_len, &out->training_set_num, &out->validation_set_num, &out->testing_set_num, &cache,
                   &out->epoch, out->feature_path);
    fclose(f);
    if (n < 10) {
        set_error("meta config %s: %d fields parsed, at least 10 expected", file, n);
        return LEGION_E_ARG;
    }
    out->node_num = nodes;
    out->edge_num = edges;
    out->cache_memory = cache;
    if (n < 11) snprintf(out->feature_path, sizeof(out->feature_path), "%s", out->dataset_path);
    return LEGION_OK;
}

// legion_server.py:45-46
extern "C" int legion_meta_config_write(const char *file, const LegionMetaConfig *m)
{
    LG_ARG(file != nullptr && m != nullptr, "NULL pointer");
    FILE *f = fopen(file, "w");
    if (!f) {
        set_error("unable to write meta config file %s", file);
        return LEGION_E_SYS;
    }
    fprintf(f, "%s %d %lld %lld %d %d %d %d %lld %d %s\n", m->dataset_path, m->raw_batch_size, (long long)m->node_num,
            (long long)m->edge_num, m->float_feature_len, m->training_set_num, m->validation_set_num, m->testing_set_num,
            (long long)m->cache_memory, m->epoch, m->feature_path[0] ? m->feature_path : m->dataset_path);
    fclose(f);
    return LEGION_OK;
}

extern "C" int legion_dataset_destroy(LegionDataset *d)
{
    if (d == nullptr) return LEGION_OK;
    host_free(d->indptr, d->pinned);
    host_free(d->indices, d->pinned);
    host_free(d->features, d->pinned);
    delete d;
    return LEGION_OK;
}

// LoadGraph + LoadFeature (storage_management.cu:106-279) without the per-GPU split.
extern "C" int legion_dataset_load(LegionDataset **out, const LegionMetaConfig *meta, int32_t pin, int32_t load_features)
{
    LG_ARG(out != nullptr && meta != nullptr, "NULL pointer");
    LG_ARG(meta->node_num > 0 && meta->node_num < (1ll << 31) && meta->edge_num >= 0, "bad node or edge count");
    LG_ARG(meta->float_feature_len > 0, "bad feature length");
    LegionDataset *d = new LegionDataset();
    d->meta = *meta;
    d->pinned = pin ? 1 : 0;
    d->indptr = nullptr; d->indices = nullptr; d->features = nullptr;
    d->has_partition = false;
    std::string dir = meta->dataset_path, fdir = meta->feature_path[0] ? meta->feature_path : meta->dataset_path;
    if (!dir.empty() && dir.back() != '/') dir += "/";
    if (!fdir.empty() && fdir.back() != '/') fdir += "/";
    const int64_t n = meta->node_num, e = meta->edge_num, f = meta->float_feature_len;
    int rc = LEGION_OK;
    d->indptr = (int64_t *)host_alloc(8 * (n + 1), d->pinned);
    d->indices = (int32_t *)host_alloc(4 * e, d->pinned);
    if (load_features) d->features = (float *)host_alloc(4 * n * f, d->pinned);
    if (!d->indptr || !d->indices || (load_features && !d->features)) {
        set_error("legion_dataset_load: host allocation failed");
        rc = LEGION_E_NOMEM;
    }
    if (rc == LEGION_OK) rc = read_whole(dir + "edge_src", d->indptr, 8 * (n + 1), true, nullptr);
    if (rc == LEGION_OK) rc = read_whole(dir + "edge_dst", d->indices, 4 * e, true, nullptr);
    if (rc == LEGION_OK && (d->indptr[0] != 0 || d->indptr[n] != e)) {
        set_error("edge_src is not a CSR offset array for %lld edges", (long long)e);
        rc = LEGION_E_ARG;
    }
    if (rc == LEGION_OK && load_features) rc = read_whole(fdir + "features", d->features, 4 * n * f, false, nullptr);
    if (rc == LEGION_OK) {
        d->labels.resize(n);
        rc = read_whole(dir + "labels", d->labels.data(), 4 * n, false, nullptr);
    }
    const char *names[3] = { "trainingset", "validationset", "testingset" };
    const int32_t counts[3] = { meta->training_set_num, meta->validation_set_num, meta->testing_set_num };
    for (int m = 0; m < 3 && rc == LEGION_OK; ++m) {
        d->sets[m].resize(counts[m] > 0 ? counts[m] : 0);
        if (counts[m] > 0) rc = read_whole(dir + names[m], d->sets[m].data(), 4ll * counts[m], false, nullptr);
        for (int32_t v : d->sets[m])
            if (rc == LEGION_OK && (v < 0 || v >= n)) {
                set_error("%s holds node id %d outside [0, %lld)", names[m], v, (long long)n);
                rc = LEGION_E_ARG;
            }
    }
    if (rc == LEGION_OK) {
        std::string pfile = dir + "partition";
        if (access(pfile.c_str(), R_OK) == 0) {  // optional, storage_management.cu:176-180
            d->partition.resize(n);
            rc = read_whole(pfile, d->partition.data(), 4 * n, false, nullptr);
            d->has_partition = rc == LEGION_OK;
        }
    }
    if (rc != LEGION_OK) {
        legion_dataset_destroy(d);
        return rc;
    }
    *out = d;
    return LEGION_OK;
}

extern "C" int legion_dataset_arrays(LegionDataset *d, const int64_t **indptr, const int32_t **indices,
                                     const float **features, const int32_t **labels)
{
    LG_ARG(d != nullptr, "dataset is NULL");
    if (indptr) *indptr = d->indptr;
    if (indices) *indices = d->indices;
    if (features) *features = d->features;
    if (labels) *labels = d->labels.data();
    return LEGION_OK;
}

// ---- host table packed by rank -------------------------------------------------------------------------------
// The reference keeps the feature table in node-id order (cpu_float_features[id * F], cache/cache_impl.cuh:283-286;
// loaded by storage/storage_management.cu:160-175).  Random zero-copy reads of widely scattered host pages are
// slow on this platform, and the rows that miss a ranked cache are not spread evenly: the better a node's rank,
// the more often it is asked for.  Packed order: the rows of the nodes that the clique's caches do NOT hold, by
// rising rank (the likeliest misses next to each other), followed by the rows of the cached nodes (read once, at
// fill time).  row of rank t = t - n_cached for t >= n_cached, n - n_cached + t otherwise.
__global__ void pack_row_of_kernel(const int32_t *__restrict__ order, int64_t n, int64_t n_cached, int32_t *row_of)
{
    for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < n; t += (int64_t)gridDim.x * blockDim.x)
        row_of[order[t]] = (int32_t)(t >= n_cached ? t - n_cached : n - n_cached + t);
}

// one warp per destination row; source and destination are page-locked host memory
__global__ void __launch_bounds__(256)
pack_rows_kernel(const uint8_t *__restrict__ src, uint8_t *dst, const int32_t *__restrict__ order, int64_t n, int64_t n_cached,
                 int64_t row_bytes)
{
    const int lane = threadIdx.x & 31;
    const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t r = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < n; r += n_warps) {
        const int64_t t = r < n - n_cached ? r + n_cached : r - (n - n_cached);
        const uint32_t *s4 = reinterpret_cast<const uint32_t *>(src + (int64_t)order[t] * row_bytes);
        uint32_t *d4 = reinterpret_cast<uint32_t *>(dst + r * row_bytes);
        for (int64_t w = lane; w < (row_bytes >> 2); w += 32) d4[w] = s4[w];
    }
}

extern "C" int legion_cache_pack_order(int32_t dev_id, const int32_t *order_dev, int64_t n_nodes, int64_t n_cached,
                                       int32_t *row_of_dev, void *stream)
{
    LG_ARG(order_dev != nullptr && row_of_dev != nullptr, "NULL pointer");
    LG_ARG(n_nodes > 0 && n_nodes < (1ll << 31) && n_cached >= 0 && n_cached <= n_nodes, "bad counts");
    LG_CUDA(cudaSetDevice(dev_id));
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev_id);
    pack_row_of_kernel<<<sms * 8, 256, 0, (cudaStream_t)stream>>>(order_dev, n_nodes, n_cached, row_of_dev);
    LG_LAUNCH_CHECK();
    LG_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    return LEGION_OK;
}

extern "C" int legion_dataset_pack_features(LegionDataset *d, int32_t dev_id, const int32_t *order_dev, int64_t n_cached)
{
    LG_ARG(d != nullptr && d->features != nullptr && d->pinned, "the dataset needs its features in page-locked memory");
    LG_ARG(order_dev != nullptr && n_cached >= 0 && n_cached <= d->meta.node_num, "bad order or count");
    LG_CUDA(cudaSetDevice(dev_id));
    const int64_t n = d->meta.node_num, row_bytes = 4ll * d->meta.float_feature_len;
    float *packed = (float *)host_alloc(n * row_bytes, 1);
    if (packed == nullptr) {
        set_error("legion_dataset_pack_features: no page-locked memory for a second copy of the table (%lld bytes)",
                  (long long)(n * row_bytes));
        return LEGION_E_NOMEM;
    }
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev_id);
    pack_rows_kernel<<<sms * 8, 256>>>((const uint8_t *)d->features, (uint8_t *)packed, order_dev, n, n_cached, row_bytes);
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        host_free(packed, 1);
        LG_CUDA(e);
    }
    host_free(d->features, 1);
    d->features = packed;
    return LEGION_OK;
}

// The seeds of one GPU for one mode (storage_management.cu:214-250): owner = partition[id] when a
// partition file exists (training set only, as in the reference), else id % partition_count.  List
// order is kept.  Call with ids_out == NULL to get the count.
extern "C" int legion_dataset_split(LegionDataset *d, int32_t mode, int32_t partition_count, int32_t part_id,
                                    int32_t *ids_out, int32_t *labels_out, int32_t *count_out)
{
    LG_ARG(d != nullptr && count_out != nullptr, "NULL pointer");
    LG_ARG(mode >= 0 && mode <= 2, "mode must be 0, 1 or 2");
    LG_ARG(partition_count >= 1 && part_id >= 0 && part_id < partition_count, "bad partition");
    int32_t k = 0;
    for (int32_t v : d->sets[mode]) {
        int32_t owner = (mode == 0 && d->has_partition) ? d->partition[v] : v % partition_count;
        if (owner != part_id) continue;
        if (ids_out) ids_out[k] = v;
        if (labels_out) labels_out[k] = d->labels[v];
        ++k;
    }
    *count_out = k;
    return LEGION_OK;
}
