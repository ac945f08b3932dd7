// Test infrastructure: drives the REFERENCE's own cache kernels on a GPU so that the CUDA library can
// be compared with them on the same inputs.  Nothing of the reference is copied: this file only
// includes sampling_server/src/cache/cache_impl.cuh (and, through it, the bucketed cuckoo hash table
// under include/hashmap) from where the reference lies, and calls its kernels in the order
// PreSCCacheController::InitializeMap / Insert / FindFeat (cache/cache.cu:74-192) and
// UnifiedCache::FillUp / FeatCacheLookup (cache/cache.cu:559-656,743-781) call them.  The binary is
// built into oracle/_ref/ by oracle/Makefile when the reference tree is present.
//
//   ref_cache_driver <in.bin> <out.bin>
//   in : int64 n_nodes, feat_len, capacity, kg, dev_in_clique, n_ids ; int32 QF[n_nodes] ;
//        float table[n_nodes*feat_len] ; int32 ids[n_ids]
//   out: int32 cache_index[n_ids] ; float rows[n_ids*feat_len]
//
// The clique of kg GPUs is emulated on one device: every member's partition is a separate
// allocation on it, reached through the float** pointer table exactly like peer memory.
#include "cache_impl.cuh"

#include <cstdio>
#include <cstdlib>
#include <vector>

#define CK(x)                                                                        \
    do {                                                                             \
        cudaError_t e_ = (x);                                                        \
        if (e_ != cudaSuccess) {                                                     \
            fprintf(stderr, "%s:%d %s\n", __FILE__, __LINE__, cudaGetErrorString(e_)); \
            return 2;                                                                \
        }                                                                            \
    } while (0)

int main(int argc, char **argv)
{
    if (argc != 3) return 1;
    FILE *f = fopen(argv[1], "rb");
    if (!f) return 1;
    int64_t hdr[6];
    if (fread(hdr, 8, 6, f) != 6) return 1;
    const int64_t n_nodes = hdr[0], feat_len = hdr[1], capacity = hdr[2], kg = hdr[3], dev_in_clique = hdr[4], n_ids = hdr[5];
    std::vector<int32_t> qf(n_nodes), ids(n_ids);
    float *cpu_features = nullptr;
    CK(cudaHostAlloc(&cpu_features, sizeof(float) * n_nodes * feat_len, cudaHostAllocMapped));  // storage_management.cu:171
    if (fread(qf.data(), 4, n_nodes, f) != (size_t)n_nodes) return 1;
    if (fread(cpu_features, 4, n_nodes * feat_len, f) != (size_t)(n_nodes * feat_len)) return 1;
    if (fread(ids.data(), 4, n_ids, f) != (size_t)n_ids) return 1;
    fclose(f);

    int32_t *d_qf = nullptr, *d_ids = nullptr, *d_cache_index = nullptr, *d_nc = nullptr;
    CK(cudaMalloc(&d_qf, 4 * n_nodes));
    CK(cudaMemcpy(d_qf, qf.data(), 4 * n_nodes, cudaMemcpyHostToDevice));
    CK(cudaMalloc(&d_ids, 4 * n_ids));
    CK(cudaMemcpy(d_ids, ids.data(), 4 * n_ids, cudaMemcpyHostToDevice));
    CK(cudaMalloc(&d_cache_index, 8 * n_ids));
    CK(cudaMalloc(&d_nc, 64));

    // InitializeMap + Insert (cache.cu:74-112)
    auto *node_map = new bght::bcht<int32_t, int32_t>(int64_t(capacity * kg) * 2, CACHEMISS_FLAG, CACHEMISS_FLAG);
    pair_type *pair = nullptr;
    CK(cudaMalloc(&pair, sizeof(pair_type) * capacity * kg));
    cudaStream_t stream;
    CK(cudaStreamCreate(&stream));
    InitPair<<<dim3(80, 1), dim3(1024, 1)>>>(pair, d_qf, (int32_t)capacity, (int32_t)kg, (int32_t)kg);
    CK(cudaGetLastError());
    bool ok = node_map->insert(pair, pair + capacity * kg, stream);
    CK(cudaDeviceSynchronize());
    fprintf(stderr, "bcht insert ok=%d\n", (int)ok);

    // FillUp (cache.cu:601-622): one partition per clique member + the pointer table
    std::vector<float *> parts(kg);
    float **d_ptrs = nullptr;
    CK(cudaMalloc(&d_ptrs, sizeof(float *) * kg));
    for (int ki = 0; ki < kg; ++ki) {
        CK(cudaMalloc(&parts[ki], sizeof(float) * capacity * feat_len));
        FeatFillUp<<<dim3(128, 1), dim3(1024, 1)>>>((int32_t)capacity, (int32_t)feat_len, parts[ki], cpu_features, d_qf,
                                                     (int32_t)kg, ki);
        CK(cudaGetLastError());
        init_feature_cache<<<1, 1>>>(d_ptrs, parts[ki], ki);
        CK(cudaGetLastError());
    }
    CK(cudaDeviceSynchronize());

    // FindFeat (cache.cu:157-173) for one lookup op: op_id 1 reads nc[2], nc[3]
    int32_t nc[16] = { 0 };
    nc[2] = 0;
    nc[3] = (int32_t)n_ids;
    CK(cudaMemcpy(d_nc, nc, 64, cudaMemcpyHostToDevice));
    node_map->find(d_ids, d_ids + n_ids, d_cache_index, stream);
    CK(cudaStreamSynchronize(stream));

    // FeatCacheLookup (cache.cu:743-781)
    float *d_dst = nullptr;
    CK(cudaMalloc(&d_dst, sizeof(float) * n_ids * feat_len));
    CK(cudaMemset(d_dst, 0, sizeof(float) * n_ids * feat_len));
    multiGPU_feat_cache_lookup<<<dim3(64, 1), dim3(512, 1), 0, stream>>>(cpu_features, d_ptrs, (int32_t)feat_len, d_ids,
                                                                        d_cache_index, (int32_t)capacity, d_nc, d_dst,
                                                                        (int32_t)n_nodes, (int32_t)dev_in_clique, 1);
    CK(cudaGetLastError());
    CK(cudaStreamSynchronize(stream));

    std::vector<int32_t> h_ci(n_ids);
    std::vector<float> h_dst(n_ids * feat_len);
    CK(cudaMemcpy(h_ci.data(), d_cache_index, 4 * n_ids, cudaMemcpyDeviceToHost));
    CK(cudaMemcpy(h_dst.data(), d_dst, sizeof(float) * n_ids * feat_len, cudaMemcpyDeviceToHost));
    FILE *o = fopen(argv[2], "wb");
    if (!o) return 1;
    fwrite(h_ci.data(), 4, n_ids, o);
    fwrite(h_dst.data(), 4, n_ids * feat_len, o);
    fclose(o);
    return ok ? 0 : 3;
}
