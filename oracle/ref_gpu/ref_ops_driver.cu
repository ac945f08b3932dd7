// Test infrastructure: drives the REFERENCE's own operator kernels on a GPU -- batch_generate,
// counter_update, construct_graph and ClearPosMap of sampling_server/src/engine/operator_impl.cu:28-91,
// 304-317,598-604 -- so that the CUDA library and the CPU checker can be compared with them on the same
// inputs.  Nothing of the reference is copied: this file includes engine/operator_impl.cu from where the
// reference lies and launches its kernels with the grids and in the order that BatchGenerate /
// RandomSample / FeatureCacheLookup / IOComplete use (operator_impl.cu:158-168,497-540,571,631-634).
//
// random_sample / pre_sample are NOT run: they call __syncthreads() under loop trip counts that differ
// between the threads of a block (operator_impl.cu:212-301), which may hang a GPU, and their picks are
// neither seedable nor reproducible.  Their outputs are fed in instead: for every hop the sampled edges
// (neighbour id, id of the node it was sampled for) and the new nodes in the order they were appended,
// written exactly where random_sample writes them (operator_impl.cu:107-121).
//
//   ref_ops_driver <in.bin> <out.bin>
//   in : int64 n_nodes, batch_size, counter, total_cap, hop_num ; int32 all_ids[total_cap] ;
//        int32 all_labels[total_cap] ; per hop: int64 E, C ; int32 src[E] ; int32 dst[E] ; int32 new_nodes[C]
//   out: int32 trace[2 + 2 * hop_num][32] (node_counter, edge_counter after op 0, op 1, and after ops 3h, 3h+1
//        of every hop) ; int32 sampled_ids[total] ; int32 labels[size] ; int32 agg_src_off[edges] ;
//        int32 agg_dst_off[edges] ; int64 entries of position_map that are non-zero after ClearPosMap
//
// The binary is built into oracle/_ref/ by oracle/Makefile when the reference tree is present.
#include "operator_impl.cu"

#include <cstdio>
#include <cstdlib>
#include <vector>

// The operator entry points of the included file call into UnifiedCache, whose implementation needs the
// absent compression library; none of them is called here.
static void not_linked() { fprintf(stderr, "ref_ops_driver: a UnifiedCache method was called\n"); abort(); }
void UnifiedCache::FindFeat(int32_t *, int32_t *, int32_t *, int32_t, void *, int32_t) { not_linked(); }
void UnifiedCache::FindTopo(int32_t *, char *, int32_t *, int32_t, int32_t, void *, int32_t) { not_linked(); }
void UnifiedCache::CacheProfiling(int32_t *, int32_t *, int32_t *, int32_t *, int32_t *, int32_t *, int32_t *, void *, int32_t) { not_linked(); }
unsigned long long int *UnifiedCache::GetEdgeAccessedMap(int32_t) { not_linked(); return nullptr; }
void UnifiedCache::FeatCacheLookup(int32_t *, int32_t *, int32_t *, float *, int32_t, int32_t, cudaStream_t) { not_linked(); }

#define CK(x)                                                                        \
    do {                                                                             \
        cudaError_t e_ = (x);                                                        \
        if (e_ != cudaSuccess) {                                                     \
            fprintf(stderr, "%s:%d %s\n", __FILE__, __LINE__, cudaGetErrorString(e_)); \
            return 2;                                                                \
        }                                                                            \
    } while (0)

// what random_sample does with a new node (operator_impl.cu:112-115): append it and remember its position
__global__ void append_new_nodes(const int32_t *new_nodes, int32_t count, int32_t node_base, int32_t *sampled_ids,
                                 int32_t *position_map)
{
    for (int32_t i = threadIdx.x + blockDim.x * blockIdx.x; i < count; i += gridDim.x * blockDim.x) {
        sampled_ids[node_base + i] = new_nodes[i];
        position_map[new_nodes[i]] = node_base + i;
    }
}

__global__ void count_nonzero(const int32_t *a, int64_t n, unsigned long long *out)
{
    for (int64_t i = threadIdx.x + (int64_t)blockDim.x * blockIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        if (a[i] != 0) atomicAdd(out, 1ull);
}

int main(int argc, char **argv)
{
    if (argc != 3) return 1;
    FILE *f = fopen(argv[1], "rb");
    if (!f) return 1;
    int64_t hdr[5];
    if (fread(hdr, 8, 5, f) != 5) return 1;
    const int64_t n_nodes = hdr[0], batch_size = hdr[1], counter = hdr[2], total_cap = hdr[3], hop_num = hdr[4];
    if (n_nodes <= 0 || batch_size <= 0 || total_cap <= 0 || hop_num < 0 || hop_num > 3) return 1;
    std::vector<int32_t> all_ids(total_cap), all_labels(total_cap);
    if (fread(all_ids.data(), 4, total_cap, f) != (size_t)total_cap) return 1;
    if (fread(all_labels.data(), 4, total_cap, f) != (size_t)total_cap) return 1;
    std::vector<std::vector<int32_t>> h_src(hop_num), h_dst(hop_num), h_new(hop_num);
    int64_t tot_e = 0, tot_c = 0;
    for (int h = 0; h < hop_num; ++h) {
        int64_t ec2[2];
        if (fread(ec2, 8, 2, f) != 2) return 1;
        h_src[h].resize(ec2[0]); h_dst[h].resize(ec2[0]); h_new[h].resize(ec2[1]);
        if (ec2[0] && fread(h_src[h].data(), 4, ec2[0], f) != (size_t)ec2[0]) return 1;
        if (ec2[0] && fread(h_dst[h].data(), 4, ec2[0], f) != (size_t)ec2[0]) return 1;
        if (ec2[1] && fread(h_new[h].data(), 4, ec2[1], f) != (size_t)ec2[1]) return 1;
        tot_e += ec2[0];
        tot_c += ec2[1];
    }
    fclose(f);
    // every id that will index position_map / accessed_map must be a node (checked here, on the host)
    for (int64_t i = 0; i < total_cap; ++i) if (all_ids[i] < 0 || all_ids[i] >= n_nodes) return 3;
    for (int h = 0; h < hop_num; ++h) {
        for (int32_t v : h_src[h]) if (v < 0 || v >= n_nodes) return 3;
        for (int32_t v : h_dst[h]) if (v < 0 || v >= n_nodes) return 3;
        for (int32_t v : h_new[h]) if (v < 0 || v >= n_nodes) return 3;
    }
    // BatchGenerate's size (operator_impl.cu:162); only whole batches are driven (the kernel is handed
    // `size` where it multiplies by the batch size, which differs for a shortened last batch)
    const int32_t size = (batch_size * (counter + 1) >= total_cap) ? (int32_t)(total_cap - batch_size * counter) : (int32_t)batch_size;
    if (size != batch_size) return 4;
    const int64_t max_nodes = size + tot_c, max_edges = tot_e > 0 ? tot_e : 1;

    int32_t *d_all_ids, *d_all_labels, *sampled_ids, *labels, *position_map, *nc, *ec;
    int32_t *agg_src_ids, *agg_dst_ids, *agg_src_off, *agg_dst_off, *d_new;
    uint32_t *accessed_map;
    unsigned long long *d_cnt;
    CK(cudaMalloc(&d_all_ids, 4 * total_cap));
    CK(cudaMalloc(&d_all_labels, 4 * total_cap));
    CK(cudaMemcpy(d_all_ids, all_ids.data(), 4 * total_cap, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(d_all_labels, all_labels.data(), 4 * total_cap, cudaMemcpyHostToDevice));
    CK(cudaMalloc(&sampled_ids, 4 * max_nodes));
    CK(cudaMalloc(&labels, 4 * size));
    CK(cudaMalloc(&position_map, 4 * n_nodes));
    CK(cudaMemset(position_map, 0, 4 * n_nodes));
    CK(cudaMalloc(&accessed_map, 4 * (n_nodes / 32 + 1)));
    CK(cudaMalloc(&nc, 64));
    CK(cudaMalloc(&ec, 64));
    CK(cudaMalloc(&agg_src_ids, 4 * max_edges));
    CK(cudaMalloc(&agg_dst_ids, 4 * max_edges));
    CK(cudaMalloc(&agg_src_off, 4 * max_edges));
    CK(cudaMalloc(&agg_dst_off, 4 * max_edges));
    CK(cudaMalloc(&d_new, 4 * (tot_c > 0 ? tot_c : 1)));
    CK(cudaMalloc(&d_cnt, 8));
    cudaStream_t s;
    CK(cudaStreamCreate(&s));

    std::vector<int32_t> trace;
    auto snap = [&]() -> int {
        int32_t h[32];
        CK(cudaStreamSynchronize(s));
        CK(cudaMemcpy(h, nc, 64, cudaMemcpyDeviceToHost));
        CK(cudaMemcpy(h + 16, ec, 64, cudaMemcpyDeviceToHost));
        trace.insert(trace.end(), h, h + 32);
        return 0;
    };

    // BatchGenerate (operator_impl.cu:154-168)
    CK(cudaMemsetAsync(accessed_map, 0, (n_nodes / 32 + 1) * sizeof(uint32_t), s));
    CK(cudaMemsetAsync(nc, 0, 64, s));
    CK(cudaMemsetAsync(ec, 0, 64, s));
    batch_generate<<<(size - 1) / OP_THREAD_NUM + 1, OP_THREAD_NUM, 0, s>>>(sampled_ids, labels, size, (int32_t)counter, d_all_ids,
                                                                            d_all_labels, (int32_t)total_cap, position_map, accessed_map);
    CK(cudaGetLastError());
    counter_update<<<1, 1, 0, s>>>(nc, ec, 0, size, (int32_t)hop_num);
    CK(cudaGetLastError());
    if (snap()) return 2;
    // FeatureCacheLookup of the seeds (operator_impl.cu:571)
    counter_update<<<1, 1, 0, s>>>(nc, ec, 1, 0, 0);
    CK(cudaGetLastError());
    if (snap()) return 2;
    for (int h = 0; h < hop_num; ++h) {
        const int32_t op = INTRABATCH_CON * (h + 1);
        const int32_t *hn = &trace[trace.size() - 32];
        const int32_t node_base = hn[0] + hn[1], edge_base = hn[16] + hn[17];
        const int32_t E = (int32_t)h_src[h].size(), C = (int32_t)h_new[h].size();
        if (node_base + C > max_nodes || edge_base + E > max_edges) return 3;
        // random_sample's output (operator_impl.cu:107-121)
        if (E) CK(cudaMemcpyAsync(agg_src_ids + edge_base, h_src[h].data(), 4 * E, cudaMemcpyHostToDevice, s));
        if (E) CK(cudaMemcpyAsync(agg_dst_ids + edge_base, h_dst[h].data(), 4 * E, cudaMemcpyHostToDevice, s));
        if (C) {
            CK(cudaMemcpyAsync(d_new, h_new[h].data(), 4 * C, cudaMemcpyHostToDevice, s));
            append_new_nodes<<<64, 256, 0, s>>>(d_new, C, node_base, sampled_ids, position_map);
            CK(cudaGetLastError());
        }
        CK(cudaMemcpyAsync(nc + INTRABATCH_CON * 2, &C, 4, cudaMemcpyHostToDevice, s));
        CK(cudaMemcpyAsync(ec + 2, &E, 4, cudaMemcpyHostToDevice, s));
        CK(cudaStreamSynchronize(s));
        // RandomSample's tail (operator_impl.cu:523-528) and the lookup of the hop's nodes (:571)
        construct_graph<<<16, OP_THREAD_NUM, 0, s>>>(agg_src_ids, agg_dst_ids, agg_src_off, agg_dst_off, position_map, ec, nc, op, 0);
        CK(cudaGetLastError());
        counter_update<<<1, 1, 0, s>>>(nc, ec, op, 0, 0);
        CK(cudaGetLastError());
        if (snap()) return 2;
        counter_update<<<1, 1, 0, s>>>(nc, ec, op + 1, 0, 0);
        CK(cudaGetLastError());
        if (snap()) return 2;
    }
    const int32_t *fin = &trace[trace.size() - 32];
    const int64_t n_total = fin[INTRABATCH_CON * 3 + hop_num];
    const int64_t e_total = (int64_t)fin[16] + fin[17];
    std::vector<int32_t> o_ids(n_total), o_lab(size), o_src(e_total > 0 ? e_total : 1), o_dst(e_total > 0 ? e_total : 1);
    CK(cudaMemcpy(o_ids.data(), sampled_ids, 4 * n_total, cudaMemcpyDeviceToHost));
    CK(cudaMemcpy(o_lab.data(), labels, 4 * size, cudaMemcpyDeviceToHost));
    if (e_total) CK(cudaMemcpy(o_src.data(), agg_src_off, 4 * e_total, cudaMemcpyDeviceToHost));
    if (e_total) CK(cudaMemcpy(o_dst.data(), agg_dst_off, 4 * e_total, cudaMemcpyDeviceToHost));
    // IOComplete (operator_impl.cu:631-634)
    ClearPosMap<<<32, OP_THREAD_NUM, 0, s>>>(position_map, sampled_ids, nc);
    CK(cudaGetLastError());
    CK(cudaMemsetAsync(d_cnt, 0, 8, s));
    count_nonzero<<<256, 256, 0, s>>>(position_map, n_nodes, d_cnt);
    CK(cudaGetLastError());
    unsigned long long nonzero = 0;
    CK(cudaStreamSynchronize(s));
    CK(cudaMemcpy(&nonzero, d_cnt, 8, cudaMemcpyDeviceToHost));

    FILE *o = fopen(argv[2], "wb");
    if (!o) return 1;
    fwrite(trace.data(), 4, trace.size(), o);
    fwrite(o_ids.data(), 4, n_total, o);
    fwrite(o_lab.data(), 4, size, o);
    fwrite(o_src.data(), 4, e_total, o);
    fwrite(o_dst.data(), 4, e_total, o);
    int64_t nz = (int64_t)nonzero;
    fwrite(&nz, 8, 1, o);
    fclose(o);
    return 0;
}
