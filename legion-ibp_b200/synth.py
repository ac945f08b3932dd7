"""Seeded synthetic inputs with the shapes of the benchmark configurations.

R-MAT topology (a=.57, b=.19, c=.19, d=.05), symmetrised, self loops dropped, duplicate edges
merged, CSR with int64 offsets and int32 indices as the reference stores it
(sampling_server/src/include/buildinfo.h:60-61); N(0,1) feature rows; uniform labels; random
seed split (dataset/gen_sets.py:62-76).  They stand in for the OGB datasets of
dataset_info.py:3-18,75-82, which are not available offline.  torch does the generation (on the
GPU for the large graphs); it is data synthesis, not part of the sampling path.
"""
import math

import torch


def rmat_csr(n_nodes, n_pairs, seed=0, device="cpu", a=0.57, b=0.19, c=0.19, chunk=1 << 26):
    """Returns (indptr int64 [n+1], indices int32 [E]) of the symmetrised R-MAT graph."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    scale = max(1, math.ceil(math.log2(n_nodes)))
    keys = []
    done = 0
    while done < n_pairs:
        m = min(chunk, n_pairs - done)
        u = torch.zeros(m, dtype=torch.int64, device=device)
        v = torch.zeros(m, dtype=torch.int64, device=device)
        for _ in range(scale):
            r = torch.rand(m, device=device, generator=g)
            ubit = (r >= a + b).to(torch.int64)                      # quadrants c, d
            vbit = (((r >= a) & (r < a + b)) | (r >= a + b + c)).to(torch.int64)  # quadrants b, d
            u = (u << 1) | ubit
            v = (v << 1) | vbit
        # spread the 2^scale id space over [0, n) and decorrelate id from degree
        u = (u * n_nodes) >> scale
        v = (v * n_nodes) >> scale
        mult = _coprime_multiplier(n_nodes)
        u = (u * mult + 12345) % n_nodes
        v = (v * mult + 12345) % n_nodes
        keep = u != v
        u, v = u[keep], v[keep]
        keys.append(u * n_nodes + v)
        keys.append(v * n_nodes + u)
        done += m
        del r, ubit, vbit, keep
    key = torch.cat(keys)
    del keys
    key = torch.unique(key)  # sorted, duplicates merged
    src = torch.div(key, n_nodes, rounding_mode="floor")
    indices = (key - src * n_nodes).to(torch.int32)
    del key
    counts = torch.bincount(src, minlength=n_nodes)
    del src
    indptr = torch.zeros(n_nodes + 1, dtype=torch.int64, device=device)
    torch.cumsum(counts, 0, out=indptr[1:])
    return indptr, indices


def _coprime_multiplier(n):
    m = 2654435761 % n
    if m < 2:
        m = 2
    while math.gcd(m, n) != 1:
        m += 1
    return m


def features_into(out, seed=0, chunk_rows=1 << 20):
    """Fills a [N, F] tensor (pinned host or device) with N(0,1) values, chunk by chunk."""
    n = out.shape[0]
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    for r0 in range(0, n, chunk_rows):
        r1 = min(n, r0 + chunk_rows)
        blk = torch.randn(r1 - r0, out.shape[1], device=dev, generator=g, dtype=torch.float32).to(out.dtype)
        out[r0:r1].copy_(blk, non_blocking=False)
    return out


def labels_and_split(n_nodes, n_classes, train_frac, seed=0, device="cpu", valid_frac=0.0, test_frac=0.0):
    """Uniform labels and a random split; returns (labels int32 [N], train, valid, test id tensors)."""
    g = torch.Generator(device=device)
    g.manual_seed(seed + 1)
    labels = torch.randint(0, n_classes, (n_nodes,), device=device, generator=g, dtype=torch.int32)
    perm_key = torch.rand(n_nodes, device=device, generator=g)
    n_train = int(n_nodes * train_frac)
    n_valid = int(n_nodes * valid_frac)
    n_test = int(n_nodes * test_frac)
    order = torch.argsort(perm_key)[: n_train + n_valid + n_test].to(torch.int32)
    return labels, order[:n_train].contiguous(), order[n_train:n_train + n_valid].contiguous(), \
        order[n_train + n_valid:].contiguous()


def zipf_seeds(n_nodes, count, s=1.1, seed=0, device="cpu"):
    """`count` node ids drawn Zipf(s) over node id (rank = id + 1), by inverse-CDF on a bounded support."""
    g = torch.Generator(device=device)
    g.manual_seed(seed + 2)
    u = torch.rand(count, device=device, generator=g, dtype=torch.float64)
    # continuous approximation of the bounded Zipf CDF: F(x) = (x^(1-s) - 1) / (N^(1-s) - 1)
    e = 1.0 - s
    x = (u * (float(n_nodes) ** e - 1.0) + 1.0) ** (1.0 / e)
    return (x.clamp(1, n_nodes).to(torch.int64) - 1).to(torch.int32)
