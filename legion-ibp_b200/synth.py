"""Seeded synthetic inputs with the shapes of the benchmark configurations.

R-MAT topology (a=.57, b=.19, c=.19, d=.05), symmetrised, self loops dropped, duplicate edges
merged, CSR with int64 offsets and int32 indices as the reference stores it
(sampling_server/src/include/buildinfo.h:60-61); bell-shaped feature rows of mean 0 and variance 1 that
are a pure function of the node id; uniform labels; random
seed split (dataset/gen_sets.py:62-76).  They stand in for the OGB datasets of
dataset_info.py:3-18,75-82, which are not available offline.  torch does the generation (on the
GPU for the large graphs); it is data synthesis, not part of the sampling path.
"""
import math

import torch


def rmat_csr(n_nodes, n_pairs, seed=0, device="cpu", a=0.57, b=0.19, c=0.19, chunk=1 << 26, max_sort=1 << 30):
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
    total = sum(int(k.numel()) for k in keys)
    # The sort behind torch.unique takes fewer than 2^31 keys: larger edge lists are sorted bucket by bucket,
    # each bucket a range of source nodes (ids are scrambled, so the ranges hold about the same number of keys),
    # and the sorted buckets follow one another.
    n_buckets = max(1, -(-total // max_sort))
    counts = torch.zeros(n_nodes, dtype=torch.int64, device=device)
    parts = []
    for b in range(n_buckets):
        lo, hi = n_nodes * b // n_buckets, n_nodes * (b + 1) // n_buckets
        if n_buckets == 1:
            key = torch.cat(keys)
            keys = []
        else:
            key = torch.cat([k[(k >= lo * n_nodes) & (k < hi * n_nodes)] for k in keys])
        key = torch.unique(key)  # sorted, duplicates merged
        src = torch.div(key, n_nodes, rounding_mode="floor")
        parts.append((key - src * n_nodes).to(torch.int32))
        del key
        if src.numel():
            counts[lo:hi] += torch.bincount(src - lo, minlength=hi - lo)
        del src
    del keys
    indices = parts[0] if len(parts) == 1 else torch.cat(parts)
    del parts
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


_M32 = 0xFFFFFFFF


def _mix32(h):
    """murmur3 finaliser on the low 32 bits of an int64 tensor."""
    h = h ^ (h >> 16)
    h = (h * 0x85EBCA6B) & _M32
    h = h ^ (h >> 13)
    h = (h * 0xC2B2AE35) & _M32
    return h ^ (h >> 16)


def feature_rows(ids, feat_len, seed=0, dtype=torch.float32):
    """Feature rows of the given node ids, [len(ids), feat_len]: a pure function of (seed, id, column), so
    that any row of a table of any size can be made again on demand, on the host or on the device, with
    the same bits.  Every value is the standardised sum of four uniform bytes of a 32-bit hash (mean 0,
    variance 1, bell-shaped): the stand-in for the N(0,1) features of the benchmark configurations."""
    x = _mix32((ids.to(torch.int64) ^ ((seed * 0x9E3779B1 + 0x7F4A7C15) & _M32)) & _M32)
    col = (torch.arange(feat_len, device=ids.device, dtype=torch.int64) * 0x9E3779B9) & _M32
    h = _mix32((x[:, None] + col[None, :]) & _M32)
    s = (h & 255) + ((h >> 8) & 255) + ((h >> 16) & 255) + (h >> 24)
    # sum of four uniform bytes: mean 510, variance 4 * (256^2 - 1) / 12
    return ((s - 510).to(torch.float32) * (1.0 / 147.80054127)).to(dtype)


def features_into(out, seed=0, chunk_rows=1 << 18, row_ids=None, first=0, last=None):
    """Fills rows [first, last) of a [N, F] tensor (pinned host or device): row r holds the features of
    node r, or of node row_ids[r] for a table that is not stored in node-id order."""
    n = out.shape[0] if last is None else last
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    for r0 in range(first, n, chunk_rows):
        r1 = min(n, r0 + chunk_rows)
        ids = torch.arange(r0, r1, device=dev) if row_ids is None else row_ids[r0:r1].to(dev)
        out[r0:r1].copy_(feature_rows(ids, out.shape[1], seed, out.dtype), non_blocking=False)
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
