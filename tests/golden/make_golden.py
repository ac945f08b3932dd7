"""Writes tests/golden/hotpath_small.npz: frozen inputs and outputs of the CPU checker.

The reference cannot run here (CUDA-only, un-vendored dependency) and ships no stored answers for
this path, so these vectors freeze the checker's own answers: they catch a silent change of the
checker, and the GPU tests compare the CUDA path with the same numbers.  The Philox vectors are
the published Random123 known-answer vectors for philox4x32-10.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(HERE)), "oracle"))
import oracle as O  # noqa: E402


def small_csr(rng, n, avg_deg):
    """Skewed random multigraph -> symmetrised simple CSR (numpy only, so the fixture is self-contained)."""
    m = n * avg_deg // 2
    w = 1.0 / np.arange(1, n + 1) ** 0.8
    w /= w.sum()
    u = rng.choice(n, m, p=w)
    v = rng.choice(n, m, p=w)
    keep = u != v
    u, v = u[keep], v[keep]
    key = np.unique(np.concatenate([u * n + v, v * n + u]).astype(np.int64))
    src, dst = key // n, (key % n).astype(np.int32)
    indptr = np.zeros(n + 1, np.int64)
    np.cumsum(np.bincount(src, minlength=n), out=indptr[1:])
    return indptr, dst


def main():
    rng = np.random.default_rng(20240607)
    out = {}
    out["philox_ctr"] = np.array([[0, 0, 0, 0], [0xffffffff] * 4,
                                  [0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344]], dtype=np.uint32)
    out["philox_key"] = np.array([[0, 0], [0xffffffff] * 2, [0xa4093822, 0x299f31d0]], dtype=np.uint32)
    out["philox_out"] = np.array([[0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8],
                                  [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd],
                                  [0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1]], dtype=np.uint32)
    n = 600
    indptr, indices = small_csr(rng, n, 40)
    out["indptr"], out["indices"] = indptr, indices
    train = rng.permutation(n)[:90].astype(np.int32)
    labels = rng.integers(0, 47, 90).astype(np.int32)
    out["train"], out["labels"] = train, labels
    cases = [(32, [25, 10], 0, 3, 0xABCDEF12345, 64), (32, [25, 10], 2, 9, 0xABCDEF12345, 64),
             (40, [5, 4, 3], 1, 77, 42, 64), (16, [32], 0, 5, 7, 1)]
    out["case_params"] = np.array([[b, len(f), it, gb, seed, mr] + f + [0] * (3 - len(f))
                                   for b, f, it, gb, seed, mr in cases], dtype=np.int64)
    for i, (b, f, it, gb, seed, mr) in enumerate(cases):
        r = O.run_batch(indptr, indices, train, labels, b, it, f, gb, seed, max_rounds=mr)
        for k in ("ids", "labels", "agg_src", "agg_dst", "src_global", "node_counter", "edge_counter"):
            out["case%d_%s" % (i, k)] = r[k]
    order = O.degree_order(indptr)
    out["degree_order"] = order
    out["lut_cap100_kg1"] = O.static_cache_lut(order, 100, 1)
    out["lut_cap40_kg4"] = O.static_cache_lut(order, 40, 4)
    table = rng.standard_normal((n, 20)).astype(np.float32)
    out["table"] = table
    out["quant_int8"] = O.quant_rows(table[:16], 1)
    out["quant_e4m3"] = O.quant_rows(table[:16], 2)
    out["dequant_int8"] = O.dequant_rows(out["quant_int8"], 20, 1)
    out["dequant_e4m3"] = O.dequant_rows(out["quant_e4m3"], 20, 2)
    lru = O.LruCache(16, 4)
    seq, cis, slots = [], [], []
    for clock in range(1, 9):
        ids = rng.permutation(200)[:48].astype(np.int32)
        ci = lru.lookup(ids, clock)
        _, slot = lru.insert(ids, ci, clock)
        seq.append(ids); cis.append(ci); slots.append(slot)
    out["lru_ids"], out["lru_cache_index"], out["lru_inserted_slot"] = np.array(seq), np.array(cis), np.array(slots)
    out["lru_final_keys"], out["lru_final_stamps"] = lru.keys.copy(), lru.stamps.copy()
    np.savez_compressed(os.path.join(HERE, "hotpath_small.npz"), **out)
    print("wrote", os.path.join(HERE, "hotpath_small.npz"))


if __name__ == "__main__":
    main()
