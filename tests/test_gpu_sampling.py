"""Sampling, dedup / relabel and counter parity of the CUDA path against the CPU checker.

Bit-exact: node ids, labels, local edge lists and both counter arrays must equal the host
replay for the same seeds, RNG seed and batch number.
"""
import numpy as np
import pytest

import legion_ibp_b200 as L
from conftest import small_graph

pytestmark = pytest.mark.gpu


def _setup(indptr, indices, train_ids, labels, batch, fanout, row_bytes=16, pipes=2):
    import torch
    dev = 0
    d_indptr = torch.from_numpy(indptr).cuda()
    d_indices = torch.from_numpy(indices).cuda()
    g = L.GraphStorage(dev, d_indptr, d_indices)
    f = L.FeatureStorage(dev, len(indptr) - 1, row_bytes, None)
    d_ids = torch.from_numpy(train_ids).cuda()
    d_lab = torch.from_numpy(labels).cuda()
    f.set_split(L.TRAINMODE, d_ids, d_lab)
    pool = L.MemoryPool(dev, batch, fanout, row_bytes, pipes)
    return g, f, pool


def _run_ops(g, f, pool, batch, it, fanout, global_batch, pipe=0, cache=None):
    pool.set_batch(it, L.TRAINMODE, pipe, global_batch)
    L.BatchGenerate(None, f, cache, pool, batch, it, 0, 0, L.TRAINMODE, False, len(fanout))
    L.FeatureCacheLookup(None, cache, pool, 1, 0)
    L.IOSubmit(None, f, pool, 2, 0)
    for h, k in enumerate(fanout):
        L.RandomSample(None, g, cache, pool, k, 0, 3 * (h + 1))
        L.FeatureCacheLookup(None, cache, pool, 3 * (h + 1) + 1, 0)
        L.IOSubmit(None, f, pool, 3 * (h + 1) + 2, 0)
    L.IOComplete(None, cache, pool, 0, L.TRAINMODE)


def _fetch(pool, pipe=0):
    nc = pool.read(L.BUF_NODE_COUNTER, pipe, 16, np.int32)
    ec = pool.read(L.BUF_EDGE_COUNTER, pipe, 16, np.int32)
    hops = int(nc[8])
    n_nodes = int(nc[9 + hops])
    n_edges = int(ec[0] + ec[1])
    return dict(node_counter=nc, edge_counter=ec,
                ids=pool.read(L.BUF_IDS, pipe, n_nodes, np.int32),
                labels=pool.read(L.BUF_LABELS, pipe, int(nc[9]), np.int32),
                agg_src=pool.read(L.BUF_AGG_SRC, pipe, n_edges, np.int32),
                agg_dst=pool.read(L.BUF_AGG_DST, pipe, n_edges, np.int32),
                src_global=pool.read(L.BUF_SRC_GLOBAL, pipe, n_edges, np.int32))


def _compare(got, ref):
    np.testing.assert_array_equal(got["node_counter"], ref["node_counter"])
    np.testing.assert_array_equal(got["edge_counter"], ref["edge_counter"])
    for k in ("ids", "labels", "src_global", "agg_dst", "agg_src"):
        np.testing.assert_array_equal(got[k], ref[k], err_msg=k)


CASES = [
    # n_nodes, n_pairs, batch, fanout, seed
    (3000, 40000, 64, [25, 10], 1),
    (3000, 40000, 200, [5, 5, 5], 2),
    (500, 20000, 50, [32, 32], 3),      # dense: most nodes above the fanout, heavy dedup
    (20000, 30000, 300, [25, 10], 4),   # sparse: many isolated and low-degree nodes
    (3000, 60000, 1, [25, 10], 5),      # single seed
    (3000, 40000, 100, [1], 6),
    (3000, 40000, 128, [15, 10, 5], 7),
]


@pytest.mark.parametrize("n_nodes,n_pairs,batch,fanout,seed", CASES)
def test_batch_matches_host_replay(oracle_mod, n_nodes, n_pairs, batch, fanout, seed):
    indptr, indices = small_graph(n_nodes, n_pairs, seed)
    rng = np.random.default_rng(seed)
    train = rng.permutation(n_nodes)[: max(batch * 3 + 7, 10)].astype(np.int32)
    labels = rng.integers(0, 47, len(train)).astype(np.int32)
    g, f, pool = _setup(indptr, indices, train, labels, batch, fanout)
    pool.set_rng(0x1234ABCD5678EF00 + seed, 64)
    n_batches = (len(train) - 1) // batch + 1
    for it in range(n_batches):  # includes the shortened tail batch
        _run_ops(g, f, pool, batch, it, fanout, global_batch=100 + it, pipe=it % 2)
        got = _fetch(pool, it % 2)
        ref = oracle_mod.run_batch(indptr, indices, train, labels, batch, it, fanout, 100 + it,
                                   0x1234ABCD5678EF00 + seed)
        _compare(got, ref)
        assert pool.device_error() == 0
    pool.close(); f.close(); g.close()


@pytest.mark.parametrize("shift", [20, 6, 0])
def test_id_map_front_and_back_regions(oracle_mod, shift):
    """The id map tries a small front region first and falls back to the worst-case-sized back region.
    With a front of 64 slots nearly every node lands in the back region, which must then be cleared
    before the next batch on the same pipe; with shift 0 the front alone is as large as the worst case."""
    n_nodes, n_pairs, batch, fanout, seed = 3000, 40000, 128, [15, 10, 5], 7
    indptr, indices = small_graph(n_nodes, n_pairs, seed)
    rng = np.random.default_rng(seed)
    train = rng.permutation(n_nodes)[: batch * 6].astype(np.int32)
    labels = rng.integers(0, 47, len(train)).astype(np.int32)
    L._check(L.lib().legion_set_tunable(b"map_front_shift", shift))
    try:
        g, f, pool = _setup(indptr, indices, train, labels, batch, fanout)
    finally:
        L._check(L.lib().legion_set_tunable(b"map_front_shift", -1))
    pool.set_rng(77, 64)
    for it in range(6):
        pipe = 0 if it < 4 else 1          # four batches in a row on one pipe, then the other
        _run_ops(g, f, pool, batch, it, fanout, global_batch=it, pipe=pipe)
        _compare(_fetch(pool, pipe), oracle_mod.run_batch(indptr, indices, train, labels, batch, it, fanout, it, 77))
        assert pool.device_error() == 0
    pool.close(); f.close(); g.close()


@pytest.mark.parametrize("max_rounds", [1, 2, 3])
def test_fallback_after_few_rounds(oracle_mod, max_rounds):
    """With the rejection rounds cut short the lane-ordered fallback settles the draws."""
    indptr, indices = small_graph(400, 12000, 11)
    rng = np.random.default_rng(0)
    train = rng.permutation(400)[:150].astype(np.int32)
    labels = np.zeros(len(train), np.int32)
    fanout = [25, 10]
    g, f, pool = _setup(indptr, indices, train, labels, 50, fanout)
    pool.set_rng(77, max_rounds)
    for it in range(3):
        _run_ops(g, f, pool, 50, it, fanout, global_batch=it)
        ref = oracle_mod.run_batch(indptr, indices, train, labels, 50, it, fanout, it, 77, max_rounds=max_rounds)
        _compare(_fetch(pool), ref)
    pool.close(); f.close(); g.close()


def test_structure_properties_large_batch(oracle_mod):
    """Size-independent properties on a batch too large to eyeball: every edge is a real CSR edge,
    no neighbour is drawn twice for one node, dst nodes are a prefix of src nodes, ids are unique."""
    n = 200000
    indptr, indices = small_graph(n, 3000000, 21)
    rng = np.random.default_rng(1)
    train = rng.permutation(n)[:8000].astype(np.int32)
    labels = rng.integers(0, 172, len(train)).astype(np.int32)
    fanout = [25, 10]
    g, f, pool = _setup(indptr, indices, train, labels, 8000, fanout)
    pool.set_rng(5, 64)
    _run_ops(g, f, pool, 8000, 0, fanout, global_batch=9)
    got = _fetch(pool)
    nc, ec = got["node_counter"], got["edge_counter"]
    ids = got["ids"]
    assert len(np.unique(ids)) == len(ids)
    np.testing.assert_array_equal(ids[:8000], train[:8000])
    assert nc[8] == 2 and nc[9] == 8000 and nc[11] == len(ids)
    e1, e2 = int(ec[10]), int(ec[11])
    assert ec[13] == 0 and ec[14] == e1
    src, dst = got["agg_src"], got["agg_dst"]
    # hop 1 samples for the seeds only, hop 2 for every node known after hop 1
    assert dst[:e1].max() < nc[9] and dst[e1:e1 + e2].max() < nc[10]
    assert src[:e1].max() < nc[10] and src.max() < nc[11]
    np.testing.assert_array_equal(ids[src], got["src_global"])
    # membership and no duplicate per (hop, dst)
    for lo, hi, k in ((0, e1, 25), (e1, e1 + e2, 10)):
        d = ids[dst[lo:hi]].astype(np.int64)
        s = got["src_global"][lo:hi].astype(np.int64)
        key = d * n + s
        # a multigraph-free CSR: (d, s) pairs of one hop must be unique
        assert len(np.unique(key)) == len(key)
        full = np.repeat(np.arange(n, dtype=np.int64), np.diff(indptr)) * n + indices
        assert np.isin(key, full).all()
        cnt = np.bincount(dst[lo:hi])
        deg = np.diff(indptr)[ids[:len(cnt)]]
        np.testing.assert_array_equal(cnt, np.minimum(deg, k))
    ref = oracle_mod.run_batch(indptr, indices, train, labels, 8000, 0, fanout, 9, 5)
    _compare(got, ref)
    pool.close(); f.close(); g.close()


def test_uniformity_chi_square(oracle_mod):
    """Each neighbour of a node of degree d is kept with probability k/d: chi-square over many batches."""
    n = 64
    train = np.arange(n, dtype=np.int32)
    labels = np.zeros(n, np.int32)
    for kk, dd in ((10, 40), (25, 30)):   # direct draw, and the leave-out branch
        indptr = np.arange(n + 1, dtype=np.int64) * dd
        indices = np.tile(np.arange(dd, dtype=np.int32), n)
        g, f, pool = _setup(indptr, indices, train, labels, n, [kk])
        pool.set_rng(2024, 64)
        counts = np.zeros(dd, np.int64)
        reps = 200
        for b in range(reps):
            _run_ops(g, f, pool, n, 0, [kk], global_batch=b)
            got = _fetch(pool)
            assert len(got["src_global"]) == n * kk
            counts += np.bincount(got["src_global"], minlength=dd)[:dd]
        expected = reps * n * kk / dd
        chi2 = float(((counts - expected) ** 2 / expected).sum())
        # dd-1 degrees of freedom; 99.99% quantile of chi2(39) ~ 78, chi2(29) ~ 64
        assert chi2 < 90, (kk, dd, chi2)
        pool.close(); f.close(); g.close()


def test_rejects_bad_arguments():
    import torch
    indptr, indices = small_graph(300, 2000, 1)
    train = np.arange(50, dtype=np.int32)
    g, f, pool = _setup(indptr, indices, train, train.copy(), 10, [5])
    with pytest.raises(L.LegionError):
        L.RandomSample(None, g, None, pool, 33, 0, 3)          # fanout above 32
    with pytest.raises(L.LegionError):
        L.RandomSample(None, g, None, pool, 5, 0, 4)           # not a sampling op id
    with pytest.raises(L.LegionError):
        L.BatchGenerate(None, f, None, pool, 11, 0, 0, 0, L.TRAINMODE, False, 1)  # above the pool's batch
    with pytest.raises(L.LegionError):
        L.MemoryPool(0, 10, [40], 16)
    pool.close(); f.close(); g.close()


def test_isolated_nodes_hubs_and_empty_topology(oracle_mod):
    """Edge cases of the topology: a graph without edges (every hop is empty), a star (one hub whose
    degree is far above the fanout, leaves of degree 1) plus isolated seeds, and ids at both ends of
    the id range."""
    # no edges at all
    n = 100
    indptr = np.zeros(n + 1, np.int64)
    indices = np.zeros(1, np.int32)
    train = np.arange(n, dtype=np.int32)[::-1].copy()
    labels = np.arange(n, dtype=np.int32)
    g, f, pool = _setup(indptr, indices, train, labels, 40, [25, 10])
    pool.set_rng(1, 64)
    for it in range(3):
        _run_ops(g, f, pool, 40, it, [25, 10], global_batch=it, pipe=it % 2)
        got = _fetch(pool, it % 2)
        ref = oracle_mod.run_batch(indptr, indices, train, labels, 40, it, [25, 10], it, 1)
        _compare(got, ref)
        assert got["edge_counter"][10] == 0 and got["edge_counter"][11] == 0 and len(got["ids"]) == min(40, 100 - 40 * it)
    pool.close(); f.close(); g.close()
    # star: node 0 is the hub of 5000 leaves; nodes 5001..5999 are isolated
    n = 6000
    deg = np.zeros(n, np.int64)
    deg[0] = 5000
    deg[1:5001] = 1
    indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    indices = np.concatenate([np.arange(1, 5001), np.zeros(5000)]).astype(np.int32)
    train = np.array([0, 5999, 1, 5000, 5500, 2500, 5001], np.int32)
    labels = np.arange(len(train), dtype=np.int32)
    for fanout in ([25, 10], [32, 32, 32], [1, 1]):
        g, f, pool = _setup(indptr, indices, train, labels, 7, fanout)
        pool.set_rng(9, 64)
        for gb in range(3):
            _run_ops(g, f, pool, 7, 0, fanout, global_batch=gb)
            got = _fetch(pool)
            ref = oracle_mod.run_batch(indptr, indices, train, labels, 7, 0, fanout, gb, 9)
            _compare(got, ref)
            e1 = int(got["edge_counter"][10])
            assert e1 == min(fanout[0], 5000) + 3        # the hub's picks + one edge for each of the three leaves
            assert pool.device_error() == 0
        pool.close(); f.close(); g.close()
