"""The CPU checker against published vectors, independent restatements and its frozen fixtures."""
import ctypes as C
import os

import numpy as np
import pytest

from conftest import ROOT, small_graph

GOLD = os.path.join(ROOT, "tests", "golden", "hotpath_small.npz")


# ---- an independent pure-Python restatement of the sampler (small cases only) -----------------------

M32 = 0xFFFFFFFF


def py_philox(ctr, key):
    c0, c1, c2, c3 = [int(x) for x in ctr]
    k0, k1 = [int(x) for x in key]
    for _ in range(10):
        p0 = 0xD2511F53 * c0
        p1 = 0xCD9E8D57 * c2
        c0, c1, c2, c3 = ((p1 >> 32) ^ c1 ^ k0) & M32, p1 & M32, ((p0 >> 32) ^ c3 ^ k1) & M32, p0 & M32
        k0 = (k0 + 0x9E3779B9) & M32
        k1 = (k1 + 0xBB67AE85) & M32
    return [c0, c1, c2, c3]


def py_draw(i, lane, rnd, hop, batch, seed, n):
    w = py_philox([i, rnd * 32 + lane, hop, batch], [seed & M32, seed >> 32])
    return (((w[1] << 32) | w[0]) * n) >> 64


def py_distinct(m, n, i, hop, batch, seed, max_rounds):
    x, kept = [None] * m, [False] * m
    for r in range(max(1, max_rounds)):
        if all(kept):
            break
        pre = list(kept)
        for l in range(m):
            if not pre[l]:
                x[l] = py_draw(i, l, r, hop, batch, seed, n)
        for l in range(m):
            if pre[l]:
                continue
            if not any(j != l and x[j] == x[l] and (pre[j] or j < l) for j in range(m)):
                kept[l] = True
    for l in range(m):
        if not kept[l]:
            cand = x[l]
            while any(kept[j] and x[j] == cand for j in range(m)):
                cand = (cand + 1) % n
            x[l], kept[l] = cand, True
    return x


def py_sample_hop(indptr, indices, ids, k, hop, batch, seed, max_rounds=64):
    src, dst = [], []
    for i, v in enumerate(ids):
        if v < 0:
            continue
        s, deg = int(indptr[v]), int(indptr[v + 1] - indptr[v])
        if deg <= k:
            pos = list(range(deg))
        elif deg >= 2 * k:
            pos = py_distinct(k, deg, i, hop, batch, seed, max_rounds)
        else:
            out = set(py_distinct(deg - k, deg, i, hop, batch, seed, max_rounds))
            pos = [p for p in range(deg) if p not in out]
        src += [int(indices[s + p]) for p in pos]
        dst += [i] * len(pos)
    return np.array(src, np.int32), np.array(dst, np.int32)


def py_run_batch(indptr, indices, train, labels, batch, it, fanout, gb, seed, max_rounds=64):
    first = batch * it
    size = min(batch, len(train) - first)
    ids = [int(v) for v in train[first:first + size]]
    pos = {v: i for i, v in enumerate(ids)}
    agg_src, agg_dst, counts, ecounts = [], [], [len(ids)], []
    for h, k in enumerate(fanout):
        s, d = py_sample_hop(indptr, indices, ids, k, h, gb, seed, max_rounds)
        for u in s:
            if int(u) not in pos:
                pos[int(u)] = len(ids)
                ids.append(int(u))
        agg_src += [pos[int(u)] for u in s]
        agg_dst += list(d)
        counts.append(len(ids))
        ecounts.append(len(s))
    return np.array(ids, np.int32), np.array(agg_src, np.int32), np.array(agg_dst, np.int32), counts, ecounts


# ---- tests ----------------------------------------------------------------------------------------------

def test_philox_known_answers(oracle_mod):
    g = np.load(GOLD)
    for c, k, o in zip(g["philox_ctr"], g["philox_key"], g["philox_out"]):
        np.testing.assert_array_equal(oracle_mod.philox4x32_10(c, k), o)
        assert py_philox(c, k) == [int(v) for v in o]


def test_philox_agrees_with_curand_host_generator(oracle_mod):
    """cuRAND's host Philox4_32_10 generator: its first four outputs for seed s are
    philox4x32-10(counter = 0, key = (s_lo, s_hi))."""
    try:
        cr = C.CDLL("/usr/local/cuda/lib64/libcurand.so")
    except OSError:
        pytest.skip("libcurand not present")
    gen = C.c_void_p()
    if cr.curandCreateGeneratorHost(C.byref(gen), 161) != 0:
        pytest.skip("cuRAND host generator unavailable")
    for seed in (0, 1, 0x299f31d0a4093822, 0xDEADBEEF12345678):
        assert cr.curandSetPseudoRandomGeneratorSeed(gen, C.c_ulonglong(seed)) == 0
        assert cr.curandSetGeneratorOffset(gen, C.c_ulonglong(0)) == 0
        out = (C.c_uint32 * 4)()
        assert cr.curandGenerate(gen, out, C.c_size_t(4)) == 0
        np.testing.assert_array_equal(np.array(list(out), np.uint32),
                                      oracle_mod.philox4x32_10([0, 0, 0, 0], [seed & M32, seed >> 32]))
    cr.curandDestroyGenerator(gen)


@pytest.mark.parametrize("max_rounds", [64, 2, 1])
def test_sampler_matches_python_restatement(oracle_mod, max_rounds):
    indptr, indices = small_graph(300, 6000, 4)
    rng = np.random.default_rng(0)
    ids = rng.permutation(300)[:40].astype(np.int32)
    ids[7] = -1  # invalid seeds produce nothing
    for k, hop in ((25, 0), (10, 1), (32, 2), (1, 0)):
        s, d = oracle_mod.sample_hop(indptr, indices, ids, k, hop, 17, 0x1122334455667788, max_rounds)
        ps, pd = py_sample_hop(indptr, indices, ids, k, hop, 17, 0x1122334455667788, max_rounds)
        np.testing.assert_array_equal(s, ps)
        np.testing.assert_array_equal(d, pd)


def test_run_batch_matches_python_restatement_and_counter_trace(oracle_mod):
    indptr, indices = small_graph(400, 7000, 8)
    rng = np.random.default_rng(1)
    train = rng.permutation(400)[:70].astype(np.int32)
    labels = rng.integers(0, 9, 70).astype(np.int32)
    for fanout in ([25, 10], [4, 3, 2], [6]):
        for it in range(3):  # 32 + 32 + 6 (shortened tail)
            r = oracle_mod.run_batch(indptr, indices, train, labels, 32, it, fanout, 5 + it, 99)
            ids, src, dst, counts, ecounts = py_run_batch(indptr, indices, train, labels, 32, it, fanout, 5 + it, 99)
            np.testing.assert_array_equal(r["ids"], ids)
            np.testing.assert_array_equal(r["agg_src"], src)
            np.testing.assert_array_equal(r["agg_dst"], dst)
            nc, ec = r["node_counter"], r["edge_counter"]
            hops = len(fanout)
            # what the trainer reads (ipc_cuda_kernel.cu:194-240, ipc_service.cpp:61-79)
            assert nc[8] == hops
            assert list(nc[9:9 + hops + 1]) == counts
            assert list(ec[10:10 + hops]) == ecounts
            assert list(ec[13:13 + hops]) == list(np.cumsum([0] + ecounts[:-1]))
            # end-of-batch state of the bookkeeping kernel
            assert nc[0] == counts[-2] and nc[1] == counts[-1] - counts[-2] and nc[7] == counts[-1]
            assert nc[2] == nc[0] and nc[3] == nc[1] and nc[4] == 0 and nc[5] == 0 and nc[6] == 0
            assert ec[0] == sum(ecounts[:-1]) and ec[1] == ecounts[-1] and ec[2] == 0
            np.testing.assert_array_equal(r["labels"], labels[32 * it: 32 * it + counts[0]])


def test_structure_invariants(oracle_mod):
    indptr, indices = small_graph(5000, 60000, 2)
    n = 5000
    deg = np.diff(indptr)
    full = np.repeat(np.arange(n, dtype=np.int64), deg) * n + indices
    rng = np.random.default_rng(3)
    train = rng.permutation(n)[:900].astype(np.int32)
    r = oracle_mod.run_batch(indptr, indices, train, train, 300, 1, [25, 10], 1, 1)
    ids, nc, ec = r["ids"], r["node_counter"], r["edge_counter"]
    assert len(np.unique(ids)) == len(ids)
    lo = 0
    for h, k in enumerate([25, 10]):
        e = int(ec[10 + h])
        d, s = r["agg_dst"][lo:lo + e], r["src_global"][lo:lo + e]
        np.testing.assert_array_equal(np.bincount(d, minlength=nc[9 + h]), np.minimum(deg[ids[:nc[9 + h]]], k))
        key = ids[d].astype(np.int64) * n + s
        assert len(np.unique(key)) == len(key) and np.isin(key, full).all()
        assert (np.diff(d) >= 0).all()  # edges are laid out input after input
        lo += e
    np.testing.assert_array_equal(ids[r["agg_src"]], r["src_global"])
    # new nodes appear in order of first appearance in the edge list
    seen_at = {}
    for e, u in enumerate(r["src_global"]):
        seen_at.setdefault(int(u), e)
    new = ids[nc[9]:]
    firsts = [seen_at[int(u)] for u in new]
    assert firsts == sorted(firsts)


def test_uniform_marginals_chi_square(oracle_mod):
    n = 64
    for kk, dd in ((10, 40), (25, 30), (5, 200)):
        indptr = np.arange(n + 1, dtype=np.int64) * dd
        indices = (np.tile(np.arange(dd, dtype=np.int32), n))
        counts = np.zeros(dd)
        reps = 100
        for b in range(reps):
            s, _ = oracle_mod.sample_hop(indptr, indices, np.arange(n, dtype=np.int32), kk, 0, b, 2024)
            assert len(s) == n * kk
            counts += np.bincount(s, minlength=dd)
        exp = reps * n * kk / dd
        chi2 = float(((counts - exp) ** 2 / exp).sum())
        assert chi2 < dd + 6 * np.sqrt(2 * dd), (kk, dd, chi2)


def test_pair_inclusion_is_uniform(oracle_mod):
    """Beyond the marginals: every pair of neighbours is kept together equally often (k=3 of 7)."""
    dd, kk, n = 7, 3, 32
    indptr = np.arange(n + 1, dtype=np.int64) * dd
    indices = np.tile(np.arange(dd, dtype=np.int32), n)
    pair = np.zeros((dd, dd))
    reps = 400
    for b in range(reps):
        s, d = oracle_mod.sample_hop(indptr, indices, np.arange(n, dtype=np.int32), kk, 0, b, 5)
        for row in s.reshape(n, kk):
            for a in row:
                for c in row:
                    if a < c:
                        pair[a, c] += 1
    vals = pair[np.triu_indices(dd, 1)]
    exp = reps * n * (kk * (kk - 1) / 2) / (dd * (dd - 1) / 2)
    chi2 = float(((vals - exp) ** 2 / exp).sum())
    assert chi2 < 60, chi2  # 20 degrees of freedom


def test_static_cache_against_numpy(oracle_mod):
    indptr, _ = small_graph(2000, 20000, 6)
    n = 2000
    deg = np.diff(indptr)
    order = oracle_mod.degree_order(indptr)
    np.testing.assert_array_equal(order, np.lexsort((np.arange(n), -deg)).astype(np.int32))
    rng = np.random.default_rng(0)
    table = rng.standard_normal((n, 12)).astype(np.float32)
    for cap, kg in ((300, 1), (100, 4), (700, 3), (0, 1), (2000, 2)):
        lut = oracle_mod.static_cache_lut(order, cap, kg)
        cached = min(n, cap * kg)
        exp = np.full(n, -2, np.int32)
        t = np.arange(cached)
        exp[order[:cached]] = (t % kg) * cap + t // kg
        np.testing.assert_array_equal(lut, exp)
        parts = [oracle_mod.static_cache_fill(order, cap, kg, ki, table) for ki in range(kg)]
        ids = rng.integers(0, n, 500).astype(np.int32)
        ids[3] = -1
        ci = oracle_mod.find_feat(ids, lut)
        assert ci[3] == -2
        out = oracle_mod.gather(ids, ci, cap, parts, table)
        valid = ids >= 0
        np.testing.assert_array_equal(out[valid], table[ids[valid]])
        assert (out[3] == 0).all()  # rows of invalid ids are left untouched
        for ki in range(kg):       # every cached row is a bit copy of its host row
            rows = order[ki:cached:kg]
            np.testing.assert_array_equal(parts[ki][:len(rows)], table[rows])


def test_quantised_rows(oracle_mod):
    import torch
    rng = np.random.default_rng(0)
    x = rng.standard_normal((64, 100)).astype(np.float32)
    x[0] = 0
    x[1, :3] = [1e-30, -300.0, 300.0]
    for codec in (1, 2):
        q = oracle_mod.quant_rows(x, codec)
        assert q.shape == (64, 112)
        d = oracle_mod.dequant_rows(q, 100, codec)
        absmax = np.abs(x).max(axis=1, keepdims=True)
        if codec == 1:
            tol = absmax / 254 + absmax * 2.0 ** -22
            codes = q[:, :100].view(np.int8)
            exp = np.clip(np.rint((x * np.where(absmax > 0, np.float32(127) / np.where(absmax > 0, absmax, 1), 0)
                                   .astype(np.float32)).astype(np.float32)), -127, 127)
            np.testing.assert_array_equal(codes, exp.astype(np.int8))
        else:
            tol = np.maximum(np.abs(x) * 2.0 ** -4, absmax / 448 * 2.0 ** -10) * (1 + 1e-5)
            inv = np.where(absmax > 0, np.float32(448) / np.where(absmax > 0, absmax, 1), 0).astype(np.float32)
            ref = torch.from_numpy((x * inv).astype(np.float32)).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
            np.testing.assert_array_equal(q[:, :100], ref)
        assert (np.abs(d - x) <= tol + 1e-30).all()
        assert (d[0] == 0).all()
    # every e4m3 code decodes like torch's
    mine = np.array([oracle_mod.e4m3_to_float(b) for b in range(256)], np.float32)
    ref = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).to(torch.float32).numpy()
    assert ((mine == ref) | (np.isnan(mine) & np.isnan(ref))).all()
    assert oracle_mod.float_to_e4m3(1e9) == 0x7E and oracle_mod.float_to_e4m3(-500.0) == 0xFE
    assert oracle_mod.float_to_e4m3(2.0 ** -10) == 0 and oracle_mod.float_to_e4m3(2.0 ** -10 * 1.01) == 1


def test_lru_against_python_model(oracle_mod):
    """Dictionary model of the replacement rule: victim = smallest stamp (empty = -1), ways touched in
    this batch are kept, first claimant in id order wins, one insertion per way and batch."""
    rng = np.random.default_rng(5)
    sets, ways = 13, 4
    c = oracle_mod.LruCache(sets, ways)
    keys = [[-1] * ways for _ in range(sets)]
    stamps = [[0] * ways for _ in range(sets)]
    for clock in range(1, 40):
        ids = rng.permutation(150)[:40].astype(np.int32)
        ci = c.lookup(ids, clock)
        exp_ci = []
        for v in ids:
            s = int(v) % sets
            if int(v) in keys[s]:
                w = keys[s].index(int(v))
                stamps[s][w] = clock
                exp_ci.append(s * ways + w)
            else:
                exp_ci.append(-1)
        np.testing.assert_array_equal(ci, exp_ci)
        n_ins, slot = c.insert(ids, ci, clock)
        claimed, picks = {}, []
        for r, v in enumerate(ids):
            if exp_ci[r] >= 0:
                picks.append(None)
                continue
            s = int(v) % sets
            cand = [(-1 if keys[s][w] == -1 else stamps[s][w], w) for w in range(ways)]
            cand = [t for t in cand if t[0] != clock]
            if not cand:
                picks.append(None)
                continue
            w = min(cand)[1]
            picks.append((s, w))
            claimed.setdefault((s, w), r)
        exp_slot = np.full(len(ids), -1, np.int64)
        for r, pk in enumerate(picks):
            if pk is not None and claimed[pk] == r:
                keys[pk[0]][pk[1]] = int(ids[r])
                stamps[pk[0]][pk[1]] = clock
                exp_slot[r] = pk[0] * ways + pk[1]
        np.testing.assert_array_equal(slot, exp_slot)
        assert n_ins == int((exp_slot >= 0).sum())
        np.testing.assert_array_equal(c.keys, np.array(keys).reshape(-1))
        np.testing.assert_array_equal(c.stamps, np.array(stamps).reshape(-1))


def test_step_arithmetic(oracle_mod):
    steps, vbs, tbs = oracle_mod.coordinate([24491, 24490], [4900, 4899], [276630, 276629], 8000)
    assert list(steps) == [(24490 - 1) // 8000, (4900 - 1) // 512 + 1, (276630 - 1) // 512 + 1]
    assert list(vbs) == [(4900 - 1) // steps[1] + 1, (4899 - 1) // steps[1] + 1]
    tr, va, te, ep = 3, 2, 4, 2
    seq = [oracle_mod.mode_of_batch(b, tr, va, te, ep) for b in range((tr + va) * ep + te)]
    assert seq == [(0, 0), (0, 1), (0, 2), (1, 0), (1, 1)] * 2 + [(2, 0), (2, 1), (2, 2), (2, 3)]


def test_counter_update_literal(oracle_mod):
    nc, ec = np.zeros(16, np.int32), np.zeros(16, np.int32)
    oracle_mod.counter_update(nc, ec, 0, 800, 2)
    assert nc[0] == 0 and nc[1] == 800 and nc[8] == 2 and nc[9] == 800
    oracle_mod.counter_update(nc, ec, 1)
    assert nc[2] == 0 and nc[3] == 800
    nc[6], ec[2] = 5000, 20000          # what one sampling hop accumulates
    oracle_mod.counter_update(nc, ec, 3)
    assert list(nc[[0, 1, 6, 7, 10]]) == [800, 5000, 0, 5800, 5800]
    assert list(ec[[0, 1, 2, 10, 13]]) == [0, 20000, 0, 20000, 0]
    nc[6], ec[2] = 70000, 58000
    oracle_mod.counter_update(nc, ec, 6)
    assert list(nc[[0, 1, 7, 11]]) == [5800, 70000, 75800, 75800]
    assert list(ec[[0, 1, 11, 14]]) == [20000, 58000, 58000, 20000]


def test_frozen_fixture(oracle_mod):
    g = np.load(GOLD)
    indptr, indices, train, labels = g["indptr"], g["indices"], g["train"], g["labels"]
    for i, row in enumerate(g["case_params"]):
        b, hops, it, gb, seed, mr = [int(v) for v in row[:6]]
        fanout = [int(v) for v in row[6:6 + hops]]
        r = oracle_mod.run_batch(indptr, indices, train, labels, b, it, fanout, gb, seed, max_rounds=mr)
        for k in ("ids", "labels", "agg_src", "agg_dst", "src_global", "node_counter", "edge_counter"):
            np.testing.assert_array_equal(r[k], g["case%d_%s" % (i, k)], err_msg="case %d %s" % (i, k))
    order = oracle_mod.degree_order(indptr)
    np.testing.assert_array_equal(order, g["degree_order"])
    np.testing.assert_array_equal(oracle_mod.static_cache_lut(order, 100, 1), g["lut_cap100_kg1"])
    np.testing.assert_array_equal(oracle_mod.static_cache_lut(order, 40, 4), g["lut_cap40_kg4"])
    np.testing.assert_array_equal(oracle_mod.quant_rows(g["table"][:16], 1), g["quant_int8"])
    np.testing.assert_array_equal(oracle_mod.quant_rows(g["table"][:16], 2), g["quant_e4m3"])
    np.testing.assert_array_equal(oracle_mod.dequant_rows(g["quant_int8"], 20, 1), g["dequant_int8"])
    np.testing.assert_array_equal(oracle_mod.dequant_rows(g["quant_e4m3"], 20, 2), g["dequant_e4m3"])
    lru = oracle_mod.LruCache(16, 4)
    for clock, ids in enumerate(g["lru_ids"], start=1):
        ci = lru.lookup(ids, clock)
        np.testing.assert_array_equal(ci, g["lru_cache_index"][clock - 1])
        _, slot = lru.insert(ids, ci, clock)
        np.testing.assert_array_equal(slot, g["lru_inserted_slot"][clock - 1])
    np.testing.assert_array_equal(lru.keys, g["lru_final_keys"])
    np.testing.assert_array_equal(lru.stamps, g["lru_final_stamps"])
