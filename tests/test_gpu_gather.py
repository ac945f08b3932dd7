"""Cache build, cache lookup and feature gather parity against the CPU checker.

Gathered rows and hit / miss sets are bit-exact; dequantised rows of the compressed caches are
bit-exact against the host dequantiser and within the stated tolerance of the fp32 rows.
"""
import numpy as np
import pytest

import legion_ibp_b200 as L
from conftest import small_graph

pytestmark = pytest.mark.gpu


def _pinned(arr):
    import torch
    t = torch.from_numpy(np.ascontiguousarray(arr)).pin_memory()
    return t


class Rig:
    """One GPU's storage objects around a host table, with the id list as the seed list (0 hops)."""

    def __init__(self, table, ids_list, batch, lru=None, capacity=0, kg=1, ki=0, codec=L.CODEC_RAW, order=None,
                 out_row_bytes=None, row_of=None):
        import torch
        self.table = table
        self.n = table.shape[0]
        self.row_bytes = table.strides[0]
        self.h_table = _pinned(table)
        self.ids = torch.from_numpy(ids_list.astype(np.int32)).cuda()
        self.lab = torch.zeros_like(self.ids)
        self.f = L.FeatureStorage(0, self.n, self.row_bytes, self.h_table)
        self.f.set_split(L.TRAINMODE, self.ids, self.lab)
        self.pool = L.MemoryPool(0, batch, [], out_row_bytes or self.row_bytes, 2)
        if lru is not None:
            self.cache = L.UnifiedCache(0, self.n, self.row_bytes, 0, lru=lru)
            self.cache.set_host_table(self.h_table)
        else:
            self.cache = L.UnifiedCache(0, self.n, self.row_bytes, capacity, kg, ki, codec)
            if order is not None:
                self.order = torch.from_numpy(order.astype(np.int32)).cuda()
                self.row_of = torch.from_numpy(row_of.astype(np.int32)).cuda() if row_of is not None else None
                self.cache.fill_static(self.order, self.h_table, row_of_id=self.row_of)
        self.batch = batch

    def gather(self, it, pipe=0):
        self.pool.set_batch(it, L.TRAINMODE, pipe, it)
        L.BatchGenerate(None, self.f, self.cache, self.pool, self.batch, it, 0, 0, L.TRAINMODE, False, 0)
        L.FeatureCacheLookup(None, self.cache, self.pool, 1, 0)
        L.IOComplete(None, self.cache, self.pool, 0, L.TRAINMODE)
        nc = self.pool.read(L.BUF_NODE_COUNTER, pipe, 16, np.int32)
        n = int(nc[9])
        feat = self.pool.read(L.BUF_FEATURES, pipe, n * self.pool.row_bytes_out, np.uint8)
        return n, feat.reshape(n, self.pool.row_bytes_out), nc

    def close(self):
        self.pool.close(); self.cache.close(); self.f.close()


@pytest.mark.parametrize("feat_len,dtype", [(100, np.float32), (128, np.float32), (768, np.float16),
                                            (3, np.float32), (602, np.float32), (512, np.float32), (1, np.float32)])
@pytest.mark.parametrize("cached_frac", [0.0, 0.2, 1.0])
def test_static_cache_gather(oracle_mod, feat_len, dtype, cached_frac):
    rng = np.random.default_rng(feat_len)
    indptr, _ = small_graph(4000, 50000, 3)
    n = len(indptr) - 1
    table = rng.standard_normal((n, feat_len)).astype(dtype)
    ids_list = rng.integers(0, n, 5000).astype(np.int32)
    cap = int(n * cached_frac)
    order = oracle_mod.degree_order(indptr)
    rig = Rig(table, ids_list, 1237, capacity=cap, order=order)
    lut = oracle_mod.static_cache_lut(order, cap, 1)
    part = oracle_mod.static_cache_fill(order, cap, 1, 0, table)
    got_lut = np.empty(n, np.int32)
    L._check(L.lib().legion_copy(got_lut.ctypes.data_as(L.C.c_void_p), L.C.c_void_p(rig.cache.lut_ptr()),
                                 L.C.c_int64(n * 4), L.C.c_int32(2)))
    np.testing.assert_array_equal(got_lut, lut)
    if cap:
        p, b = rig.cache.partition()
        got_part = np.empty(b, np.uint8)
        L._check(L.lib().legion_copy(got_part.ctypes.data_as(L.C.c_void_p), L.C.c_void_p(p), L.C.c_int64(b),
                                     L.C.c_int32(2)))
        np.testing.assert_array_equal(got_part, part.view(np.uint8).reshape(-1))
    for it in range(5):  # 4 full batches and the tail
        cnt, feat, nc = rig.gather(it)
        ids = ids_list[it * 1237: it * 1237 + cnt]
        assert cnt == len(ids)
        ci = oracle_mod.find_feat(ids, lut)
        ref = oracle_mod.gather(ids, ci, cap, [part], table)
        np.testing.assert_array_equal(feat, ref.view(np.uint8).reshape(cnt, -1))
        got_ci = rig.pool.read(L.BUF_CACHE_INDEX, 0, cnt, np.int32)
        np.testing.assert_array_equal(got_ci, ci)
        assert nc[2] == 0 and nc[3] == cnt
    st = rig.cache.stats()
    assert st["local_hits"] + st["misses"] == 5000 and st["peer_hits"] == 0
    rig.close()


@pytest.mark.parametrize("feat_len,codec", [(128, L.CODEC_RAW), (100, L.CODEC_RAW), (128, L.CODEC_INT8)])
def test_host_table_in_another_row_order(oracle_mod, feat_len, codec):
    """A host table whose rows are permuted (row_of[id] = row holding node id): cache fill, hit / miss
    index and gathered rows are those of the id-ordered table."""
    rng = np.random.default_rng(feat_len)
    indptr, _ = small_graph(5000, 60000, 4)
    n = len(indptr) - 1
    table = rng.standard_normal((n, feat_len)).astype(np.float32)
    perm = rng.permutation(n)                    # row r of the stored table holds node perm[r]
    stored = np.ascontiguousarray(table[perm])
    row_of = np.empty(n, np.int64)
    row_of[perm] = np.arange(n)
    ids_list = rng.integers(0, n, 7000).astype(np.int32)
    ids_list[11] = -1
    cap = n // 5
    order = oracle_mod.degree_order(indptr)
    rig = Rig(stored, ids_list, 7000, capacity=cap, order=order, codec=codec, row_of=row_of)
    lut = oracle_mod.static_cache_lut(order, cap, 1)
    ci = oracle_mod.find_feat(ids_list, lut)
    cnt, feat, _ = rig.gather(0)
    got = feat.view(np.float32).reshape(cnt, feat_len)
    np.testing.assert_array_equal(rig.pool.read(L.BUF_CACHE_INDEX, 0, cnt, np.int32), ci)   # misses still read -2
    if codec == L.CODEC_RAW:
        part = oracle_mod.static_cache_fill(order, cap, 1, 0, table)
        ref = oracle_mod.gather(ids_list, ci, cap, [part], table)
    else:
        part = oracle_mod.quant_rows(table[order[:cap]], codec)
        ref = oracle_mod.gather_quant(ids_list, ci, cap, [part], table, codec)
    valid = ids_list >= 0
    np.testing.assert_array_equal(got[valid].view(np.uint32), ref[valid].view(np.uint32))
    # the allocation-free entry point reads the same table
    import torch
    if codec == L.CODEC_RAW:
        out = torch.zeros((cnt, feat_len), dtype=torch.float32, device="cuda")
        L.gather_rows_noalloc(None, 0, rig.ids, rig.cache.lut_ptr(), cap, 1, 0, [rig.cache.partition()[0]], rig.h_table, n,
                              feat_len * 4, out)
        torch.cuda.synchronize()
        np.testing.assert_array_equal(out.cpu().numpy()[valid], table[ids_list[valid]])
    rig.close()


def test_degree_order_matches(oracle_mod):
    import torch
    for seed, n, pairs in ((0, 5000, 60000), (1, 70000, 200000)):
        indptr, _ = small_graph(n, pairs, seed)
        d = torch.from_numpy(indptr).cuda()
        out = torch.empty(n, dtype=torch.int32, device="cuda")
        L.UnifiedCache.degree_order(0, d, out)
        np.testing.assert_array_equal(out.cpu().numpy(), oracle_mod.degree_order(indptr))


@pytest.mark.parametrize("kg", [2, 4, 8])
def test_clique_striped_cache_on_one_device(oracle_mod, kg):
    """The kg members of a clique emulated on one GPU: every member holds its stripe, the others'
    stripes are reached through the partition pointer table exactly as peer memory would be."""
    rng = np.random.default_rng(kg)
    indptr, _ = small_graph(6000, 80000, 5)
    n = len(indptr) - 1
    table = rng.standard_normal((n, 128)).astype(np.float32)
    ids_list = rng.integers(0, n, 3000).astype(np.int32)
    cap = n // (kg * 2)  # half of the table cached over the clique
    order = oracle_mod.degree_order(indptr)
    rigs = [Rig(table, ids_list, 3000, capacity=cap, kg=kg, ki=ki, order=order) for ki in range(kg)]
    for a in range(kg):
        for b in range(kg):
            if a != b:
                rigs[a].cache.set_peer(b, rigs[b].cache.partition()[0])
    lut = oracle_mod.static_cache_lut(order, cap, kg)
    parts = [oracle_mod.static_cache_fill(order, cap, kg, ki, table) for ki in range(kg)]
    ci = oracle_mod.find_feat(ids_list, lut)
    ref = oracle_mod.gather(ids_list, ci, cap, parts, table)
    for ki in (0, kg - 1):
        cnt, feat, _ = rigs[ki].gather(0)
        np.testing.assert_array_equal(feat.view(np.float32), ref)
        np.testing.assert_array_equal(rigs[ki].pool.read(L.BUF_CACHE_INDEX, 0, cnt, np.int32), ci)
        st = rigs[ki].cache.stats()
        owner = ci[ci >= 0] // cap
        assert st["local_hits"] == int((owner == ki).sum())
        assert st["peer_hits"] == int((owner != ki).sum())
        assert st["misses"] == int((ci < 0).sum())
    for r in rigs:
        r.close()


@pytest.mark.parametrize("kg,codec", [(2, L.CODEC_RAW), (4, L.CODEC_RAW), (8, L.CODEC_RAW), (4, L.CODEC_INT8)])
def test_clique_with_private_replicas(oracle_mod, kg, codec):
    """Hot rows that the striping gave to peers, copied into a member's own memory: gathered rows are
    unchanged, the replicated nodes turn from peer hits into local hits, and the cache index names
    them as member `kg`."""
    rng = np.random.default_rng(40 + kg)
    indptr, _ = small_graph(6000, 80000, 5)
    n = len(indptr) - 1
    table = rng.standard_normal((n, 128)).astype(np.float32)
    ids_list = rng.integers(0, n, 3000).astype(np.int32)
    cap = n // (kg * 2)
    n_rep = cap // 3
    order = oracle_mod.degree_order(indptr)
    rigs = [Rig(table, ids_list, 3000, capacity=cap, kg=kg, ki=ki, order=order, codec=codec) for ki in range(kg)]
    for a in range(kg):
        for b in range(kg):
            if a != b:
                rigs[a].cache.set_peer(b, rigs[b].cache.partition()[0])
    lut = oracle_mod.static_cache_lut(order, cap, kg)
    ci = oracle_mod.find_feat(ids_list, lut)
    if codec == L.CODEC_RAW:
        parts = [oracle_mod.static_cache_fill(order, cap, kg, ki, table) for ki in range(kg)]
        ref = oracle_mod.gather(ids_list, ci, cap, parts, table)
    else:
        parts = [oracle_mod.quant_rows(table[order[ki:cap * kg:kg]], codec) for ki in range(kg)]
        ref = oracle_mod.gather_quant(ids_list, ci, cap, parts, table, codec)
    rank_of = np.full(n, -1, np.int64)
    rank_of[order] = np.arange(n)
    for ki in (0, kg - 1):
        cnt, before, _ = rigs[ki].gather(0)
        np.testing.assert_array_equal(before.view(np.uint32), ref.view(np.uint32))
        st0 = rigs[ki].cache.stats()
        rigs[ki].cache.add_replicas(rigs[ki].order, n_rep)
        with pytest.raises(L.LegionError, match="already holds replicas"):
            rigs[ki].cache.add_replicas(rigs[ki].order, n_rep)
        with pytest.raises(L.LegionError, match="replicas"):
            rigs[ki].cache.lut_ptr()
        # the s-th rank that is not this member's own, in rank order
        foreign = np.array([t for t in range(cap * kg) if t % kg != ki][:n_rep])
        slot_of_rank = {int(t): s for s, t in enumerate(foreign)}
        cnt, after, _ = rigs[ki].gather(0)
        np.testing.assert_array_equal(after, before)
        got_ci = rigs[ki].pool.read(L.BUF_CACHE_INDEX, 0, cnt, np.int32)
        want_ci = ci.copy()
        for i, v in enumerate(ids_list):
            s = slot_of_rank.get(int(rank_of[v]))
            if s is not None:
                want_ci[i] = kg * cap + s
        np.testing.assert_array_equal(got_ci, want_ci)
        st1 = rigs[ki].cache.stats()
        moved = int(sum(1 for v in ids_list if int(rank_of[v]) in slot_of_rank))
        owner = ci[ci >= 0] // cap
        assert moved > 0
        assert st1["local_hits"] - st0["local_hits"] == int((owner == ki).sum()) + moved
        assert st1["peer_hits"] - st0["peer_hits"] == int((owner != ki).sum()) - moved
        assert st1["misses"] - st0["misses"] == int((ci < 0).sum())
    single = Rig(table, ids_list, 3000, capacity=cap, kg=1, ki=0, order=order)
    with pytest.raises(L.LegionError, match="nothing to replicate"):
        single.cache.add_replicas(single.order, 10)
    single.close()
    for r in rigs:
        r.close()


def test_partitions_shared_through_file_descriptors(oracle_mod):
    """The cross-process path on one GPU: a member's partition is exported as a file descriptor and
    mapped a second time through it, as a peer process would; rows read through that mapping are the
    rows of the partition."""
    import os
    rng = np.random.default_rng(3)
    indptr, _ = small_graph(8000, 100000, 6)
    n = len(indptr) - 1
    table = rng.standard_normal((n, 128)).astype(np.float32)
    ids_list = rng.integers(0, n, 6000).astype(np.int32)
    kg, cap = 2, n // 4
    order = oracle_mod.degree_order(indptr)
    rigs = [Rig(table, ids_list, 6000, capacity=cap, kg=kg, ki=ki, order=order) for ki in range(kg)]
    fds = []
    for a in range(kg):
        fd, nbytes = rigs[1 - a].cache.export_partition()
        assert fd >= 0 and nbytes >= cap * 512 and nbytes % (2 << 20) == 0
        rigs[a].cache.import_peer(1 - a, fd, nbytes)
        fds.append(fd)
    for fd in fds:
        os.close(fd)
    lut = oracle_mod.static_cache_lut(order, cap, kg)
    parts = [oracle_mod.static_cache_fill(order, cap, kg, ki, table) for ki in range(kg)]
    ci = oracle_mod.find_feat(ids_list, lut)
    ref = oracle_mod.gather(ids_list, ci, cap, parts, table)
    for ki in range(kg):
        cnt, feat, _ = rigs[ki].gather(0)
        np.testing.assert_array_equal(feat.view(np.float32), ref)
        st = rigs[ki].cache.stats()
        assert st["peer_hits"] == int(((ci >= 0) & (ci // cap != ki)).sum()) and st["peer_hits"] > 0
    with pytest.raises(L.LegionError):
        rigs[0].cache.import_peer(0, 0, 1 << 21)  # own index
    single = Rig(table, ids_list, 6000, capacity=cap, kg=1, ki=0, order=order)
    with pytest.raises(L.LegionError, match="not allocated as shareable"):
        single.cache.export_partition()
    single.close()
    for r in rigs:
        r.close()


@pytest.mark.parametrize("codec", [L.CODEC_INT8, L.CODEC_E4M3])
@pytest.mark.parametrize("feat_len", [100, 128])
def test_compressed_cache(oracle_mod, codec, feat_len):
    rng = np.random.default_rng(codec * 10 + feat_len)
    indptr, _ = small_graph(3000, 40000, 9)
    n = len(indptr) - 1
    table = rng.standard_normal((n, feat_len)).astype(np.float32)
    table[5] = 0.0                      # an all-zero row: scale 0
    table[6, 0] = 1e-30                 # tiny values next to a large one
    table[6, 1] = 300.0
    ids_list = rng.integers(0, n, 4000).astype(np.int32)
    ids_list[:8] = np.arange(8)
    cap = n // 2
    order = np.arange(n, dtype=np.int32)  # rows 0..cap-1 cached
    rig = Rig(table, ids_list, 4000, capacity=cap, codec=codec, order=order)
    rq = oracle_mod.quant_row_bytes(feat_len)
    part = oracle_mod.quant_rows(table[:cap], codec)
    p, b = rig.cache.partition()
    assert b == cap * rq
    got_part = np.empty(b, np.uint8)
    L._check(L.lib().legion_copy(got_part.ctypes.data_as(L.C.c_void_p), L.C.c_void_p(p), L.C.c_int64(b), L.C.c_int32(2)))
    np.testing.assert_array_equal(got_part.reshape(cap, rq), part)
    lut = oracle_mod.static_cache_lut(order, cap, 1)
    ci = oracle_mod.find_feat(ids_list, lut)
    ref = oracle_mod.gather_quant(ids_list, ci, cap, [part], table, codec)
    cnt, feat, _ = rig.gather(0)
    got = feat.view(np.float32).reshape(cnt, feat_len)
    np.testing.assert_array_equal(got.view(np.uint32), ref.view(np.uint32))
    # stated tolerance against the fp32 rows
    exact = table[ids_list]
    absmax = np.abs(exact).max(axis=1, keepdims=True)
    if codec == L.CODEC_INT8:
        tol = absmax / 254.0 + absmax * 2.0 ** -22 + 1e-30   # half a quantisation step + fp32 rounding
    else:
        tol = np.maximum(np.abs(exact) * 2.0 ** -4, absmax / 448.0 * 2.0 ** -10) * (1 + 1e-5) + 1e-30  # half ulp of e4m3
    assert (np.abs(got - exact) <= tol).all()
    hit = ci >= 0
    np.testing.assert_array_equal(got[~hit], exact[~hit])  # misses are raw fp32 rows
    rig.close()


@pytest.mark.parametrize("codec", [L.CODEC_INT8, L.CODEC_E4M3])
@pytest.mark.parametrize("feat_len,kg", [(128, 1), (100, 1), (256, 1), (128, 2)])
def test_compressed_host_table(oracle_mod, codec, feat_len, kg):
    """Host table held as compressed rows: the table encoder matches the host quantiser byte for byte,
    the cache is filled with copies of those rows, and hits, peer hits, replicas and host-link misses all
    decode to the host dequantiser's values."""
    import torch
    rng = np.random.default_rng(codec * 100 + feat_len)
    indptr, _ = small_graph(3000, 40000, 9)
    n = len(indptr) - 1
    table = rng.standard_normal((n, feat_len)).astype(np.float32)
    table[5] = 0.0
    table[6, :2] = (1e-30, 300.0)
    rq = oracle_mod.quant_row_bytes(feat_len)
    want_rows = oracle_mod.quant_rows(table, codec)
    src = torch.from_numpy(table).pin_memory()
    stored = torch.zeros((n, rq), dtype=torch.uint8).pin_memory()
    L.quantize_table(0, codec, src, n, feat_len, stored)
    np.testing.assert_array_equal(stored.numpy(), want_rows)
    with pytest.raises(L.LegionError, match="feature_len % 4"):
        L.quantize_table(0, codec, src, n, 3, stored)

    ids_list = rng.integers(0, n, 4000).astype(np.int32)
    ids_list[:8] = np.arange(8)
    ids_list[9] = -1
    ids = torch.from_numpy(ids_list).cuda()
    lab = torch.zeros_like(ids)
    cap = n // (3 * kg)
    order_np = oracle_mod.degree_order(indptr)
    order = torch.from_numpy(order_np.astype(np.int32)).cuda()
    feats = L.FeatureStorage(0, n, feat_len * 4, stored)
    feats.set_split(L.TRAINMODE, ids, lab)
    caches, pools = [], []
    for ki in range(kg):
        c = L.UnifiedCache(0, n, feat_len * 4, cap, kg, ki, codec)
        c.set_host_codec(codec)
        c.fill_static(order, stored)
        caches.append(c)
        pools.append(L.MemoryPool(0, 4000, [], feat_len * 4, 2))
    with pytest.raises(L.LegionError, match="same codec"):
        raw = L.UnifiedCache(0, n, feat_len * 4, cap, 1, 0, L.CODEC_RAW)
        try:
            raw.set_host_codec(codec)
        finally:
            raw.close()
    for a in range(kg):
        for b in range(kg):
            if a != b:
                caches[a].set_peer(b, caches[b].partition()[0])
    if kg > 1:
        caches[0].add_replicas(order, cap // 2)
    # every member's partition is a copy of the stored rows
    for ki in range(kg):
        p, b = caches[ki].partition()
        got_part = np.empty(b, np.uint8)
        L._check(L.lib().legion_copy(got_part.ctypes.data_as(L.C.c_void_p), L.C.c_void_p(p), L.C.c_int64(b), L.C.c_int32(2)))
        np.testing.assert_array_equal(got_part.reshape(cap, rq), want_rows[order_np[ki:cap * kg:kg]])
    valid = ids_list >= 0
    want = oracle_mod.dequant_rows(want_rows[ids_list[valid]], feat_len, codec)
    for ki in range(kg):
        pools[ki].set_batch(0, L.TRAINMODE, 0, 0)
        L.BatchGenerate(None, feats, caches[ki], pools[ki], 4000, 0, 0, 0, L.TRAINMODE, False, 0)
        L.FeatureCacheLookup(None, caches[ki], pools[ki], 1, 0)
        L.IOComplete(None, caches[ki], pools[ki], 0, L.TRAINMODE)
        got = pools[ki].read(L.BUF_FEATURES, 0, 4000 * feat_len * 4, np.uint8).view(np.float32).reshape(4000, feat_len)
        np.testing.assert_array_equal(got[valid].view(np.uint32), want.view(np.uint32))
        st = caches[ki].stats()
        assert st["misses"] > 0 and st["local_hits"] > 0 and (kg == 1 or st["peer_hits"] > 0)
    for c in caches:
        c.close()
    for p_ in pools:
        p_.close()
    feats.close()


@pytest.mark.parametrize("ways,sets,feat_len", [(8, 64, 128), (4, 100, 32), (32, 7, 128), (1, 50, 4), (16, 33, 384)])
def test_lru_cache_sequence(oracle_mod, ways, sets, feat_len):
    """Hot-set workload of the reference's stale dynamic-cache smoke test (1000 nodes, 130 hot ids
    hit 90% of the time): per-batch hit / miss sets, cache state and rows follow the host replay."""
    rng = np.random.default_rng(ways)
    n = 1000
    table = rng.standard_normal((n, feat_len)).astype(np.float32)
    hot = rng.integers(0, n, 130)
    batches = []
    for _ in range(30):
        pick = np.where(rng.random(128) < 0.9, hot[rng.integers(0, 130, 128)], rng.integers(0, n, 128))
        batches.append(np.unique(pick).astype(np.int32)[:128])  # ids of a batch are unique after dedup
    bsz = 128
    flat = np.full(30 * bsz, -1, np.int32)
    for i, b in enumerate(batches):
        flat[i * bsz: i * bsz + len(b)] = rng.permutation(b)
    rig = Rig(table, flat, bsz, lru=(sets, ways))
    ref = oracle_mod.LruCache(sets, ways)
    rows_ref = np.zeros((sets * ways, feat_len), np.float32)
    total_inserts = 0
    for it in range(30):
        ids = flat[it * bsz:(it + 1) * bsz]
        clock = rig.cache.lru_clock()
        assert clock == it + 1
        cnt, feat, _ = rig.gather(it, pipe=it % 2)
        assert cnt == bsz
        ci = ref.lookup(ids, clock)
        got_ci = rig.pool.read(L.BUF_CACHE_INDEX, it % 2, cnt, np.int64)
        np.testing.assert_array_equal(got_ci, ci)
        valid = ids >= 0
        got = feat.view(np.float32).reshape(cnt, feat_len)
        np.testing.assert_array_equal(got[valid], table[ids[valid]])
        n_ins, slot = ref.insert(ids, ci, clock)
        total_inserts += n_ins
        for r in np.nonzero(slot >= 0)[0]:
            rows_ref[slot[r]] = table[ids[r]]
        k, s, rw = rig.cache.lru_state()
        keys = np.empty(sets * ways, np.int32); stamps = np.empty(sets * ways, np.int32)
        rows = np.empty((sets * ways, feat_len), np.float32)
        for dst, src in ((keys, k), (stamps, s), (rows, rw)):
            L._check(L.lib().legion_copy(dst.ctypes.data_as(L.C.c_void_p), L.C.c_void_p(src), L.C.c_int64(dst.nbytes),
                                         L.C.c_int32(2)))
        np.testing.assert_array_equal(keys, ref.keys)
        np.testing.assert_array_equal(stamps, ref.stamps)
        live = ref.keys >= 0
        np.testing.assert_array_equal(rows[live], rows_ref[live])
        np.testing.assert_array_equal(rows[live], table[ref.keys[live]])
    st = rig.cache.stats()
    assert st["lru_inserts"] == total_inserts
    assert st["local_hits"] > 0 and st["misses"] > 0
    rig.close()


def test_gather_full_size_rows_roundtrip(oracle_mod):
    """Paper100M-sized batch (2.3 M rows of 512 B, cache at 20%): every output row equals its
    source row, checked through a per-row checksum computed on both sides."""
    import torch
    rng = np.random.default_rng(0)
    n = 400000
    table = rng.integers(-2**31, 2**31 - 1, (n, 128), dtype=np.int64).astype(np.int32)
    ids_list = rng.integers(0, n, 2288000).astype(np.int32)
    indptr, _ = small_graph(n, 2000000, 13)
    order = oracle_mod.degree_order(indptr)
    cap = n // 5
    rig = Rig(table, ids_list, len(ids_list), capacity=cap, order=order)
    cnt, feat, _ = rig.gather(0)
    assert cnt == len(ids_list)
    got_sum = feat.view(np.int32).reshape(cnt, 128).astype(np.int64).sum(axis=1)
    ref_sum = table.astype(np.int64).sum(axis=1)[ids_list]
    np.testing.assert_array_equal(got_sum, ref_sum)
    sample = rng.integers(0, cnt, 5000)
    np.testing.assert_array_equal(feat.view(np.int32).reshape(cnt, 128)[sample], table[ids_list[sample]])
    st = rig.cache.stats()
    lut = oracle_mod.static_cache_lut(order, cap, 1)
    assert st["local_hits"] == int((lut[ids_list] >= 0).sum())
    rig.close()


def test_host_register_makes_plain_memory_readable_by_kernels(oracle_mod):
    """Host memory that CUDA did not allocate (here a numpy array standing for a shared segment) is
    page-locked once and then serves as the host table; registering it again is not an error."""
    import torch
    rng = np.random.default_rng(77)
    n, f = 3000, 64
    table = rng.standard_normal((n, f)).astype(np.float32)          # pageable
    t = torch.from_numpy(table)
    L.host_register(0, t)
    L.host_register(0, t)
    ids_list = rng.integers(0, n, 2000).astype(np.int32)
    ids = torch.from_numpy(ids_list).cuda()
    feats = L.FeatureStorage(0, n, f * 4, t)
    feats.set_split(L.TRAINMODE, ids, torch.zeros_like(ids))
    cache = L.UnifiedCache(0, n, f * 4, 0)
    cache.set_host_table(t)
    pool = L.MemoryPool(0, 2000, [], f * 4, 2)
    pool.set_batch(0, L.TRAINMODE, 0, 0)
    L.BatchGenerate(None, feats, cache, pool, 2000, 0, 0, 0, L.TRAINMODE, False, 0)
    L.FeatureCacheLookup(None, cache, pool, 1, 0)
    L.IOComplete(None, cache, pool, 0, L.TRAINMODE)
    got = pool.read(L.BUF_FEATURES, 0, 2000 * f, np.float32).reshape(2000, f)
    np.testing.assert_array_equal(got, table[ids_list])
    with pytest.raises(L.LegionError):
        L._check(L.lib().legion_host_register(L.C.c_int32(0), L.C.c_void_p(0), L.C.c_int64(4096)))
    pool.close(); cache.close(); feats.close()
    assert int(torch.cuda.cudart().cudaHostUnregister(t.data_ptr())) == 0


@pytest.mark.parametrize("feat_len,dtype,kg", [(128, np.float32, 1), (100, np.float32, 1), (256, np.float32, 1),
                                               (768, np.float16, 1), (128, np.float32, 4)])
def test_bulk_copy_engine_gathers_the_same_rows(oracle_mod, feat_len, dtype, kg):
    """The gather that moves rows by bulk asynchronous copies through shared memory (opt-in engine 1):
    same rows, same hit / miss index and same counters as the register path, and no device error."""
    rng = np.random.default_rng(500 + feat_len + kg)
    indptr, _ = small_graph(6000, 80000, 5)
    n = len(indptr) - 1
    table = rng.standard_normal((n, feat_len)).astype(dtype)
    ids_list = rng.integers(0, n, 5000).astype(np.int32)
    ids_list[7] = -1
    cap = n // (kg * 3)
    order = oracle_mod.degree_order(indptr)
    rigs = [Rig(table, ids_list, 5000, capacity=cap, kg=kg, ki=ki, order=order) for ki in range(kg)]
    for a in range(kg):
        for b in range(kg):
            if a != b:
                rigs[a].cache.set_peer(b, rigs[b].cache.partition()[0])
    valid = ids_list >= 0
    try:
        L._check(L.lib().legion_set_tunable(b"gather_engine", 0))
        cnt0, feat0, nc0 = rigs[0].gather(0)
        ci0 = rigs[0].pool.read(L.BUF_CACHE_INDEX, 0, cnt0, np.int32)
        L._check(L.lib().legion_set_tunable(b"gather_engine", 1))
        cnt1, feat1, nc1 = rigs[0].gather(0, pipe=1)   # the other pipe's buffers: nothing left over from engine 0
        ci1 = rigs[0].pool.read(L.BUF_CACHE_INDEX, 1, cnt1, np.int32)
    finally:
        L._check(L.lib().legion_set_tunable(b"gather_engine", 0))
    assert cnt0 == cnt1
    np.testing.assert_array_equal(feat1[valid], feat0[valid])
    np.testing.assert_array_equal(feat1[valid], table[ids_list[valid]].view(np.uint8).reshape(int(valid.sum()), -1))
    np.testing.assert_array_equal(ci1, ci0)
    np.testing.assert_array_equal(nc1, nc0)
    assert rigs[0].pool.device_error() == 0
    with pytest.raises(L.LegionError):
        L._check(L.lib().legion_set_tunable(b"gather_engine", 2))
    for r in rigs:
        r.close()


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_native_cache_plan_matches_the_host_planner(oracle_mod, world):
    """legion_cache_plan (weights scanned on the device) picks the split that server.plan_clique_cache
    picks from the same weights, for degree weights and for presampled counts."""
    import torch
    from legion_ibp_b200 import server
    indptr, _ = small_graph(20000, 300000, 13)
    n = len(indptr) - 1
    d_indptr = torch.from_numpy(indptr).cuda()
    order = torch.empty(n, dtype=torch.int32, device="cuda")
    L.UnifiedCache.degree_order(0, d_indptr, order)
    rng = np.random.default_rng(world)
    counts = torch.from_numpy(rng.zipf(1.5, n).clip(0, 10 ** 6).astype(np.int32)).cuda()
    corder = torch.empty(n, dtype=torch.int32, device="cuda")
    L.UnifiedCache.hotness_order(0, counts, corder)

    def cost(mass, stripe, rep):
        c_l, c_p, c_h = server.ROW_COST
        if world == 1:
            return c_h * (1 - mass(stripe)) + c_l * mass(stripe)
        cov = min(n, stripe * world)
        top = min(cov, rep * world // (world - 1))
        return (c_h * (1 - mass(cov)) + c_p * (mass(cov) - mass(top)) * (world - 1) / world +
                c_l * (mass(top) + (mass(cov) - mass(top)) / world))

    for budget in (n // 50, n // 10, n // 5, n):
        for kind in ("degree", "counts"):
            if kind == "degree":
                mass = server.degree_mass(d_indptr, order)
                got = L.UnifiedCache.plan(0, order, n, budget, world, indptr=d_indptr)
            else:
                mass = server.weight_mass(counts, corder)
                got = L.UnifiedCache.plan(0, corder, n, budget, world, counts=counts)
            want = server.plan_clique_cache(mass, n, budget, world)
            assert got[0] + got[1] <= budget and got[1] <= got[0]
            assert got == tuple(want) or abs(cost(mass, *got) - cost(mass, *want)) <= 1e-9 * max(1.0, cost(mass, *want))
    with pytest.raises(L.LegionError):
        L.UnifiedCache.plan(0, order, n, 10, 2)     # neither degrees nor counts


@pytest.mark.parametrize("kg", [1, 4])
def test_table_spread_over_the_clique_without_a_host_copy(oracle_mod, kg):
    """The MAG240M-shaped layout: legion_cache_place_static builds the lookup table only, every member writes the
    rows of its own stripe into its partition (row s = node order[s * kg + ki], made on the fly from the node id),
    and there is no host table at all.  Every node is cached somewhere, so every row of a gather must come back,
    local or from a peer, bit for bit; the clique is emulated on one GPU."""
    import torch
    from legion_ibp_b200 import synth
    indptr, _ = small_graph(9000, 110000, 5)
    n, f = len(indptr) - 1, 768
    row_bytes = f * 2                                        # 768 x fp16 = 1536-byte rows
    order = oracle_mod.degree_order(indptr)
    d_order = torch.from_numpy(order).cuda()
    cap = (n + kg - 1) // kg
    rng = np.random.default_rng(kg)
    ids_list = rng.integers(0, n, 6000).astype(np.int32)
    d_ids = torch.from_numpy(ids_list).cuda()
    caches = []
    for ki in range(kg):
        c = L.UnifiedCache(0, n, row_bytes, cap, kg=kg, ki=ki)
        c.place_static(d_order)
        t = torch.arange(cap, device="cuda", dtype=torch.int64) * kg + ki
        t = t[t < n]
        c.write_partition_rows(0, synth.feature_rows(d_order[t], f, 0, torch.float16))
        with pytest.raises(L.LegionError, match="outside the partition"):
            c.write_partition_rows(cap, synth.feature_rows(d_order[t[:1]], f, 0, torch.float16))
        caches.append(c)
    for a in range(kg):
        for b in range(kg):
            if a != b:
                caches[a].set_peer(b, caches[b].partition()[0])
    fs = L.FeatureStorage(0, n, row_bytes, None)
    fs.set_split(L.TRAINMODE, d_ids, torch.zeros_like(d_ids))
    want = synth.feature_rows(d_ids, f, 0, torch.float16).cpu().numpy().view(np.uint8).reshape(len(ids_list), row_bytes)
    for ki in (0, kg - 1):
        pool = L.MemoryPool(0, len(ids_list), [], row_bytes, 1)
        pool.set_batch(0, L.TRAINMODE, 0, 0)
        L.BatchGenerate(None, fs, caches[ki], pool, len(ids_list), 0, 0, 0, L.TRAINMODE, False, 0)
        L.FeatureCacheLookup(None, caches[ki], pool, 1, 0)
        got = pool.read(L.BUF_FEATURES, 0, len(ids_list) * row_bytes, np.uint8).reshape(len(ids_list), row_bytes)
        np.testing.assert_array_equal(got, want)
        ci = pool.read(L.BUF_CACHE_INDEX, 0, len(ids_list), np.int32)
        np.testing.assert_array_equal(ci, oracle_mod.find_feat(ids_list, oracle_mod.static_cache_lut(order, cap, kg)))
        assert (ci >= 0).all()
        st = caches[ki].stats()
        assert st["misses"] == 0 and (st["peer_hits"] > 0) == (kg > 1)
        pool.close()
    for c in caches:
        c.close()
    fs.close()
