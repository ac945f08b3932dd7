"""Whole-batch paths: the two-stream runner with batches in flight, the host-buffer call, and the
hand-off to a trainer process over CUDA IPC + semaphores."""
import os
import subprocess
import sys

import numpy as np
import pytest

import legion_ibp_b200 as L
from conftest import ROOT, small_graph

pytestmark = pytest.mark.gpu


def _world(oracle_mod, n=5000, pairs=70000, feat_len=128, batch=96, fanout=(25, 10), cached_frac=0.3, seed=0, pipes=2,
           slots=None):
    import torch
    rng = np.random.default_rng(seed)
    indptr, indices = small_graph(n, pairs, seed)
    table = rng.standard_normal((n, feat_len)).astype(np.float32)
    train = rng.permutation(n)[: batch * 6 + 5].astype(np.int32)
    labels = rng.integers(0, 47, len(train)).astype(np.int32)
    w = dict(indptr=indptr, indices=indices, table=table, train=train, labels=labels, batch=batch,
             fanout=list(fanout), n=n)
    w["d_indptr"] = torch.from_numpy(indptr).cuda()
    w["d_indices"] = torch.from_numpy(indices).cuda()
    w["h_table"] = torch.from_numpy(table).pin_memory()
    w["g"] = L.GraphStorage(0, w["d_indptr"], w["d_indices"])
    w["f"] = L.FeatureStorage(0, n, feat_len * 4, w["h_table"])
    w["d_train"] = torch.from_numpy(train).cuda()
    w["d_labels"] = torch.from_numpy(labels).cuda()
    w["f"].set_split(L.TRAINMODE, w["d_train"], w["d_labels"])
    cap = int(n * cached_frac)
    order = oracle_mod.degree_order(indptr)
    w["cache"] = L.UnifiedCache(0, n, feat_len * 4, cap)
    w["d_order"] = torch.from_numpy(order).cuda()
    w["cache"].fill_static(w["d_order"], w["h_table"])
    w["pool"] = L.MemoryPool(0, batch, list(fanout), feat_len * 4, pipes, slots=slots)
    w["pool"].set_rng(99, 64)
    return w


def _check_pipe(oracle_mod, w, pipe, it, global_batch):
    pool = w["pool"]
    ref = oracle_mod.run_batch(w["indptr"], w["indices"], w["train"], w["labels"], w["batch"], it, w["fanout"],
                               global_batch, 99)
    nc = pool.read(L.BUF_NODE_COUNTER, pipe, 16, np.int32)
    ec = pool.read(L.BUF_EDGE_COUNTER, pipe, 16, np.int32)
    np.testing.assert_array_equal(nc, ref["node_counter"])
    np.testing.assert_array_equal(ec, ref["edge_counter"])
    n_nodes, n_edges = len(ref["ids"]), len(ref["agg_src"])
    np.testing.assert_array_equal(pool.read(L.BUF_IDS, pipe, n_nodes, np.int32), ref["ids"])
    np.testing.assert_array_equal(pool.read(L.BUF_AGG_SRC, pipe, n_edges, np.int32), ref["agg_src"])
    np.testing.assert_array_equal(pool.read(L.BUF_AGG_DST, pipe, n_edges, np.int32), ref["agg_dst"])
    np.testing.assert_array_equal(pool.read(L.BUF_LABELS, pipe, int(nc[9]), np.int32), ref["labels"])
    feat = pool.read(L.BUF_FEATURES, pipe, n_nodes * w["table"].shape[1], np.float32).reshape(n_nodes, -1)
    np.testing.assert_array_equal(feat, w["table"][ref["ids"]])


@pytest.mark.parametrize("use_graph", [True, False])
def test_runner_two_batches_in_flight(oracle_mod, use_graph):
    w = _world(oracle_mod)
    r = L.Runner(0, w["g"], w["f"], w["cache"], w["pool"], None)
    r.set_options(use_graph=use_graph, time_kernels=True)
    # pairs of batches are enqueued back to back, then both pipes are checked
    for it in range(0, 6, 2):
        r.enqueue(it, L.TRAINMODE, it)
        r.enqueue(it + 1, L.TRAINMODE, it + 1)
        r.sync()
        _check_pipe(oracle_mod, w, 0, it, it)
        _check_pipe(oracle_mod, w, 1, it + 1, it + 1)
        t = r.timing()
        assert t["batches"] == 2 and t["timed"] == 2 and t["batch_ms"] > 0 and t["gather_ms"] > 0 and t["miss_ms"] > 0
    # many batches without a sync in between: only the last two survive in the pipes
    for it in range(6):
        r.enqueue(10 + it, L.TRAINMODE, it)
    r.sync()
    _check_pipe(oracle_mod, w, 0, 4, 14)
    _check_pipe(oracle_mod, w, 1, 5, 15)
    assert w["pool"].device_error() == 0
    r.RunOnce(20, L.TRAINMODE, 2)
    _check_pipe(oracle_mod, w, 0, 2, 20)
    # switching the launch mode in the middle of a run keeps the results
    r.set_options(use_graph=not use_graph, time_kernels=False)
    r.enqueue(31, L.TRAINMODE, 3)
    r.enqueue(32, L.TRAINMODE, 4)
    r.sync()
    _check_pipe(oracle_mod, w, 1, 3, 31)
    _check_pipe(oracle_mod, w, 0, 4, 32)
    assert r.timing()["timed"] == 0
    r.Finalize()


def test_runner_with_lru_cache_keeps_batches_in_order(oracle_mod):
    """Graph replay with an LRU cache: hit / miss sets of consecutive batches follow the host replay,
    which inserts the rows of batch k before looking up batch k+1."""
    import torch
    w = _world(oracle_mod, n=3000, pairs=40000, feat_len=128, batch=64, fanout=(10, 5), seed=8)
    sets, ways = 256, 8
    cache = L.UnifiedCache(0, w["n"], 128 * 4, 0, lru=(sets, ways))
    cache.set_host_table(w["h_table"])
    ref = oracle_mod.LruCache(sets, ways)
    for use_graph in (True, False):
        r = L.Runner(0, w["g"], w["f"], cache, w["pool"], None)
        r.set_options(use_graph=use_graph)
        base = 0 if use_graph else 4
        for it in range(4):
            r.enqueue(base + it, L.TRAINMODE, (base + it) % 6)
        r.sync()
        # replay all four, compare the two that are still in the pipes and the final cache state
        for it in range(4):
            b = oracle_mod.run_batch(w["indptr"], w["indices"], w["train"], w["labels"], w["batch"], (base + it) % 6,
                                     w["fanout"], base + it, 99)
            clock = base + it + 1
            ci = ref.lookup(b["ids"], clock)
            ref.insert(b["ids"], ci, clock)
            if it >= 2:
                pipe = (base + it) % 2
                got_ci = w["pool"].read(L.BUF_CACHE_INDEX, pipe, len(b["ids"]), np.int64)
                np.testing.assert_array_equal(got_ci, ci)
                feat = w["pool"].read(L.BUF_FEATURES, pipe, len(b["ids"]) * 128, np.float32).reshape(-1, 128)
                np.testing.assert_array_equal(feat, w["table"][b["ids"]])
        k, s, _ = cache.lru_state()
        keys = np.empty(sets * ways, np.int32); stamps = np.empty(sets * ways, np.int32)
        for dst, src in ((keys, k), (stamps, s)):
            L._check(L.lib().legion_copy(dst.ctypes.data_as(L.C.c_void_p), L.C.c_void_p(src), L.C.c_int64(dst.nbytes),
                                         L.C.c_int32(2)))
        np.testing.assert_array_equal(keys, ref.keys)
        np.testing.assert_array_equal(stamps, ref.stamps)
        r.Finalize()
    cache.close()


def test_run_batch_host_buffers(oracle_mod):
    w = _world(oracle_mod, seed=3)
    pool = w["pool"]
    ids = np.empty(pool.max_nodes, np.int32); lab = np.empty(w["batch"], np.int32)
    src = np.empty(pool.max_edges, np.int32); dst = np.empty(pool.max_edges, np.int32)
    nc = np.zeros(16, np.int32); ec = np.zeros(16, np.int32)
    feat = np.empty((pool.max_nodes, w["table"].shape[1]), np.float32)
    for it in range(3):
        seeds = w["train"][it * w["batch"]:(it + 1) * w["batch"]]
        labels = w["labels"][it * w["batch"]:(it + 1) * w["batch"]]
        pool.set_batch(it, L.TRAINMODE, it % 2, 40 + it)
        n_nodes, n_edges = L.run_batch_host(w["g"], w["f"], w["cache"], pool, 0, seeds, labels, ids, lab, src, dst,
                                            nc, ec, feat)
        ref = oracle_mod.run_batch(w["indptr"], w["indices"], w["train"], w["labels"], w["batch"], it, w["fanout"],
                                   40 + it, 99)
        assert n_nodes == len(ref["ids"]) and n_edges == len(ref["agg_src"])
        np.testing.assert_array_equal(nc, ref["node_counter"])
        np.testing.assert_array_equal(ec, ref["edge_counter"])
        np.testing.assert_array_equal(ids[:n_nodes], ref["ids"])
        np.testing.assert_array_equal(src[:n_edges], ref["agg_src"])
        np.testing.assert_array_equal(dst[:n_edges], ref["agg_dst"])
        np.testing.assert_array_equal(lab[:len(seeds)], ref["labels"])
        np.testing.assert_array_equal(feat[:n_nodes], w["table"][ref["ids"]])


@pytest.mark.parametrize("use_graph", [True, False])
def test_submit_collect_host_pipelined(oracle_mod, use_graph):
    """Host-buffer batches with two in flight: results arrive in submission order and match the replay."""
    w = _world(oracle_mod, seed=4)
    pool = w["pool"]
    r = L.Runner(0, w["g"], w["f"], w["cache"], pool, None)
    r.set_options(use_graph=use_graph)
    ids = np.empty(pool.max_nodes, np.int32); lab = np.empty(w["batch"], np.int32)
    src = np.empty(pool.max_edges, np.int32); dst = np.empty(pool.max_edges, np.int32)
    nc = np.zeros(16, np.int32); ec = np.zeros(16, np.int32)
    feat = np.empty((pool.max_nodes, w["table"].shape[1]), np.float32)
    b = w["batch"]

    def submit(it):
        r.submit_host(w["train"][it * b:(it + 1) * b], w["labels"][it * b:(it + 1) * b], 70 + it)

    def collect_and_check(it, with_features):
        n_nodes, n_edges = r.collect_host(ids, lab, src, dst, nc, ec, feat if with_features else None)
        ref = oracle_mod.run_batch(w["indptr"], w["indices"], w["train"], w["labels"], b, it, w["fanout"], 70 + it, 99)
        assert n_nodes == len(ref["ids"]) and n_edges == len(ref["agg_src"])
        np.testing.assert_array_equal(nc, ref["node_counter"])
        np.testing.assert_array_equal(ec, ref["edge_counter"])
        np.testing.assert_array_equal(ids[:n_nodes], ref["ids"])
        np.testing.assert_array_equal(src[:n_edges], ref["agg_src"])
        np.testing.assert_array_equal(dst[:n_edges], ref["agg_dst"])
        np.testing.assert_array_equal(lab[:b], ref["labels"])
        if with_features:
            np.testing.assert_array_equal(feat[:n_nodes], w["table"][ref["ids"]])

    submit(0)
    for it in range(1, 6):
        submit(it)
        collect_and_check(it - 1, with_features=(it % 2 == 0))
    submit(0)                       # two in flight now (5 and 0)
    with pytest.raises(L.LegionError, match="in flight"):
        submit(1)
    collect_and_check(5, True)
    collect_and_check(0, True)
    with pytest.raises(L.LegionError, match="nothing was submitted"):
        r.collect_host(ids, lab, src, dst, nc, ec, None)
    r.Finalize()


@pytest.mark.parametrize("use_graph", [True, False])
def test_submit_host_to_writes_pinned_buffers(oracle_mod, use_graph):
    """Output arrays named at submit time: the batch writes ids, labels and edge lists into the
    page-locked buffers itself and collect only returns the counters; contents match the replay."""
    import torch
    w = _world(oracle_mod, seed=5)
    pool = w["pool"]
    r = L.Runner(0, w["g"], w["f"], w["cache"], pool, None)
    r.set_options(use_graph=use_graph)
    b = w["batch"]

    def pinned(n):
        return torch.full((n,), -7, dtype=torch.int32).pin_memory().numpy()
    outs = [dict(ids=pinned(pool.max_nodes), lab=pinned(b), src=pinned(pool.max_edges), dst=pinned(pool.max_edges))
            for _ in range(2)]
    nc = np.zeros(16, np.int32); ec = np.zeros(16, np.int32)

    def submit(it):
        o = outs[it % 2]
        r.submit_host_to(w["train"][it * b:(it + 1) * b], w["labels"][it * b:(it + 1) * b], 30 + it, o["ids"], o["lab"],
                         o["src"], o["dst"])

    def collect_and_check(it):
        n_nodes, n_edges = r.collect_host(None, None, None, None, nc, ec, None)
        o = outs[it % 2]
        ref = oracle_mod.run_batch(w["indptr"], w["indices"], w["train"], w["labels"], b, it, w["fanout"], 30 + it, 99)
        assert n_nodes == len(ref["ids"]) and n_edges == len(ref["agg_src"])
        np.testing.assert_array_equal(nc, ref["node_counter"])
        np.testing.assert_array_equal(ec, ref["edge_counter"])
        np.testing.assert_array_equal(o["ids"][:n_nodes], ref["ids"])
        np.testing.assert_array_equal(o["src"][:n_edges], ref["agg_src"])
        np.testing.assert_array_equal(o["dst"][:n_edges], ref["agg_dst"])
        np.testing.assert_array_equal(o["lab"][:b], ref["labels"])
        # the gathered rows stay in the device hand-off buffer of the batch's pipe
        feat = pool.read(L.BUF_FEATURES, it % 2, n_nodes * w["table"].shape[1], np.float32)
        np.testing.assert_array_equal(feat.reshape(n_nodes, -1), w["table"][ref["ids"]])
        for a in o.values():
            a[:] = -7

    submit(0)
    for it in range(1, 5):
        submit(it)
        collect_and_check(it - 1)
    collect_and_check(4)
    # three deep: the third batch samples and exports while both pipes still hold uncollected batches
    outs.append(dict(ids=pinned(pool.max_nodes), lab=pinned(b), src=pinned(pool.max_edges), dst=pinned(pool.max_edges)))

    def submit3(it):
        o = outs[it % 3]
        r.submit_host_to(w["train"][it * b:(it + 1) * b], w["labels"][it * b:(it + 1) * b], 30 + it, o["ids"], o["lab"],
                         o["src"], o["dst"])

    def collect3(it, pipe):
        n_nodes, n_edges = r.collect_host(None, None, None, None, nc, ec, None)
        o = outs[it % 3]
        ref = oracle_mod.run_batch(w["indptr"], w["indices"], w["train"], w["labels"], b, it, w["fanout"], 30 + it, 99)
        assert n_nodes == len(ref["ids"]) and n_edges == len(ref["agg_src"])
        np.testing.assert_array_equal(nc, ref["node_counter"])
        np.testing.assert_array_equal(ec, ref["edge_counter"])
        np.testing.assert_array_equal(o["ids"][:n_nodes], ref["ids"])
        np.testing.assert_array_equal(o["src"][:n_edges], ref["agg_src"])
        np.testing.assert_array_equal(o["dst"][:n_edges], ref["agg_dst"])
        np.testing.assert_array_equal(o["lab"][:b], ref["labels"])
        feat = pool.read(L.BUF_FEATURES, pipe, n_nodes * w["table"].shape[1], np.float32)
        np.testing.assert_array_equal(feat.reshape(n_nodes, -1), w["table"][ref["ids"]])

    p0 = r.current_pipe()
    for it in range(3):
        submit3(it)
    with pytest.raises(L.LegionError, match="in flight"):
        submit3(3)                      # only one batch may run ahead of the pipes
    for it in range(3, 6):
        collect3(it - 3, (p0 + it - 3) % 2)
        submit3(it)
    for it in range(6, 9):
        collect3(it - 3, (p0 + it - 3) % 2)
    # a plain submit cannot run ahead
    r.submit_host(w["train"][:b], w["labels"][:b], 30)
    r.submit_host(w["train"][b:2 * b], w["labels"][b:2 * b], 31)
    with pytest.raises(L.LegionError, match="in flight"):
        r.submit_host_to(w["train"][:b], w["labels"][:b], 32, outs[0]["ids"], outs[0]["lab"], outs[0]["src"], outs[0]["dst"])
    ids_p = np.empty(pool.max_nodes, np.int32); lab_p = np.empty(b, np.int32)
    src_p = np.empty(pool.max_edges, np.int32); dst_p = np.empty(pool.max_edges, np.int32)
    r.collect_host(ids_p, lab_p, src_p, dst_p, nc, ec, None)
    r.collect_host(ids_p, lab_p, src_p, dst_p, nc, ec, None)
    for o in outs:
        for a in o.values():
            a[:] = -7
    # a NULL array is skipped; pageable memory is refused
    o = outs[1]
    r.submit_host_to(w["train"][:b], w["labels"][:b], 30, o["ids"], None, None, o["dst"])
    r.collect_host(None, None, None, None, nc, ec, None)
    assert (o["src"] == -7).all() and (o["lab"] == -7).all() and o["ids"][0] == w["train"][0]
    with pytest.raises(L.LegionError, match="page-locked"):
        r.submit_host_to(w["train"][:b], w["labels"][:b], 30, np.empty(pool.max_nodes, np.int32), None, None, None)
    r.Finalize()


def test_edge_counts_in_the_place_of_agg_dst(oracle_mod):
    """set_edge_counts: the array named as agg_dst receives one byte per destination and hop; expanding the
    counts gives agg_dst of the replay, through bound buffers (batches of growing then shrinking size, so the
    copy-ahead size is both too small and too large) and through a plain collect."""
    import torch
    w = _world(oracle_mod, seed=11)
    pool = w["pool"]
    r = L.Runner(0, w["g"], w["f"], w["cache"], pool, None)
    b = w["batch"]
    hops = len(w["fanout"])

    def pinned(n, dt=torch.int32):
        return torch.full((n,), -7, dtype=dt).pin_memory().numpy()
    outs = [dict(ids=pinned(pool.max_nodes), lab=pinned(b), src=pinned(pool.max_edges),
                 cnt=pinned(hops * pool.max_nodes + 16, torch.uint8)) for _ in range(2)]
    nc = np.zeros(16, np.int32); ec = np.zeros(16, np.int32)
    r.submit_host(w["train"][:b], w["labels"][:b], 30)
    with pytest.raises(L.LegionError, match="waiting to be collected"):
        r.set_edge_counts(True)
    r.collect_host(None, None, None, None, nc, ec, None)
    r.set_edge_counts(True)
    sizes = [b // 4, b, b // 2, b, 3]

    def seeds_of(it):
        return w["train"][it * b:it * b + sizes[it]], w["labels"][it * b:it * b + sizes[it]]

    def check(it, cnt):
        sd, lb = seeds_of(it)
        ref = oracle_mod.run_batch(w["indptr"], w["indices"], sd, lb, len(sd), 0, w["fanout"], 40 + it, 99)
        np.testing.assert_array_equal(nc, ref["node_counter"])
        n_cnt = int(sum(nc[9 + h] for h in range(hops)))
        assert int(cnt[:n_cnt].astype(np.int64).sum()) == len(ref["agg_dst"])
        np.testing.assert_array_equal(L.agg_dst_from_counts(cnt[:n_cnt], nc), ref["agg_dst"])
        return ref

    for it in range(len(sizes) + 1):
        if it < len(sizes):
            o = outs[it % 2]
            sd, lb = seeds_of(it)
            r.submit_host_to(sd, lb, 40 + it, o["ids"], o["lab"], o["src"], o["cnt"])
        if it >= 1:
            n_nodes, n_edges = r.collect_host(None, None, None, None, nc, ec, None)
            o = outs[(it - 1) % 2]
            ref = check(it - 1, o["cnt"])
            np.testing.assert_array_equal(o["ids"][:n_nodes], ref["ids"])
            np.testing.assert_array_equal(o["src"][:n_edges], ref["agg_src"])
    # plain collect: the counts are copied out at collect time
    sd, lb = seeds_of(1)
    r.submit_host(sd, lb, 41)
    cnt = np.zeros(hops * pool.max_nodes, np.uint8)
    r.collect_host(None, None, None, cnt, nc, ec, None)
    check(1, cnt)
    r.set_edge_counts(False)
    dst = np.zeros(pool.max_edges, np.int32)
    r.submit_host(sd, lb, 41)
    _, n_edges = r.collect_host(None, None, None, dst, nc, ec, None)
    ref = oracle_mod.run_batch(w["indptr"], w["indices"], sd, lb, len(sd), 0, w["fanout"], 41, 99)
    np.testing.assert_array_equal(dst[:n_edges], ref["agg_dst"])
    r.Finalize()


CONSUMER = r'''
import ctypes as C, sys, os, mmap, numpy as np
sys.path.insert(0, os.path.join(sys.argv[1], "tests"))
import conftest
import legion_ibp_b200 as L
# Trainer side, as training_backend/ipc_cuda_kernel.cu:37-106,177-243 does it: open the segment,
# open the 7 handles of each pipe for device 0, post sem_r once per pipe, then per batch
# wait sem_w, read both counters, slice ids / labels / edge lists / features, post sem_r.
shm_name, n_batches, feat_len, out_path = sys.argv[2], int(sys.argv[3]), int(sys.argv[4]), sys.argv[5]
lay = L.ipc_layout()
lib = L.lib()
fd = os.open("/dev/shm/" + shm_name, os.O_RDWR)
seg = mmap.mmap(fd, lay["segment_bytes"])
steps = np.frombuffer(seg, dtype=np.int32, count=3).copy()
class Handle(C.Structure):
    _fields_ = [("reserved", C.c_char * 64)]
ptrs = []
for pipe in range(2):
    row = []
    for k in range(7):
        off = lay["handles_offset"] + ((0 * 2 + pipe) * 7 + k) * 64
        h = Handle.from_buffer_copy(seg[off:off + 64])
        p = C.c_void_p()
        err = lib.legion_ipc_open_handle(C.byref(h), C.byref(p))
        assert err == 0, ("legion_ipc_open_handle", err, pipe, k, lib.legion_last_error())
        row.append(p.value)
    ptrs.append(row)
libc = C.CDLL("libc.so.6", use_errno=True)
libc.sem_open.restype = C.c_void_p
libc.sem_open.argtypes = [C.c_char_p, C.c_int, C.c_uint, C.c_uint]
libc.sem_wait.argtypes = [C.c_void_p]; libc.sem_post.argtypes = [C.c_void_p]
prefix = "" if shm_name == "simpleIPCshm" else shm_name + "_"
semr = [libc.sem_open((prefix + "sem_r_0_%d" % i).encode(), os.O_CREAT | os.O_RDWR, 0o666, 0) for i in range(2)]
semw = [libc.sem_open((prefix + "sem_w_0_%d" % i).encode(), os.O_CREAT | os.O_RDWR, 0o666, 0) for i in range(2)]
for i in range(2):
    libc.sem_post(semr[i])
def d2h(ptr, count, dtype):
    out = np.empty(count, dtype)
    if out.nbytes:
        assert lib.legion_copy(C.c_void_p(out.ctypes.data), C.c_void_p(ptr), C.c_int64(out.nbytes), C.c_int32(2)) == 0
    return out
res = {"steps": steps}
pipe = 0
for b in range(n_batches):
    libc.sem_wait(semw[pipe])
    nc = d2h(ptrs[pipe][5], 16, np.int32); ec = d2h(ptrs[pipe][6], 16, np.int32)
    hops = int(nc[8]); n = int(nc[9 + hops])
    res["nc%d" % b] = nc; res["ec%d" % b] = ec
    res["ids%d" % b] = d2h(ptrs[pipe][0], n, np.int32)
    res["feat%d" % b] = d2h(ptrs[pipe][1], n * feat_len, np.float32)
    res["labels%d" % b] = d2h(ptrs[pipe][2], int(nc[9]), np.int32)
    for i in range(hops, 0, -1):
        eo, en = int(ec[12 + i]), int(ec[9 + i])
        res["src%d_%d" % (b, i)] = d2h(ptrs[pipe][3] + 4 * eo, en, np.int32)
        res["dst%d_%d" % (b, i)] = d2h(ptrs[pipe][4] + 4 * eo, en, np.int32)
    res["blocks%d" % b] = np.array([[nc[9 + i], nc[9 + i - 1]] for i in range(hops, 0, -1)], np.int32)
    libc.sem_post(semr[pipe])
    pipe = (pipe + 1) % 2
for row in ptrs:
    for p in row:
        lib.legion_ipc_close_handle(C.c_void_p(p))
np.savez(out_path, **res)
'''


def test_ipc_handoff_to_trainer_process(oracle_mod, tmp_path):
    """A second process plays the trainer extension; the server serves 5 batches through the
    shared segment and the semaphores, with a bounded wait so that a lost trainer cannot hang it."""
    w = _world(oracle_mod, seed=5)
    shm = "legion_b200_test_%d" % os.getpid()
    env = L.IPCEnv(1, shm)
    env.Coordinate([len(w["train"])], [1], [1], w["batch"], 1)
    steps = env.steps()
    assert steps[0] == (len(w["train"]) - 1) // w["batch"]
    env.publish_pool(w["pool"], 0)
    script = tmp_path / "consumer.py"
    script.write_text(CONSUMER)
    out = tmp_path / "consumer.npz"
    n_batches = 5
    proc = subprocess.Popen([sys.executable, str(script), ROOT, shm, str(n_batches), str(w["table"].shape[1]), str(out)],
                            stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    r = L.Runner(0, w["g"], w["f"], w["cache"], w["pool"], env)
    try:
        r.serve(0, n_batches, timeout_ms=120000)
        stdout, _ = proc.communicate(timeout=120)
    finally:
        if proc.poll() is None:
            proc.kill()
    assert proc.returncode == 0, stdout.decode()[-2000:]
    got = np.load(out)
    np.testing.assert_array_equal(got["steps"], steps)
    for b in range(n_batches):
        ref = oracle_mod.run_batch(w["indptr"], w["indices"], w["train"], w["labels"], w["batch"], b, w["fanout"], b, 99)
        np.testing.assert_array_equal(got["nc%d" % b], ref["node_counter"])
        np.testing.assert_array_equal(got["ec%d" % b], ref["edge_counter"])
        np.testing.assert_array_equal(got["ids%d" % b], ref["ids"])
        np.testing.assert_array_equal(got["labels%d" % b], ref["labels"])
        np.testing.assert_array_equal(got["feat%d" % b].reshape(len(ref["ids"]), -1), w["table"][ref["ids"]])
        ec = ref["edge_counter"]
        for i in (2, 1):
            lo, cnt = int(ec[12 + i]), int(ec[9 + i])
            np.testing.assert_array_equal(got["src%d_%d" % (b, i)], ref["agg_src"][lo:lo + cnt])
            np.testing.assert_array_equal(got["dst%d_%d" % (b, i)], ref["agg_dst"][lo:lo + cnt])
        # DGL block convention: dst nodes are a prefix of src nodes
        blocks = got["blocks%d" % b]
        assert blocks[0][1] == blocks[1][0] and blocks[1][1] == w["batch"]
        assert got["src%d_2" % b].max() < blocks[0][0] and got["dst%d_2" % b].max() < blocks[0][1]
    # the trainer is gone now: the next wait must time out instead of blocking for ever
    with pytest.raises(L.LegionError, match="did not release"):
        r.RunOnce(n_batches, L.TRAINMODE, 0, timeout_ms=300)
        r.RunOnce(n_batches + 1, L.TRAINMODE, 1, timeout_ms=300)
        r.RunOnce(n_batches + 2, L.TRAINMODE, 1, timeout_ms=300)
    r.Finalize()
    env.Finalize()
    assert not os.path.exists("/dev/shm/" + shm)


def test_dataset_files_to_batches_with_topology_in_host_memory(oracle_mod, tmp_path):
    """From Legion-format files to served batches: the loader puts CSR and features in mapped pinned
    host memory, the sampler reads the topology in place (zero-copy, as the reference does for
    uncached adjacency lists), and the result equals the host replay."""
    import torch
    from test_dataset_cpu import meta_for, write_dataset
    ref = write_dataset(tmp_path / "ds", n=4000, f=32, seed=3)
    meta = meta_for(tmp_path / "ds", ref, f=32)
    ds = L.Dataset(meta, pin=True)
    n = meta.node_num
    g = L.GraphStorage(0, ds.indptr, ds.indices)           # host pointers, read through UVA
    f = L.FeatureStorage(0, n, 32 * 4, ds.features)
    ids, lab = ds.split(L.TRAINMODE, 1, 0)
    d_ids, d_lab = torch.from_numpy(ids).cuda(), torch.from_numpy(lab).cuda()
    f.set_split(L.TRAINMODE, d_ids, d_lab)
    d_ip = torch.from_numpy(np.ascontiguousarray(ds.indptr)).cuda()
    order = torch.empty(n, dtype=torch.int32, device="cuda")
    L.UnifiedCache.degree_order(0, d_ip, order)
    cache = L.UnifiedCache(0, n, 32 * 4, n // 10)
    cache.fill_static(order, ds.features)
    pool = L.MemoryPool(0, 48, [25, 10], 32 * 4, 2)
    pool.set_rng(5, 64)
    r = L.Runner(0, g, f, cache, pool, None)
    w = dict(pool=pool, indptr=ref["indptr"], indices=ref["indices"], train=ids, labels=lab, batch=48, fanout=[25, 10],
             table=ref["feats"])
    for it in range(0, 4, 2):
        r.enqueue(it, L.TRAINMODE, it)
        r.enqueue(it + 1, L.TRAINMODE, it + 1)
        r.sync()
        for pipe in (0, 1):
            b = oracle_mod.run_batch(w["indptr"], w["indices"], ids, lab, 48, it + pipe, [25, 10], it + pipe, 5)
            np.testing.assert_array_equal(pool.read(L.BUF_IDS, pipe, len(b["ids"]), np.int32), b["ids"])
            np.testing.assert_array_equal(pool.read(L.BUF_AGG_SRC, pipe, len(b["agg_src"]), np.int32), b["agg_src"])
            np.testing.assert_array_equal(pool.read(L.BUF_NODE_COUNTER, pipe, 16, np.int32), b["node_counter"])
            feat = pool.read(L.BUF_FEATURES, pipe, len(b["ids"]) * 32, np.float32).reshape(-1, 32)
            np.testing.assert_array_equal(feat, ref["feats"][b["ids"]])
    r.Finalize(); pool.close(); cache.close(); f.close(); g.close(); ds.close()


def test_presampling_hotness_and_ranking(oracle_mod):
    """RunPreSc + CandidateSelection: access counts of a presampling epoch and the ranking made from
    them equal the host replay (counts by bincount over the replayed batches, order by (-count, id))."""
    import torch
    w = _world(oracle_mod, n=6000, pairs=80000, batch=64, fanout=(25, 10), seed=12)
    r = L.Runner(0, w["g"], w["f"], w["cache"], w["pool"], None)
    counts = torch.zeros(w["n"], dtype=torch.int32, device="cuda")
    n_batches = (len(w["train"]) - 1) // w["batch"]      # train_step of the reference
    r.presample(0, n_batches, counts)
    want = np.zeros(w["n"], np.int64)
    for it in range(n_batches):
        b = oracle_mod.run_batch(w["indptr"], w["indices"], w["train"], w["labels"], w["batch"], it, w["fanout"], it, 99)
        want += np.bincount(b["ids"], minlength=w["n"])
    np.testing.assert_array_equal(counts.cpu().numpy(), want)
    order = torch.empty(w["n"], dtype=torch.int32, device="cuda")
    L.UnifiedCache.hotness_order(0, counts, order)
    np.testing.assert_array_equal(order.cpu().numpy(), np.lexsort((np.arange(w["n"]), -want)).astype(np.int32))
    # a cache filled in that order serves the same rows
    cache = L.UnifiedCache(0, w["n"], 128 * 4, w["n"] // 10)
    cache.fill_static(order, w["h_table"])
    r2 = L.Runner(0, w["g"], w["f"], cache, w["pool"], None)
    r2.enqueue(3, L.TRAINMODE, 3)
    r2.sync()
    b = oracle_mod.run_batch(w["indptr"], w["indices"], w["train"], w["labels"], w["batch"], 3, w["fanout"], 3, 99)
    feat = w["pool"].read(L.BUF_FEATURES, 0, len(b["ids"]) * 128, np.float32).reshape(-1, 128)
    np.testing.assert_array_equal(feat, w["table"][b["ids"]])
    hot_hits = cache.stats()["local_hits"]
    assert hot_hits > 0
    r.Finalize(); r2.Finalize(); cache.close()


CLIENT = r'''
import sys, os, numpy as np, ctypes as C
sys.path.insert(0, os.path.join(sys.argv[1], "tests"))
import conftest
import legion_ibp_b200 as L
shm_name, n_batches, feat_len, out_path = sys.argv[2], int(sys.argv[3]), int(sys.argv[4]), sys.argv[5]
svc = L.ipc_service(0, shm_name)
assert svc.counters_on_host()
def d2h(ptr, count, dtype):
    out = np.empty(count, dtype)
    if out.nbytes:
        L._check(L.lib().legion_copy(C.c_void_p(out.ctypes.data), C.c_void_p(ptr), C.c_int64(out.nbytes), C.c_int32(2)))
    return out
res = {"steps": np.array(svc.get_steps(), np.int32)}
for b in range(n_batches):
    v = svc.get_next(timeout_ms=120000)
    res["ids%d" % b] = d2h(v.ids, v.n_ids, np.int32)
    res["feat%d" % b] = d2h(v.features, v.n_ids * feat_len, np.float32)
    res["labels%d" % b] = d2h(v.labels, v.n_labels, np.int32)
    res["blocks%d" % b] = np.array(svc.get_block_size(), np.int32)
    for j in range(v.hop_num):
        res["src%d_%d" % (b, j)] = d2h(v.agg_src[j], v.n_edges[j], np.int32)
        res["dst%d_%d" % (b, j)] = d2h(v.agg_dst[j], v.n_edges[j], np.int32)
    svc.synchronize()
svc.finalize()
np.savez(out_path, **res)
'''


@pytest.mark.parametrize("pipes", [2, 4])
def test_client_api_consumes_batches(oracle_mod, tmp_path, pipes):
    """The trainer-side C-ABI client (initialize / get_next / get_block_size / get_steps / synchronize /
    finalize) in a second process, fed by legion_runner_serve.  With four pipes behind the two hand-off slots
    the server samples up to four batches ahead of the trainer into private buffers and copies each block
    structure into its slot when the slot is free; what the trainer sees must not change."""
    w = _world(oracle_mod, seed=6, pipes=pipes, slots=2)
    shm = "legion_b200_cli_%d" % os.getpid()
    env = L.IPCEnv(1, shm)
    env.Coordinate([len(w["train"])], [1], [1], w["batch"], 1)
    env.publish_pool(w["pool"], 0)
    script = tmp_path / "client.py"
    script.write_text(CLIENT)
    out = tmp_path / "client.npz"
    n_batches = 6
    proc = subprocess.Popen([sys.executable, str(script), ROOT, shm, str(n_batches), str(w["table"].shape[1]), str(out)],
                            stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    r = L.Runner(0, w["g"], w["f"], w["cache"], w["pool"], env)
    if pipes == 4:
        r.stage_seeds(L.TRAINMODE)
    try:
        r.serve(0, n_batches, timeout_ms=120000)
        stdout, _ = proc.communicate(timeout=120)
    finally:
        if proc.poll() is None:
            proc.kill()
    assert proc.returncode == 0, stdout.decode()[-2000:]
    got = np.load(out)
    np.testing.assert_array_equal(got["steps"], env.steps())
    for b in range(n_batches):
        ref = oracle_mod.run_batch(w["indptr"], w["indices"], w["train"], w["labels"], w["batch"], b, w["fanout"], b, 99)
        nc, ec = ref["node_counter"], ref["edge_counter"]
        np.testing.assert_array_equal(got["ids%d" % b], ref["ids"])
        np.testing.assert_array_equal(got["labels%d" % b], ref["labels"])
        np.testing.assert_array_equal(got["feat%d" % b].reshape(len(ref["ids"]), -1), w["table"][ref["ids"]])
        assert list(got["blocks%d" % b]) == [nc[11], nc[10], nc[10], nc[9]]   # get_block_size, last hop first
        for j, hop in enumerate((2, 1)):
            lo, cnt = int(ec[12 + hop]), int(ec[9 + hop])
            np.testing.assert_array_equal(got["src%d_%d" % (b, j)], ref["agg_src"][lo:lo + cnt])
            np.testing.assert_array_equal(got["dst%d_%d" % (b, j)], ref["agg_dst"][lo:lo + cnt])
    r.Finalize()
    env.Finalize()


def test_sampling_server_binary_end_to_end(oracle_mod, tmp_path):
    """The server binary as the reference is started (`sampling_server <ngpu> <cache_agg_mode> <dyn_flags>`
    in a directory holding ./meta_config): it loads Legion-format files, prints the ready line that
    scripts/wait_file.sh waits for, and serves the whole schedule (train, validation, test batches of all
    epochs) to a trainer, which here is this process using the client API."""
    import select
    import time
    from test_dataset_cpu import meta_for, write_dataset
    ref = write_dataset(tmp_path / "ds", n=3000, f=16, seed=5)
    meta = meta_for(tmp_path / "ds", ref, f=16)
    meta.raw_batch_size = 24
    meta.epoch = 2
    meta.cache_memory = 16 * 4 * 600          # room for 600 rows
    meta.write(str(tmp_path / "meta_config"))
    shm = "legion_b200_srv_%d" % os.getpid()
    env = dict(os.environ, LEGION_SHM_NAME=shm, LEGION_ORDER="degree", LEGION_SEED="7", LEGION_TIMEOUT_MS="120000")
    binary = os.path.join(ROOT, "legion-ibp_b200", "sampling_server")
    assert os.path.exists(binary), "build the library first (make -C legion-ibp_b200/csrc)"
    proc = subprocess.Popen([binary, "1", "0", "0"], cwd=str(tmp_path), env=env, stdout=subprocess.PIPE,
                            stderr=subprocess.STDOUT)
    try:
        seen, deadline = b"", time.time() + 120
        while b"System is ready for serving" not in seen:
            assert time.time() < deadline and proc.poll() is None, seen.decode()[-2000:]
            if select.select([proc.stdout], [], [], 1.0)[0]:
                seen += os.read(proc.stdout.fileno(), 4096)
        svc = L.ipc_service(0, shm)
        assert svc.counters_on_host()     # this library's server publishes them; no device copy per batch
        train, valid, test = ref["train"], ref["valid"], ref["test"]
        steps, vbs, tbs = oracle_mod.coordinate([len(train)], [len(valid)], [len(test)], 24)
        assert svc.get_steps() == list(steps)
        total = (steps[0] + steps[1]) * 2 + steps[2]
        lists = {0: (train, 24), 1: (valid, int(vbs[0])), 2: (test, int(tbs[0]))}
        for b in range(total):
            v = svc.get_next(timeout_ms=120000)
            mode, local = oracle_mod.mode_of_batch(b, steps[0], steps[1], steps[2], 2)
            ids_all, bs = lists[mode]
            want = oracle_mod.run_batch(ref["indptr"], ref["indices"], ids_all, ref["labels"][ids_all], bs, local, [25, 10], b, 7)
            got_ids = np.empty(v.n_ids, np.int32)
            L._check(L.lib().legion_copy(got_ids.ctypes.data_as(L.C.c_void_p), L.C.c_void_p(v.ids), L.C.c_int64(got_ids.nbytes), 2))
            np.testing.assert_array_equal(got_ids, want["ids"], err_msg="batch %d mode %d" % (b, mode))
            np.testing.assert_array_equal(np.array(v.node_counter[:]), want["node_counter"])
            np.testing.assert_array_equal(np.array(v.edge_counter[:]), want["edge_counter"])
            feat = np.empty((v.n_ids, 16), np.float32)
            L._check(L.lib().legion_copy(feat.ctypes.data_as(L.C.c_void_p), L.C.c_void_p(v.features), L.C.c_int64(feat.nbytes), 2))
            np.testing.assert_array_equal(feat, ref["feats"][want["ids"]])
            lab = np.empty(v.n_labels, np.int32)
            L._check(L.lib().legion_copy(lab.ctypes.data_as(L.C.c_void_p), L.C.c_void_p(v.labels), L.C.c_int64(lab.nbytes), 2))
            np.testing.assert_array_equal(lab, want["labels"])
            svc.synchronize()
        svc.finalize()
        out, _ = proc.communicate(timeout=60)
        assert proc.returncode == 0, (seen + out).decode()[-2000:]
        assert b"System finalized" in out
    finally:
        if proc.poll() is None:
            proc.kill()
    assert not os.path.exists("/dev/shm/" + shm)


def test_seed_ids_outside_the_graph_are_skipped_and_reported(oracle_mod):
    """A client that hands in a seed id >= n_nodes (or a topology that stores one) must not make any
    kernel index with it: the slot reads -1 like a slot past the end of the seed list, the rest of the
    batch equals the batch without that seed, and the pool reports error 5."""
    w = _world(oracle_mod)
    r = L.Runner(0, w["g"], w["f"], w["cache"], w["pool"], None)
    b = w["batch"]
    seeds = w["train"][:b].copy()
    labels = w["labels"][:b].copy()
    bad = seeds.copy()
    bad[7] = w["n"]            # first id past the table
    bad[11] = 2 ** 31 - 5      # far outside
    f = w["table"].shape[1]
    outs = {}
    for name, s in (("bad", bad), ("good", seeds)):
        mn, me = w["pool"].max_nodes, w["pool"].max_edges
        ids, lab = np.empty(mn, np.int32), np.empty(b, np.int32)
        src, dst = np.empty(me, np.int32), np.empty(me, np.int32)
        nc, ec = np.zeros(16, np.int32), np.zeros(16, np.int32)
        feat = np.zeros((mn, f), np.float32)
        r.submit_host(s, labels, 5)
        nn, ne = r.collect_host(ids, lab, src, dst, nc, ec, feat)
        outs[name] = (ids[:nn].copy(), src[:ne].copy(), dst[:ne].copy(), feat[:nn].copy())
        err = w["pool"].device_error()
        assert err == (5 if name == "bad" else 0), err
    ids_bad = outs["bad"][0]
    assert ids_bad[7] == -1 and ids_bad[11] == -1
    keep = np.ones(b, bool)
    keep[[7, 11]] = False
    np.testing.assert_array_equal(ids_bad[:b][keep], seeds[keep])
    # every node that was found carries its own row, and none of the ids is out of range
    found = ids_bad >= 0
    assert ids_bad[found].max() < w["n"]
    np.testing.assert_array_equal(outs["bad"][3][found], w["table"][ids_bad[found]])
    # the error word is not sticky for this kind: the next batch is complete again
    np.testing.assert_array_equal(outs["good"][0][:b], seeds)
    assert w["pool"].device_error() == 0
    r.Finalize()


def test_partition_without_shareable_memory_needs_peer_access(oracle_mod, monkeypatch):
    """On a platform without the virtual memory management API a clique partition is plain cudaMalloc
    memory.  legion_cache_allow_device must then either enable peer access for the reading device or
    fail; it must never answer OK and leave the reader with a pointer it cannot dereference."""
    import torch
    monkeypatch.setenv("LEGION_NO_VMM", "1")
    c = L.UnifiedCache(0, 1000, 64, 100, kg=2, ki=0)
    with pytest.raises(L.LegionError):
        c.export_partition()          # not shareable memory
    assert L.lib().legion_cache_allow_device(c.h, 0) == 0   # the owner itself: nothing to do
    rc = L.lib().legion_cache_allow_device(c.h, 1)
    if torch.cuda.device_count() < 2:
        assert rc != 0                 # there is no device 1 to enable: refused, with a message
        assert L.lib().legion_last_error()
    else:
        assert rc == 0                 # peer access of device 1 to device 0 is on now
        assert L.lib().legion_enable_peer_access(1, 0) == 0   # already enabled is not an error
    c.close()


@pytest.mark.parametrize("use_graph", [True, False])
def test_seed_rows_staged_by_the_copy_engine_give_the_same_batches(oracle_mod, use_graph):
    """With seed staging the rows of uncached seeds arrive by a copy-engine transfer from a page-locked
    array in list order instead of zero-copy loads; every output must stay bit-identical, the staged rows
    must no longer be counted (or fetched) as misses, and the last, shorter batch of the list must work."""
    w = _world(oracle_mod, seed=21)
    r = L.Runner(0, w["g"], w["f"], w["cache"], w["pool"], None)
    r.set_options(use_graph=use_graph)
    lut = oracle_mod.static_cache_lut(oracle_mod.degree_order(w["indptr"]), int(w["n"] * 0.3), 1)
    uncached_seed = lut[w["train"]] < 0
    staged_total = r.stage_seeds(L.TRAINMODE)
    assert staged_total == int(uncached_seed.sum()) and staged_total > 0
    n_batches = (len(w["train"]) + w["batch"] - 1) // w["batch"]      # includes the shorter last batch
    s0 = w["cache"].stats()
    want_staged = 0
    for it in range(0, n_batches - 1, 2):
        r.enqueue(it, L.TRAINMODE, it)
        r.enqueue(it + 1, L.TRAINMODE, it + 1)
        r.sync()
        _check_pipe(oracle_mod, w, 0, it, it)
        _check_pipe(oracle_mod, w, 1, it + 1, it + 1)
        want_staged += int(uncached_seed[it * w["batch"]:(it + 2) * w["batch"]].sum())
    assert r.staged_rows() == want_staged
    # the tail batch (5 seeds)
    r.RunOnce(40, L.TRAINMODE, n_batches - 1)
    ref = oracle_mod.run_batch(w["indptr"], w["indices"], w["train"], w["labels"], w["batch"], n_batches - 1, w["fanout"], 40, 99)
    for pipe in (0, 1):
        nc = w["pool"].read(L.BUF_NODE_COUNTER, pipe, 16, np.int32)
        if np.array_equal(nc, ref["node_counter"]):
            feat = w["pool"].read(L.BUF_FEATURES, pipe, len(ref["ids"]) * 128, np.float32).reshape(-1, 128)
            np.testing.assert_array_equal(feat, w["table"][ref["ids"]])
            break
    else:
        raise AssertionError("the tail batch is in neither pipe")
    # staged rows are neither hits nor misses in the cache's counters: fewer misses than uncached rows
    s1 = w["cache"].stats()
    assert s1["misses"] - s0["misses"] > 0
    assert w["pool"].device_error() == 0
    # a refill invalidates the staging: batches still come out right, nothing is staged any more
    w["cache"].fill_static(w["d_order"], w["h_table"])
    before = r.staged_rows()
    r.enqueue(50, L.TRAINMODE, 1)
    r.sync()
    assert r.staged_rows() == before
    r.Finalize()


def test_registered_host_seed_list_is_staged_by_address(oracle_mod):
    """submit_host[_to] with a slice of a registered host list: staged; the same call with a copy of the
    slice, or after the caller changed the list, takes the zero-copy path; the results are identical."""
    w = _world(oracle_mod, seed=22)
    r = L.Runner(0, w["g"], w["f"], w["cache"], w["pool"], None)
    b, f = w["batch"], w["table"].shape[1]
    seeds = w["train"].copy()
    labels = w["labels"].copy()
    r.register_host_seeds(seeds)
    mn, me = w["pool"].max_nodes, w["pool"].max_edges

    def run(seed_arr, it, gb):
        ids, lab = np.empty(mn, np.int32), np.empty(b, np.int32)
        src, dst = np.empty(me, np.int32), np.empty(me, np.int32)
        nc, ec = np.zeros(16, np.int32), np.zeros(16, np.int32)
        feat = np.zeros((mn, f), np.float32)
        r.submit_host(seed_arr, labels[it * b:(it + 1) * b], gb)
        nn, ne = r.collect_host(ids, lab, src, dst, nc, ec, feat)
        ref = oracle_mod.run_batch(w["indptr"], w["indices"], w["train"], w["labels"], b, it, w["fanout"], gb, 99)
        np.testing.assert_array_equal(ids[:nn], ref["ids"])
        np.testing.assert_array_equal(src[:ne], ref["agg_src"])
        np.testing.assert_array_equal(dst[:ne], ref["agg_dst"])
        np.testing.assert_array_equal(nc, ref["node_counter"])
        np.testing.assert_array_equal(feat[:nn], w["table"][ref["ids"]])

    n0 = r.staged_rows()
    run(seeds[2 * b:3 * b], 2, 7)                 # a slice of the registered array
    n1 = r.staged_rows()
    assert n1 > n0
    run(seeds[2 * b:3 * b].copy(), 2, 7)          # the same ids somewhere else in memory
    assert r.staged_rows() == n1
    # three staged batches in flight
    mn_ids = [np.empty(mn, np.int32) for _ in range(2)]
    for k in range(2):
        r.submit_host(seeds[k * b:(k + 1) * b], labels[k * b:(k + 1) * b], 20 + k)
    nc, ec = np.zeros(16, np.int32), np.zeros(16, np.int32)
    for k in range(2):
        feat = np.zeros((mn, f), np.float32)
        nn, ne = r.collect_host(mn_ids[k], None, None, None, nc, ec, feat)
        ref = oracle_mod.run_batch(w["indptr"], w["indices"], w["train"], w["labels"], b, k, w["fanout"], 20 + k, 99)
        np.testing.assert_array_equal(mn_ids[k][:nn], ref["ids"])
        np.testing.assert_array_equal(feat[:nn], w["table"][ref["ids"]])
    assert r.staged_rows() > n1
    # the caller overwrites a seed inside the registered array: that slice no longer matches the staging
    n2 = r.staged_rows()
    old = seeds[4 * b + 3]
    seeds[4 * b + 3] = seeds[0]
    ids, nc, ec = np.empty(mn, np.int32), np.zeros(16, np.int32), np.zeros(16, np.int32)
    feat = np.zeros((mn, f), np.float32)
    r.submit_host(seeds[4 * b:5 * b], labels[4 * b:5 * b], 30)
    nn, _ = r.collect_host(ids, None, None, None, nc, ec, feat)
    assert r.staged_rows() == n2
    np.testing.assert_array_equal(feat[:nn], w["table"][ids[:nn]])
    seeds[4 * b + 3] = old
    assert w["pool"].device_error() == 0
    r.Finalize()


@pytest.mark.parametrize("use_graph", [True, False])
def test_batches_sampled_ahead_of_two_handoff_slots(oracle_mod, use_graph):
    """A pool with four pipes behind two hand-off slots: batches are sampled into private buffers and published
    into slot (batch % 2) when their gather is issued.  Whatever is enqueued, the two slots hold the last two
    batches, bit for bit what the host replay gives, and the per-operator and host-buffer calls refuse such a pool."""
    w = _world(oracle_mod, seed=31, pipes=4, slots=2)
    r = L.Runner(0, w["g"], w["f"], w["cache"], w["pool"], None)
    r.set_options(use_graph=use_graph)
    r.stage_seeds(L.TRAINMODE)
    for it in range(6):
        r.enqueue(it, L.TRAINMODE, it)
    r.sync()
    _check_pipe(oracle_mod, w, 0, 4, 4)
    _check_pipe(oracle_mod, w, 1, 5, 5)
    r.enqueue(6, L.TRAINMODE, 0)
    r.sync()
    _check_pipe(oracle_mod, w, 0, 0, 6)      # batch 6 ran on pipe 2 and was published into slot 0
    _check_pipe(oracle_mod, w, 1, 5, 5)      # slot 1 is untouched
    for it in range(7, 16):
        r.enqueue(it, L.TRAINMODE, it % 6)
    r.sync()
    _check_pipe(oracle_mod, w, 0, 14 % 6, 14)
    _check_pipe(oracle_mod, w, 1, 15 % 6, 15)
    assert w["pool"].device_error() == 0
    with pytest.raises(L.LegionError, match="hand-off slots"):
        r.submit_host(w["train"][:w["batch"]], w["labels"][:w["batch"]], 1)
    with pytest.raises(L.LegionError, match="numbered by slot"):
        w["pool"].buffer(L.BUF_IDS, 3)
    r.Finalize()


def test_host_table_packed_by_rank_serves_the_same_batches(oracle_mod, tmp_path):
    """The loader rewrites the feature table in packed order (uncached rows by rising rank, cached rows last)
    and every GPU gets the matching row-of-id array: the table's rows move, the batches do not change, and the
    staged seed rows are found through the same indirection."""
    import torch
    from test_dataset_cpu import meta_for, write_dataset
    f = 32
    ref = write_dataset(tmp_path / "ds", n=4000, f=f, seed=17)
    meta = meta_for(tmp_path / "ds", ref, f=f)
    ds = L.Dataset(meta, pin=True)
    n = meta.node_num
    d_ip = torch.from_numpy(np.ascontiguousarray(ds.indptr)).cuda()
    d_ix = torch.from_numpy(np.ascontiguousarray(ds.indices)).cuda()
    order = torch.empty(n, dtype=torch.int32, device="cuda")
    L.UnifiedCache.degree_order(0, d_ip, order)
    cap = n // 8
    row_of = torch.empty(n, dtype=torch.int32, device="cuda")
    L.UnifiedCache.pack_order(0, order, cap, row_of)
    before = ds.features.copy()
    ds.pack_features(0, order, cap)
    h_order, h_row_of = order.cpu().numpy(), row_of.cpu().numpy()
    np.testing.assert_array_equal(h_row_of[h_order[cap:]], np.arange(n - cap))          # uncached: by rising rank
    np.testing.assert_array_equal(h_row_of[h_order[:cap]], n - cap + np.arange(cap))    # cached: last
    np.testing.assert_array_equal(ds.features[h_row_of], before)                       # every row moved to its place
    g = L.GraphStorage(0, d_ip, d_ix)
    fs = L.FeatureStorage(0, n, f * 4, ds.features)
    ids, lab = ds.split(L.TRAINMODE, 1, 0)
    d_ids, d_lab = torch.from_numpy(ids).cuda(), torch.from_numpy(lab).cuda()
    fs.set_split(L.TRAINMODE, d_ids, d_lab)
    cache = L.UnifiedCache(0, n, f * 4, cap)
    cache.fill_static(order, ds.features, row_of_id=row_of)
    pool = L.MemoryPool(0, 48, [25, 10], f * 4, 2)
    pool.set_rng(5, 64)
    r = L.Runner(0, g, fs, cache, pool, None)
    assert r.stage_seeds(L.TRAINMODE) > 0
    for it in range(0, 4, 2):
        r.enqueue(it, L.TRAINMODE, it)
        r.enqueue(it + 1, L.TRAINMODE, it + 1)
        r.sync()
        for pipe in (0, 1):
            b = oracle_mod.run_batch(ref["indptr"], ref["indices"], ids, lab, 48, it + pipe, [25, 10], it + pipe, 5)
            np.testing.assert_array_equal(pool.read(L.BUF_IDS, pipe, len(b["ids"]), np.int32), b["ids"])
            feat = pool.read(L.BUF_FEATURES, pipe, len(b["ids"]) * f, np.float32).reshape(-1, f)
            np.testing.assert_array_equal(feat, ref["feats"][b["ids"]])
    st = cache.stats()
    assert st["local_hits"] > 0 and st["misses"] > 0 and r.staged_rows() > 0
    r.Finalize(); pool.close(); cache.close(); fs.close(); g.close(); ds.close()
