"""The CUDA library against the REFERENCE's own cache kernels, run on the same GPU and inputs.

oracle/_ref/ref_cache_driver (built from oracle/ref_gpu/ref_cache_driver.cu, which only includes the
reference's cache/cache_impl.cuh and its bucketed cuckoo hash table) runs InitPair + bcht insert,
FeatFillUp, bcht find and multiGPU_feat_cache_lookup.  Hit / miss index per row and gathered rows
must be bit-identical to this library's lookup + gather, for one GPU and for a clique emulated on
one device.  The binary is built where the reference tree is present; without it the test skips.
"""
import os
import subprocess

import numpy as np
import pytest

import legion_ibp_b200 as L
from conftest import ROOT, small_graph
from test_gpu_gather import Rig

pytestmark = pytest.mark.gpu

DRIVER = os.path.join(ROOT, "oracle", "_ref", "ref_cache_driver")


def run_reference(tmp_path, order, table, ids, capacity, kg, ki):
    n, f = table.shape
    inp, out = tmp_path / "in.bin", tmp_path / "out.bin"
    with open(inp, "wb") as fh:
        np.array([n, f, capacity, kg, ki, len(ids)], np.int64).tofile(fh)
        order.astype(np.int32).tofile(fh)
        table.astype(np.float32).tofile(fh)
        ids.astype(np.int32).tofile(fh)
    r = subprocess.run([DRIVER, str(inp), str(out)], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, timeout=300)
    assert r.returncode == 0, r.stdout.decode()[-2000:]
    raw = np.fromfile(out, dtype=np.uint8)
    ci = raw[:4 * len(ids)].view(np.int32)
    rows = raw[4 * len(ids):].view(np.float32).reshape(len(ids), f)
    return ci, rows


@pytest.mark.skipif(not os.path.exists(DRIVER), reason="reference driver not built (needs the reference tree)")
@pytest.mark.parametrize("feat_len,kg", [(128, 1), (100, 1), (128, 4), (100, 2)])
def test_lookup_and_gather_match_the_reference_kernels(oracle_mod, tmp_path, feat_len, kg):
    rng = np.random.default_rng(feat_len + kg)
    indptr, _ = small_graph(30000, 300000, 23)
    n = len(indptr) - 1
    table = rng.standard_normal((n, feat_len)).astype(np.float32)
    ids = rng.integers(0, n, 20000).astype(np.int32)
    cap = n // (kg * 4)  # a quarter of the table cached over the clique
    order = oracle_mod.degree_order(indptr)
    ref_ci, ref_rows = run_reference(tmp_path, order, table, ids, cap, kg, 0)
    # the reference rows are bit copies of the table, and its index is the t % Kg / t / Kg striping
    np.testing.assert_array_equal(ref_rows, table[ids])
    np.testing.assert_array_equal(ref_ci, oracle_mod.find_feat(ids, oracle_mod.static_cache_lut(order, cap, kg)))
    assert (ref_ci >= 0).any() and (ref_ci < 0).any()
    rigs = [Rig(table, ids, len(ids), capacity=cap, kg=kg, ki=ki, order=order) for ki in range(kg)]
    for a in range(kg):
        for b in range(kg):
            if a != b:
                rigs[a].cache.set_peer(b, rigs[b].cache.partition()[0])
    cnt, feat, _ = rigs[0].gather(0)
    np.testing.assert_array_equal(rigs[0].pool.read(L.BUF_CACHE_INDEX, 0, cnt, np.int32), ref_ci)
    np.testing.assert_array_equal(feat.view(np.float32).reshape(cnt, feat_len).view(np.uint32), ref_rows.view(np.uint32))
    for r in rigs:
        r.close()


OPS_DRIVER = os.path.join(ROOT, "oracle", "_ref", "ref_ops_driver")


def run_reference_ops(tmp_path, n_nodes, batch_size, counter, all_ids, all_labels, hops):
    """hops: list of (src_global, dst_global, new_nodes) per hop.  Returns the reference kernels' counter
    trace [2 + 2 * hops][2][16], sampled_ids, labels, agg_src_off, agg_dst_off and the number of
    position_map entries that ClearPosMap left non-zero."""
    inp, out = tmp_path / "ops_in.bin", tmp_path / "ops_out.bin"
    with open(inp, "wb") as fh:
        np.array([n_nodes, batch_size, counter, len(all_ids), len(hops)], np.int64).tofile(fh)
        all_ids.astype(np.int32).tofile(fh)
        all_labels.astype(np.int32).tofile(fh)
        for src, dst, new in hops:
            np.array([len(src), len(new)], np.int64).tofile(fh)
            src.astype(np.int32).tofile(fh)
            dst.astype(np.int32).tofile(fh)
            new.astype(np.int32).tofile(fh)
    r = subprocess.run([OPS_DRIVER, str(inp), str(out)], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, timeout=300)
    assert r.returncode == 0, (r.returncode, r.stdout.decode()[-2000:])
    raw = np.fromfile(out, dtype=np.int32)
    n_snap = 2 + 2 * len(hops)
    trace = raw[:32 * n_snap].reshape(n_snap, 2, 16)
    nc, ec = trace[-1, 0], trace[-1, 1]
    n_total, n_edges = int(nc[9 + len(hops)]), int(ec[0] + ec[1])
    p = 32 * n_snap
    ids = raw[p:p + n_total]; p += n_total
    labels = raw[p:p + batch_size]; p += batch_size
    src_off = raw[p:p + n_edges]; p += n_edges
    dst_off = raw[p:p + n_edges]; p += n_edges
    nonzero = int(raw[p:p + 2].view(np.int64)[0])
    return trace, ids, labels, src_off, dst_off, nonzero


@pytest.mark.skipif(not os.path.exists(OPS_DRIVER), reason="reference driver not built (needs the reference tree)")
@pytest.mark.parametrize("batch,fanout,it", [(96, [25, 10], 2), (800, [25, 10], 0), (64, [15, 10, 5], 3), (200, [5], 1)])
def test_batch_generate_counters_and_relabel_match_the_reference_kernels(oracle_mod, tmp_path, batch, fanout, it):
    """batch_generate, counter_update, construct_graph and ClearPosMap of the reference
    (engine/operator_impl.cu:28-91,304-317,598-604), run on this GPU, against the CPU checker and against
    this library.  The reference's sampler itself is not run (its picks are not reproducible, and it calls
    __syncthreads() under divergent trip counts): the checker's sampled edges and node order are fed to the
    reference kernels in its place, so what is pinned is everything around the random picks: seed slice
    and labels, the counter trace the trainer parses, and the relabelling of every edge to local ids."""
    import torch
    rng = np.random.default_rng(batch)
    indptr, indices = small_graph(20000, 260000, 31)
    n = len(indptr) - 1
    train = rng.permutation(n)[: batch * 5 + 3].astype(np.int32)
    labels = rng.integers(0, 47, len(train)).astype(np.int32)
    seed, gb = 4242, 17
    ref = oracle_mod.run_batch(indptr, indices, train, labels, batch, it, fanout, gb, seed)
    nc, ec = ref["node_counter"], ref["edge_counter"]
    hops = []
    for h in range(1, len(fanout) + 1):
        lo, cnt = int(ec[12 + h]), int(ec[9 + h])
        src_g = ref["src_global"][lo:lo + cnt]                      # sampled neighbour (global id)
        dst_g = ref["ids"][ref["agg_dst"][lo:lo + cnt]]             # the node it was sampled for
        new = ref["ids"][int(nc[9 + h - 1]):int(nc[9 + h])]          # new nodes in order of appearance
        hops.append((src_g, dst_g, new))
    trace, r_ids, r_lab, r_src, r_dst, nonzero = run_reference_ops(tmp_path, n, batch, it, train, labels, hops)
    # the reference kernels against the checker
    np.testing.assert_array_equal(r_ids, ref["ids"])
    np.testing.assert_array_equal(r_lab, ref["labels"])
    np.testing.assert_array_equal(r_src, ref["agg_src"])
    np.testing.assert_array_equal(r_dst, ref["agg_dst"])
    np.testing.assert_array_equal(trace[-1, 0], nc)
    np.testing.assert_array_equal(trace[-1, 1], ec)
    assert nonzero == 0                                             # ClearPosMap leaves the map empty
    # the whole counter trace, op by op, against the checker's counter_update
    t_nc, t_ec = np.zeros(16, np.int32), np.zeros(16, np.int32)
    oracle_mod.counter_update(t_nc, t_ec, 0, batch, len(fanout))
    np.testing.assert_array_equal(trace[0, 0], t_nc); np.testing.assert_array_equal(trace[0, 1], t_ec)
    oracle_mod.counter_update(t_nc, t_ec, 1)
    np.testing.assert_array_equal(trace[1, 0], t_nc); np.testing.assert_array_equal(trace[1, 1], t_ec)
    for h, (src_g, _, new) in enumerate(hops):
        t_nc[6] += len(new)
        t_ec[2] += len(src_g)
        oracle_mod.counter_update(t_nc, t_ec, 3 * (h + 1))
        np.testing.assert_array_equal(trace[2 + 2 * h, 0], t_nc); np.testing.assert_array_equal(trace[2 + 2 * h, 1], t_ec)
        oracle_mod.counter_update(t_nc, t_ec, 3 * (h + 1) + 1)
        np.testing.assert_array_equal(trace[3 + 2 * h, 0], t_nc); np.testing.assert_array_equal(trace[3 + 2 * h, 1], t_ec)
    # this library's batch against the reference kernels' output, through the operator entry points
    d_ip, d_ix = torch.from_numpy(indptr).cuda(), torch.from_numpy(indices).cuda()
    d_train, d_lab = torch.from_numpy(train).cuda(), torch.from_numpy(labels).cuda()
    g = L.GraphStorage(0, d_ip, d_ix)
    f = L.FeatureStorage(0, n, 16)
    f.set_split(L.TRAINMODE, d_train, d_lab)
    pool = L.MemoryPool(0, batch, fanout, 16, 1)
    pool.set_rng(seed, 64)
    pool.set_batch(it, L.TRAINMODE, 0, gb)
    L.BatchGenerate(None, f, None, pool, batch, it, 0, 0, L.TRAINMODE, False, len(fanout))
    L.FeatureCacheLookup(None, None, pool, 1, 0)
    for h, k in enumerate(fanout):
        L.RandomSample(None, g, None, pool, k, 0, 3 * (h + 1))
        L.FeatureCacheLookup(None, None, pool, 3 * (h + 1) + 1, 0)
        torch.cuda.synchronize()
        np.testing.assert_array_equal(pool.read(L.BUF_NODE_COUNTER, 0, 16, np.int32), trace[3 + 2 * h, 0])
        np.testing.assert_array_equal(pool.read(L.BUF_EDGE_COUNTER, 0, 16, np.int32), trace[3 + 2 * h, 1])
    np.testing.assert_array_equal(pool.read(L.BUF_IDS, 0, len(r_ids), np.int32), r_ids)
    np.testing.assert_array_equal(pool.read(L.BUF_LABELS, 0, batch, np.int32), r_lab)
    np.testing.assert_array_equal(pool.read(L.BUF_AGG_SRC, 0, len(r_src), np.int32), r_src)
    np.testing.assert_array_equal(pool.read(L.BUF_AGG_DST, 0, len(r_dst), np.int32), r_dst)
    assert pool.device_error() == 0
    pool.close(); f.close(); g.close()
