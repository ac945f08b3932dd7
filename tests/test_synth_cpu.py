"""The synthetic inputs: features that are a pure function of the node id, and the graph generator's
bucketed sort (edge lists of more than 2^31 keys are sorted range by range)."""
import numpy as np
import torch

from legion_ibp_b200 import synth


def test_feature_rows_are_a_pure_function_of_the_node_id():
    ids = torch.tensor([0, 5, 123456789, 2 ** 31 - 1, 5])
    a = synth.feature_rows(ids, 96)
    b = synth.feature_rows(ids.flip(0), 96).flip(0)
    assert torch.equal(a, b) and torch.equal(a[1], a[4])
    assert not torch.equal(a[0], a[1])
    assert not torch.equal(a, synth.feature_rows(ids, 96, seed=1))
    big = synth.feature_rows(torch.arange(20000), 64)
    assert abs(float(big.mean())) < 0.01 and abs(float(big.std()) - 1.0) < 0.01
    half = synth.feature_rows(ids, 96, dtype=torch.float16)
    assert half.dtype == torch.float16 and torch.equal(half, a.to(torch.float16))


def test_features_into_fills_rows_in_any_order_and_in_slices():
    out = torch.zeros(1000, 16)
    synth.features_into(out, chunk_rows=128)
    assert torch.equal(out[500:510], synth.feature_rows(torch.arange(500, 510), 16))
    perm = torch.randperm(1000, generator=torch.Generator().manual_seed(1)).to(torch.int32)
    out2 = torch.zeros(1000, 16)
    synth.features_into(out2, row_ids=perm, first=100, last=300, chunk_rows=64)
    assert torch.equal(out2[100:300], out[perm[100:300].long()])
    assert float(out2[:100].abs().sum()) == 0.0 and float(out2[300:].abs().sum()) == 0.0


def test_graph_generator_sorts_large_edge_lists_bucket_by_bucket():
    a = synth.rmat_csr(5000, 60000, seed=3)
    b = synth.rmat_csr(5000, 60000, seed=3, max_sort=20000)   # forces 6 buckets
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
    indptr, indices = a[0].numpy(), a[1].numpy()
    assert indptr[0] == 0 and indptr[-1] == len(indices) and (np.diff(indptr) >= 0).all()
    for v in (0, 17, 4999):      # adjacency lists are sorted, without self loops or duplicates
        adj = indices[indptr[v]:indptr[v + 1]]
        assert (np.diff(adj) > 0).all() and (adj != v).all()


def _bench_module():
    import importlib.util
    import os
    from conftest import ROOT
    spec = importlib.util.spec_from_file_location("legion_bench", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_zipf_seed_batches_hold_distinct_ids_for_every_rank():
    """The LRU stress workload's seeds: Zipf draws split by id % world; a rank whose share is dominated by
    one hot id (rank 0 of eight: node 0) still gets whole batches of distinct ids, and one rank gets the
    sequence it always got."""
    bench = _bench_module()
    for world, ranks in ((1, (0,)), (4, (0, 3)), (8, (0, 7))):
        for rank in ranks:
            t = bench.zipf_batches(50_000_000, 512, 6, 1.1, world, rank, device="cpu")
            assert t.dtype == torch.int32 and t.numel() == 6 * 512
            assert bool(((t % world) == rank).all())
            for row in t.view(6, 512):
                assert row.unique().numel() == 512
    a = bench.zipf_batches(50_000_000, 512, 6, 1.1, 1, 0, device="cpu")
    b = bench.zipf_batches(50_000_000, 512, 6, 1.1, 1, 0, device="cpu")
    assert torch.equal(a, b)
    # hot ids come up again and again across batches: that is what the LRU cache lives on
    assert a.unique().numel() < 0.8 * a.numel()


def test_edge_counts_expand_to_agg_dst(oracle_mod):
    """agg_dst_from_counts: per-destination, per-hop edge counts (what legion_runner_set_edge_counts delivers)
    give back the destination list of the checker's batch."""
    import legion_ibp_b200 as L
    from conftest import small_graph
    indptr, indices = small_graph(3000, 30000, 5)
    rng = np.random.default_rng(2)
    train = rng.permutation(3000)[:200].astype(np.int32)
    labels = rng.integers(0, 5, 200).astype(np.int32)
    for fanout in ([25, 10], [5], [15, 10, 5]):
        b = oracle_mod.run_batch(indptr, indices, train, labels, 64, 1, fanout, 9, 3)
        nc, ec = b["node_counter"], b["edge_counter"]
        counts, lo = [], 0
        for h in range(len(fanout)):
            e = int(ec[9 + h + 1])                       # edges of hop h
            counts.append(np.bincount(b["agg_dst"][lo:lo + e], minlength=int(nc[9 + h])).astype(np.uint8))
            lo += e
        np.testing.assert_array_equal(L.agg_dst_from_counts(np.concatenate(counts), nc), b["agg_dst"])
