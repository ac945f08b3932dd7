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
