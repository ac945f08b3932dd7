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
