"""The allocation-free gather entry point against the pool-based one.

`legion_gather_rows_noalloc` serves callers that cannot allocate device memory when they call in
(a trainer process whose framework allocator owns the GPU, a serving loop that cannot take a
cudaMalloc in the middle of a step): its scratch is a fixed array inside the library instead of a
LegionPool.  Two calls in a row must give the rows that `FeatureCacheLookup` gives for the same ids,
bit for bit; the second call is shorter and hits / misses differently, so anything the first call
left in the shared array would show.  This file is collected last on purpose.
"""
import ctypes as C

import numpy as np
import pytest

import legion_ibp_b200 as L
from conftest import small_graph

pytestmark = pytest.mark.gpu


def _reference_rows(table_pinned, order_dev, cap, ids_np, n, row_bytes):
    """The existing entry point: seeds = the id list, one lookup + gather through a LegionPool."""
    import torch
    d_ids = torch.from_numpy(ids_np).cuda()
    d_lab = torch.zeros_like(d_ids)
    f = L.FeatureStorage(0, n, row_bytes, table_pinned)
    f.set_split(L.TRAINMODE, d_ids, d_lab)
    cache = L.UnifiedCache(0, n, row_bytes, cap)
    cache.fill_static(order_dev, table_pinned)
    pool = L.MemoryPool(0, len(ids_np), [], row_bytes, 1)
    pool.set_batch(0, L.TRAINMODE, 0, 0)
    L.BatchGenerate(None, f, cache, pool, len(ids_np), 0, 0, 0, L.TRAINMODE, False, 0)
    L.FeatureCacheLookup(None, cache, pool, 1, 0)
    out = pool.read(L.BUF_FEATURES, 0, len(ids_np) * row_bytes, np.uint8).reshape(len(ids_np), row_bytes)
    ci = pool.read(L.BUF_CACHE_INDEX, 0, len(ids_np), np.int32)
    pool.close(); f.close()
    return out, ci, cache


@pytest.mark.parametrize("feat_len", [128, 100, 3])
def test_two_calls_match_the_pool_based_entry_point(oracle_mod, feat_len):
    import torch
    rng = np.random.default_rng(feat_len)
    indptr, _ = small_graph(20000, 200000, 17)
    n = len(indptr) - 1
    table = rng.standard_normal((n, feat_len)).astype(np.float32)
    row_bytes = feat_len * 4
    h_table = torch.from_numpy(table).pin_memory()
    order = torch.from_numpy(oracle_mod.degree_order(indptr)).cuda()
    cap = n // 5
    calls = [rng.integers(0, n, 50000).astype(np.int32), rng.integers(0, n, 777).astype(np.int32)]
    calls[1][5] = -1  # an invalid id leaves its row untouched
    calls[1][9] = n   # and so does an id past the table
    side = torch.cuda.Stream()
    # a first call makes the driver load the kernels this row size uses (code is loaded lazily, which takes
    # device memory once per kernel); the calls below must then leave the device's free memory where it was
    warm_ids = torch.arange(64, dtype=torch.int32, device="cuda")
    warm_out = torch.zeros((64, row_bytes), dtype=torch.uint8, device="cuda")
    L.gather_rows_noalloc(None, 0, warm_ids, 0, 0, 1, 0, [], h_table, n, row_bytes, warm_out)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(warm_out.cpu().numpy().view(np.float32), table[:64])
    for k, ids_np in enumerate(calls):
        want, ci, cache = _reference_rows(h_table, order, cap, ids_np, n, row_bytes)
        part_ptr, _ = cache.partition()
        d_ids = torch.from_numpy(ids_np).cuda()
        out = torch.full((len(ids_np), row_bytes), 0xA5, dtype=torch.uint8, device="cuda")
        torch.cuda.synchronize()
        # the property the entry point exists for: device memory in use does not move across the call
        # (the second call runs on a stream of its own)
        free_before, _ = torch.cuda.mem_get_info()
        reserved_before = torch.cuda.memory_reserved()
        L.gather_rows_noalloc(side if k == 1 else None, 0, d_ids, cache.lut_ptr(), cap, 1, 0, [part_ptr], h_table, n,
                              row_bytes, out)
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before
        assert torch.cuda.memory_reserved() == reserved_before
        got = out.cpu().numpy()
        valid = (ids_np >= 0) & (ids_np < n)
        np.testing.assert_array_equal(got[valid], want[valid])                       # bit-exact
        np.testing.assert_array_equal(got[valid].view(np.float32), table[ids_np[valid]])
        assert (got[~valid] == 0xA5).all()
        assert (ci[valid] >= 0).any() and (ci[valid] < 0).any()                      # both sources were exercised
        cache.close()


def test_rejects_lists_above_the_built_in_scratch():
    import torch
    ids = torch.zeros(8, dtype=torch.int32, device="cuda")
    out = torch.zeros(8 * 16, dtype=torch.uint8, device="cuda")
    rc = L.lib().legion_gather_rows_noalloc(None, 0, C.c_void_p(ids.data_ptr()), C.c_int64(L.NOALLOC_MAX_ROWS + 1),
                                            None, 0, 1, 0, None, None, C.c_int64(10), 16, C.c_void_p(out.data_ptr()))
    assert rc == -4
    assert b"above the built-in scratch" in L.lib().legion_last_error()
