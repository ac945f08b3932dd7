"""ctypes front end of the CPU checker (``legion_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by the smoke check and by the
CPU-baseline leg of the benchmark.  The product never imports this module.

Each wrapper keeps the name of the C function it calls; the C file cites the reference
lines every function restates.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "liblegion_oracle.so")

CACHEMISS_FLAG = -2
MAX_ROUNDS = 64


def build(force=False):
    src = os.path.join(_HERE, "legion_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s"])
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        _lib = C.CDLL(_SO)
        _lib.orc_sample_hop.restype = C.c_int64
        _lib.orc_run_batch.restype = C.c_int64
        _lib.orc_quant_row_bytes.restype = C.c_int64
        _lib.orc_e4m3_to_float.restype = C.c_float
        _lib.orc_e4m3_to_float.argtypes = [C.c_uint8]
        _lib.orc_float_to_e4m3.restype = C.c_uint8
        _lib.orc_float_to_e4m3.argtypes = [C.c_float]
        _lib.orc_lru_insert.restype = C.c_int64
        _lib.orc_cpu_pipeline.restype = C.c_int64
        _lib.orc_cpu_pipeline_native.restype = C.c_int64
        _lib.orc_num_threads.restype = C.c_int
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def _i64(a):
    return np.ascontiguousarray(a, dtype=np.int64)


def philox4x32_10(ctr, key):
    c = np.asarray(ctr, dtype=np.uint32)
    k = np.asarray(key, dtype=np.uint32)
    out = np.zeros(4, dtype=np.uint32)
    lib().orc_philox4x32_10(_p(c), _p(k), _p(out))
    return out


def sample_hop(indptr, indices, ids, fanout, hop, batch_id, seed, max_rounds=MAX_ROUNDS):
    indptr, indices, ids = _i64(indptr), _i32(indices), _i32(ids)
    cap = max(1, len(ids) * fanout)
    src = np.empty(cap, dtype=np.int32)
    dst = np.empty(cap, dtype=np.int32)
    e = lib().orc_sample_hop(_p(indptr), _p(indices), _p(ids), C.c_int32(len(ids)), C.c_int32(fanout),
                             C.c_int32(hop), C.c_uint32(batch_id), C.c_uint64(seed),
                             C.c_int32(max_rounds), _p(src), _p(dst))
    if e < 0:
        raise ValueError("fanout above 32")
    return src[:e].copy(), dst[:e].copy()


def batch_bounds(batch_size, fanout):
    """Worst-case node and edge counts of one batch (every hop samples all nodes so far)."""
    nodes, edges = batch_size, 0
    for f in fanout:
        e = nodes * f
        edges += e
        nodes += e
    return nodes, edges


def run_batch(indptr, indices, all_ids, all_labels, batch_size, it, fanout, batch_id, seed,
              max_rounds=MAX_ROUNDS):
    """Returns dict(ids, labels, agg_src, agg_dst, node_counter, edge_counter, src_global)."""
    indptr, indices = _i64(indptr), _i32(indices)
    all_ids, all_labels = _i32(all_ids), _i32(all_labels)
    fan = _i32(fanout)
    max_nodes, max_edges = batch_bounds(batch_size, list(fanout))
    ids = np.full(max_nodes + 1, -7, dtype=np.int32)
    labels = np.full(batch_size + 1, -7, dtype=np.int32)
    agg_src = np.full(max_edges + 1, -7, dtype=np.int32)
    agg_dst = np.full(max_edges + 1, -7, dtype=np.int32)
    src_g = np.full(max_edges + 1, -7, dtype=np.int32)
    nc = np.zeros(16, dtype=np.int32)
    ec = np.zeros(16, dtype=np.int32)
    n = lib().orc_run_batch(_p(indptr), _p(indices), _p(all_ids), _p(all_labels),
                            C.c_int32(len(all_ids)), C.c_int32(batch_size), C.c_int32(it),
                            C.c_int32(len(fan)), _p(fan), C.c_uint32(batch_id), C.c_uint64(seed),
                            C.c_int32(max_rounds), _p(ids), _p(labels), _p(agg_src), _p(agg_dst),
                            _p(src_g), _p(nc), _p(ec))
    if n < 0:
        raise RuntimeError("orc_run_batch failed: %d" % n)
    hops = len(fan)
    n_edges = int(ec[0] + ec[1])
    return dict(ids=ids[:n].copy(), labels=labels[:nc[9]].copy(), agg_src=agg_src[:n_edges].copy(),
                agg_dst=agg_dst[:n_edges].copy(), src_global=src_g[:n_edges].copy(),
                node_counter=nc, edge_counter=ec, hops=hops)


def counter_update(nc, ec, op_id, size=0, hop_num=0):
    lib().orc_counter_update(_p(nc), _p(ec), C.c_int32(op_id), C.c_int32(size), C.c_int32(hop_num))


def degree_order(indptr):
    indptr = _i64(indptr)
    n = len(indptr) - 1
    order = np.empty(n, dtype=np.int32)
    if lib().orc_degree_order(_p(indptr), C.c_int32(n), _p(order)) != 0:
        raise MemoryError
    return order


def static_cache_lut(order, capacity, kg):
    order = _i32(order)
    lut = np.empty(len(order), dtype=np.int32)
    lib().orc_static_cache_lut(_p(order), C.c_int32(len(order)), C.c_int32(capacity), C.c_int32(kg), _p(lut))
    return lut


def static_cache_fill(order, capacity, kg, ki, host_table):
    """host_table: 2-D array [N, row]; returns this GPU's partition [capacity, row]."""
    order = _i32(order)
    host_table = np.ascontiguousarray(host_table)
    row_bytes = host_table.strides[0]
    part = np.zeros((capacity,) + host_table.shape[1:], dtype=host_table.dtype)
    lib().orc_static_cache_fill(_p(order), C.c_int32(len(order)), C.c_int32(capacity), C.c_int32(kg),
                                C.c_int32(ki), _p(host_table), C.c_int64(row_bytes), _p(part))
    return part


def find_feat(ids, lut):
    ids, lut = _i32(ids), _i32(lut)
    out = np.empty(len(ids), dtype=np.int32)
    lib().orc_find_feat(_p(ids), C.c_int64(len(ids)), _p(lut), _p(out))
    return out


def gather(ids, cache_index, capacity, parts, host_table, dst=None):
    """parts: list of 2-D arrays (one per GPU of the clique); host_table 2-D [N,row]."""
    ids, cache_index = _i32(ids), _i32(cache_index)
    host_table = np.ascontiguousarray(host_table)
    parts = [np.ascontiguousarray(p) for p in parts]
    row_bytes = host_table.strides[0]
    if dst is None:
        dst = np.zeros((len(ids),) + host_table.shape[1:], dtype=host_table.dtype)
    arr = (C.c_void_p * max(1, len(parts)))(*[p.ctypes.data for p in parts])
    lib().orc_gather(_p(ids), _p(cache_index), C.c_int64(len(ids)), C.c_int32(max(1, capacity)), arr,
                     _p(host_table), C.c_int64(host_table.shape[0]), C.c_int64(row_bytes), _p(dst))
    return dst


def quant_row_bytes(f):
    return int(lib().orc_quant_row_bytes(C.c_int32(f)))


def quant_rows(x, codec):
    """x: [n,F] fp32 -> packed rows [n, quant_row_bytes(F)] uint8.  codec 1=int8, 2=e4m3."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    n, f = x.shape
    rq = quant_row_bytes(f)
    out = np.zeros((n, rq), dtype=np.uint8)
    fn = lib().orc_quant_int8_row if codec == 1 else lib().orc_quant_e4m3_row
    for i in range(n):
        fn(C.c_void_p(x.ctypes.data + i * f * 4), C.c_int32(f), C.c_void_p(out.ctypes.data + i * rq))
    return out


def dequant_rows(rows, f, codec):
    rows = np.ascontiguousarray(rows, dtype=np.uint8)
    n, rq = rows.shape
    out = np.zeros((n, f), dtype=np.float32)
    fn = lib().orc_dequant_int8_row if codec == 1 else lib().orc_dequant_e4m3_row
    for i in range(n):
        fn(C.c_void_p(rows.ctypes.data + i * rq), C.c_int32(f), C.c_void_p(out.ctypes.data + i * f * 4))
    return out


def gather_quant(ids, cache_index, capacity, parts, host_table, codec):
    ids, cache_index = _i32(ids), _i32(cache_index)
    host_table = np.ascontiguousarray(host_table, dtype=np.float32)
    parts = [np.ascontiguousarray(p, dtype=np.uint8) for p in parts]
    f = host_table.shape[1]
    dst = np.zeros((len(ids), f), dtype=np.float32)
    arr = (C.c_void_p * max(1, len(parts)))(*[p.ctypes.data for p in parts])
    lib().orc_gather_quant(_p(ids), _p(cache_index), C.c_int64(len(ids)), C.c_int32(max(1, capacity)), arr,
                           _p(host_table), C.c_int64(host_table.shape[0]), C.c_int32(f), C.c_int32(codec),
                           _p(dst))
    return dst


def float_to_e4m3(x):
    return int(lib().orc_float_to_e4m3(C.c_float(x)))


def e4m3_to_float(b):
    return float(lib().orc_e4m3_to_float(C.c_uint8(b)))


class LruCache:
    """Host replay of the set-associative LRU cache state (keys, stamps)."""

    def __init__(self, sets, ways):
        self.sets, self.ways = int(sets), int(ways)
        self.keys = np.full(self.sets * self.ways, -1, dtype=np.int32)
        self.stamps = np.zeros(self.sets * self.ways, dtype=np.int32)

    def lookup(self, ids, clock):
        ids = _i32(ids)
        out = np.empty(len(ids), dtype=np.int64)
        lib().orc_lru_lookup(_p(self.keys), _p(self.stamps), C.c_int64(self.sets), C.c_int32(self.ways),
                             C.c_int32(clock), _p(ids), C.c_int64(len(ids)), _p(out))
        return out

    def insert(self, ids, cache_index, clock):
        ids, cache_index = _i32(ids), _i64(cache_index)
        slot = np.empty(len(ids), dtype=np.int64)
        n = lib().orc_lru_insert(_p(self.keys), _p(self.stamps), C.c_int64(self.sets), C.c_int32(self.ways),
                                 C.c_int32(clock), _p(ids), _p(cache_index), C.c_int64(len(ids)), _p(slot))
        return int(n), slot


def coordinate(train_num, valid_num, test_num, raw_batch):
    tr, va, te = _i32(train_num), _i32(valid_num), _i32(test_num)
    steps = np.zeros(3, dtype=np.int32)
    vbs = np.zeros(len(tr), dtype=np.int32)
    tbs = np.zeros(len(tr), dtype=np.int32)
    lib().orc_coordinate(_p(tr), _p(va), _p(te), C.c_int32(len(tr)), C.c_int32(raw_batch), _p(steps),
                         _p(vbs), _p(tbs))
    return steps, vbs, tbs


def mode_of_batch(global_batch, train_step, valid_step, test_step, epochs):
    mode, local = C.c_int32(0), C.c_int32(0)
    lib().orc_mode_of_batch(C.c_int32(global_batch), C.c_int32(train_step), C.c_int32(valid_step),
                            C.c_int32(test_step), C.c_int32(epochs), C.byref(mode), C.byref(local))
    return mode.value, local.value


def num_threads():
    """Host cores this process may use.  Launchers such as torchrun export OMP_NUM_THREADS=1 to their
    workers, so the OpenMP default is not the answer; cpu_pipeline sets the count it is given."""
    import os
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or int(lib().orc_num_threads()))


def cpu_pipeline(indptr, indices, all_ids, all_labels, batch_size, first_iter, n_batches, fanout, seed,
                 host_table, threads=0):
    """Timed CPU baseline: sample + relabel + gather for n_batches; returns nodes gathered."""
    indptr, indices = _i64(indptr), _i32(indices)
    all_ids, all_labels = _i32(all_ids), _i32(all_labels)
    fan = _i32(fanout)
    host_table = np.ascontiguousarray(host_table)
    row_bytes = host_table.strides[0]
    t = threads if threads > 0 else num_threads()
    max_nodes, max_edges = batch_bounds(batch_size, list(fanout))
    feat = np.empty(t * max_nodes * row_bytes, dtype=np.uint8)
    scratch = np.empty(t * (max_nodes + 3 * max_edges + batch_size), dtype=np.int32)
    return int(lib().orc_cpu_pipeline(_p(indptr), _p(indices), _p(all_ids), _p(all_labels),
                                      C.c_int32(len(all_ids)), C.c_int32(batch_size), C.c_int32(first_iter),
                                      C.c_int32(n_batches), C.c_int32(len(fan)), _p(fan), C.c_uint64(seed),
                                      _p(host_table), C.c_int64(host_table.shape[0]), C.c_int64(row_bytes),
                                      C.c_int64(max_nodes), C.c_int64(max_edges), C.c_int32(t), _p(feat),
                                      _p(scratch)))


def cpu_pipeline_native(indptr, indices, all_ids, all_labels, batch_size, first_iter, n_batches, fanout, seed,
                        host_table, threads=0):
    """Timed CPU baseline with a sampler written for a CPU (Floyd's algorithm, a reusable relabelling map
    per thread); another random stream than the GPU path, so it is timed, not compared.  Returns nodes gathered."""
    indptr, indices = _i64(indptr), _i32(indices)
    all_ids, all_labels = _i32(all_ids), _i32(all_labels)
    fan = _i32(fanout)
    host_table = np.ascontiguousarray(host_table)
    row_bytes = host_table.strides[0]
    t = threads if threads > 0 else num_threads()
    max_nodes, max_edges = batch_bounds(batch_size, list(fanout))
    slots = 1024
    while slots < 2 * max_nodes:
        slots *= 2
    feat = np.empty(t * max_nodes * row_bytes, dtype=np.uint8)
    scratch = np.empty(t * (max_nodes + 2 * max_edges + batch_size + 3 * slots), dtype=np.int32)
    return int(lib().orc_cpu_pipeline_native(_p(indptr), _p(indices), _p(all_ids), _p(all_labels),
                                             C.c_int32(len(all_ids)), C.c_int32(batch_size), C.c_int32(first_iter),
                                             C.c_int32(n_batches), C.c_int32(len(fan)), _p(fan), C.c_uint64(seed),
                                             _p(host_table), C.c_int64(host_table.shape[0]), C.c_int64(row_bytes),
                                             C.c_int64(max_nodes), C.c_int64(max_edges), C.c_int32(t), _p(feat),
                                             _p(scratch), C.c_int64(slots)))
