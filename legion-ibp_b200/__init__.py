"""Host-side mirror of the sampling server's operator / runner / IPC interface over the C ABI.

The classes keep the reference's names for this path (GraphStorage, FeatureStorage,
UnifiedCache, MemoryPool, IPCEnv, Runner; sampling_server/src/engine/server.h,
engine/operator_impl.cuh, cache/cache.cuh) and call ``liblegion_b200.so`` through ctypes.
There is no CPU fallback: importing works anywhere, but every call needs the CUDA library
and a GPU, and :func:`lib` raises when the library has not been built.

torch is used by callers for device memory and streams only; nothing here computes with it.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "liblegion_b200.so")

TRAINMODE, VALIDMODE, TESTMODE = 0, 1, 2
CACHEMISS_FLAG = -2
CODEC_RAW, CODEC_INT8, CODEC_E4M3 = 0, 1, 2
(BUF_IDS, BUF_FEATURES, BUF_LABELS, BUF_AGG_SRC, BUF_AGG_DST, BUF_NODE_COUNTER, BUF_EDGE_COUNTER,
 BUF_CACHE_INDEX, BUF_SRC_GLOBAL) = range(9)
INTRABATCH_CON = 3

_lib = None


class LegionError(RuntimeError):
    pass


def build(verbose=False):
    """Compile the CUDA library in-tree for sm_100a (nvcc cross-compiles without a GPU)."""
    import subprocess
    cmd = ["make", "-C", os.path.join(_HERE, "csrc"), "-j8"]
    if not verbose:
        cmd.append("-s")
    subprocess.check_call(cmd)
    return LIB_PATH


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise LegionError("liblegion_b200.so is missing: build it with `make -C legion-ibp_b200/csrc` "
                              "(there is no CPU fallback)")
        _lib = C.CDLL(LIB_PATH)
        _lib.legion_last_error.restype = C.c_char_p
    return _lib


def _check(rc):
    if rc != 0:
        raise LegionError("legion error %d: %s" % (rc, lib().legion_last_error().decode()))


def _ptr(t):
    """Device or host address of a torch tensor / numpy array / int."""
    if t is None:
        return C.c_void_p(0)
    if isinstance(t, int):
        return C.c_void_p(t)
    if hasattr(t, "data_ptr"):
        return C.c_void_p(t.data_ptr())
    return C.c_void_p(t.ctypes.data)


def _numel(t):
    return int(t.numel()) if hasattr(t, "numel") else int(t.size)


def _stream(s):
    if s is None:
        return C.c_void_p(0)
    if isinstance(s, int):
        return C.c_void_p(s)
    return C.c_void_p(s.cuda_stream)


class GraphStorage:
    """CSR topology readable from the device (GraphStorage, storage/graph_storage.cuh:7-24)."""

    def __init__(self, dev_id, indptr, indices):
        self._keep = (indptr, indices)
        self.n_nodes = _numel(indptr) - 1
        self.n_edges = _numel(indices)
        self.h = C.c_void_p()
        _check(lib().legion_graph_create(C.byref(self.h), C.c_int32(dev_id), C.c_int64(self.n_nodes),
                                         C.c_int64(self.n_edges), _ptr(indptr), _ptr(indices)))

    def close(self):
        if self.h:
            lib().legion_graph_destroy(self.h)
            self.h = C.c_void_p()


class FeatureStorage:
    """Feature table in pinned host memory and this GPU's seed lists (storage/feature_storage.cuh:6-34)."""

    def __init__(self, dev_id, n_nodes, row_bytes, host_table=None):
        self._keep = [host_table]
        self.n_nodes, self.row_bytes = int(n_nodes), int(row_bytes)
        self.h = C.c_void_p()
        _check(lib().legion_features_create(C.byref(self.h), C.c_int32(dev_id), C.c_int64(n_nodes),
                                            C.c_int32(row_bytes), _ptr(host_table)))

    def set_split(self, mode, ids_dev, labels_dev):
        self._keep += [ids_dev, labels_dev]
        _check(lib().legion_features_set_split(self.h, C.c_int32(mode), _ptr(ids_dev), _ptr(labels_dev),
                                               C.c_int32(_numel(ids_dev))))

    def close(self):
        if self.h:
            lib().legion_features_destroy(self.h)
            self.h = C.c_void_p()


class UnifiedCache:
    """Static (clique-striped, optionally compressed) or LRU feature cache (cache/cache.cuh:66-188)."""

    def __init__(self, dev_id, n_nodes, row_bytes, capacity, kg=1, ki=0, codec=CODEC_RAW, lru=None):
        self.dev_id, self.n_nodes, self.row_bytes = dev_id, int(n_nodes), int(row_bytes)
        self.kg, self.ki, self.capacity, self.codec = kg, ki, int(capacity), codec
        self._keep = []
        self.h = C.c_void_p()
        self.lru = lru
        if lru is None:
            _check(lib().legion_cache_create(C.byref(self.h), C.c_int32(dev_id), C.c_int64(n_nodes),
                                             C.c_int32(row_bytes), C.c_int32(kg), C.c_int32(ki),
                                             C.c_int32(capacity), C.c_int32(codec)))
        else:
            sets, ways = lru
            _check(lib().legion_cache_create_lru(C.byref(self.h), C.c_int32(dev_id), C.c_int64(n_nodes),
                                                 C.c_int32(row_bytes), C.c_int64(sets), C.c_int32(ways)))

    @staticmethod
    def degree_order(dev_id, indptr, order_out, stream=None):
        _check(lib().legion_cache_degree_order(C.c_int32(dev_id), _ptr(indptr), C.c_int64(indptr.numel() - 1),
                                               _ptr(order_out), _stream(stream)))

    @staticmethod
    def hotness_order(dev_id, counts_dev, order_out, stream=None):
        _check(lib().legion_cache_hotness_order(C.c_int32(dev_id), _ptr(counts_dev), C.c_int64(_numel(counts_dev)),
                                                _ptr(order_out), _stream(stream)))

    @staticmethod
    def pack_order(dev_id, order_dev, n_cached, row_of_out, stream=None):
        """row_of[id] of a host table in packed order (Dataset.pack_features): rank t -> t - n_cached, cached ranks last."""
        _check(lib().legion_cache_pack_order(C.c_int32(dev_id), _ptr(order_dev), C.c_int64(_numel(order_dev)),
                                             C.c_int64(n_cached), _ptr(row_of_out), _stream(stream)))

    @staticmethod
    def plan(dev_id, order_dev, n_nodes, budget_rows, world, indptr=None, counts=None, cost=None, stream=None):
        """(stripe_rows, replica_rows) of a per-GPU row budget; weights from degrees or presampled counts."""
        a, b = C.c_int64(), C.c_int64()
        cost_arr = (C.c_double * 3)(*cost) if cost is not None else None
        _check(lib().legion_cache_plan(C.c_int32(dev_id), _ptr(order_dev), _ptr(indptr), _ptr(counts), C.c_int64(n_nodes),
                                       C.c_int64(budget_rows), C.c_int32(world), cost_arr, C.byref(a), C.byref(b),
                                       _stream(stream)))
        return a.value, b.value

    def fill_static(self, order_dev, host_table, stream=None, row_of_id=None):
        """row_of_id (device int32 per node): row of host_table that holds each node, for tables that are
        not in id order."""
        self._keep += [host_table]
        _check(lib().legion_cache_fill_static_rows(self.h, _ptr(order_dev), C.c_int64(order_dev.numel()),
                                                   _ptr(host_table), _ptr(row_of_id), _stream(stream)))

    def place_static(self, order_dev, stream=None):
        """Lookup table only; the caller writes row s of partition() with the row of node order[s * kg + ki]."""
        _check(lib().legion_cache_place_static(self.h, _ptr(order_dev), C.c_int64(order_dev.numel()), _stream(stream)))

    def write_partition_rows(self, first_row, rows_dev):
        """Copies a device tensor of whole rows into this GPU's partition starting at row first_row."""
        ptr, nbytes = self.partition()
        n = rows_dev.numel() * rows_dev.element_size()
        off = int(first_row) * self.row_bytes
        if off < 0 or off + n > nbytes:
            raise LegionError("write_partition_rows: rows [%d, +%d bytes) are outside the partition" % (first_row, n))
        _check(lib().legion_copy(C.c_void_p(ptr + off), _ptr(rows_dev), C.c_int64(n), C.c_int32(3)))

    def set_host_codec(self, codec):
        """The host table holds compressed rows (codes + fp32 scale) of this cache's codec."""
        _check(lib().legion_cache_set_host_codec(self.h, C.c_int32(codec)))

    def add_replicas(self, order_dev, n_rows, stream=None, row_of_id=None):
        """Private copies of the n_rows hottest rows that the striping placed on peers."""
        _check(lib().legion_cache_add_replicas(self.h, _ptr(order_dev), C.c_int64(order_dev.numel()), C.c_int64(n_rows),
                                               _ptr(row_of_id), _stream(stream)))

    def set_host_table(self, host_table):
        self._keep += [host_table]
        _check(lib().legion_cache_set_host_table(self.h, _ptr(host_table)))

    def partition(self):
        p, b = C.c_void_p(), C.c_int64()
        _check(lib().legion_cache_partition(self.h, C.byref(p), C.byref(b)))
        return p.value or 0, b.value

    def export_partition(self):
        """(fd, bytes) of this GPU's partition as shareable memory; the caller closes the fd."""
        fd, b = C.c_int32(-1), C.c_int64()
        _check(lib().legion_cache_export_partition(self.h, C.byref(fd), C.byref(b)))
        return fd.value, b.value

    def import_peer(self, k, fd, nbytes):
        _check(lib().legion_cache_import_peer(self.h, C.c_int32(k), C.c_int32(fd), C.c_int64(nbytes)))

    def set_peer(self, k, ptr):
        _check(lib().legion_cache_set_peer(self.h, C.c_int32(k), C.c_void_p(ptr)))

    def lut_ptr(self):
        p = C.c_void_p()
        _check(lib().legion_cache_lut(self.h, C.byref(p)))
        return p.value

    def lru_state(self):
        k, s, r = C.c_void_p(), C.c_void_p(), C.c_void_p()
        _check(lib().legion_cache_lru_state(self.h, C.byref(k), C.byref(s), C.byref(r)))
        return k.value, s.value, r.value

    def lru_clock(self):
        c = C.c_int32()
        _check(lib().legion_cache_lru_clock(self.h, C.byref(c)))
        return c.value

    def stats(self, stream=None):
        a = (C.c_int64 * 4)()
        _check(lib().legion_cache_stats(self.h, a, _stream(stream)))
        return dict(local_hits=a[0], peer_hits=a[1], misses=a[2], lru_inserts=a[3])

    def close(self):
        if self.h:
            lib().legion_cache_destroy(self.h)
            self.h = C.c_void_p()


def host_register(dev_id, tensor):
    """Page-locks a host tensor that CUDA did not allocate (shared segment, mapped file) for zero-copy reads."""
    _check(lib().legion_host_register(C.c_int32(dev_id), _ptr(tensor), C.c_int64(tensor.numel() * tensor.element_size())))


def quantize_table(dev_id, codec, rows, n_rows, feature_len, out_rows, stream=None):
    """fp32 rows -> compressed rows [(feature_len + 4) rounded up to 16 bytes] with the caches' quantiser."""
    _check(lib().legion_quantize_table(C.c_int32(dev_id), C.c_int32(codec), _ptr(rows), C.c_int64(n_rows),
                                       C.c_int32(feature_len), _ptr(out_rows), _stream(stream)))


class MemoryPool:
    """Scratch and double-buffered outputs of one GPU (engine/memorypool.cuh:20-221)."""

    def __init__(self, dev_id, batch_size, fanout, row_bytes_out, pipes=2, slots=None):
        """slots < pipes: batches are sampled ahead of the hand-off into private buffers (legion_pool_create_ahead)."""
        self.dev_id, self.batch_size, self.fanout = dev_id, int(batch_size), list(fanout)
        self.row_bytes_out, self.pipes = int(row_bytes_out), pipes
        self.slots = pipes if slots is None else slots
        fan = (C.c_int32 * max(1, len(fanout)))(*fanout)
        self.h = C.c_void_p()
        _check(lib().legion_pool_create_ahead(C.byref(self.h), C.c_int32(dev_id), C.c_int32(batch_size),
                                              C.c_int32(len(fanout)), fan, C.c_int32(row_bytes_out),
                                              C.c_int32(self.slots), C.c_int32(pipes)))
        mn, me = C.c_int64(), C.c_int64()
        _check(lib().legion_pool_limits(self.h, C.byref(mn), C.byref(me)))
        self.max_nodes, self.max_edges = mn.value, me.value

    def buffer(self, which, pipe=0):
        p, b = C.c_void_p(), C.c_int64()
        _check(lib().legion_pool_buffer(self.h, C.c_int32(which), C.c_int32(pipe), C.byref(p), C.byref(b)))
        return p.value, b.value

    def set_batch(self, it, mode=TRAINMODE, pipe=0, global_batch=0):
        _check(lib().legion_pool_set_batch(self.h, C.c_int32(it), C.c_int32(mode), C.c_int32(pipe),
                                           C.c_uint32(global_batch)))

    def set_rng(self, seed, max_rounds=64):
        _check(lib().legion_pool_set_rng(self.h, C.c_uint64(seed), C.c_int32(max_rounds)))

    def device_error(self, stream=None, reset=True):
        e = C.c_int32()
        _check(lib().legion_pool_device_error(self.h, _stream(stream), C.byref(e), C.c_int32(1 if reset else 0)))
        return e.value

    def read(self, which, pipe, count, dtype):
        """Copy `count` elements of an output buffer to a numpy array (tests and checks)."""
        import numpy as np
        import torch
        p, b = self.buffer(which, pipe)
        out = np.empty(count, dtype=dtype)
        nbytes = out.nbytes
        assert nbytes <= b, (nbytes, b)
        if nbytes:
            torch.cuda.synchronize()
            _check(lib().legion_copy(C.c_void_p(out.ctypes.data), C.c_void_p(p), C.c_int64(nbytes), C.c_int32(2)))
        return out

    def close(self):
        if self.h:
            lib().legion_pool_destroy(self.h)
            self.h = C.c_void_p()


# ---- the five operators, argument for argument (engine/operator_impl.cuh:11-69) ------------------

def BatchGenerate(stream, feature, cache, memorypool, batch_size, counter, part_id, dev_id, mode, is_presc,
                  hop_num, dyn_cache=0):
    _check(lib().legion_batch_generate(_stream(stream), feature.h, cache.h if cache else None, memorypool.h,
                                       C.c_int32(batch_size), C.c_int32(counter), C.c_int32(part_id),
                                       C.c_int32(dev_id), C.c_int32(mode), C.c_int32(int(is_presc)),
                                       C.c_int32(hop_num), C.c_int32(dyn_cache)))


def RandomSample(stream, graph, cache, memorypool, count, dev_id, op_id, is_presc=False, dyn_cache=0):
    _check(lib().legion_random_sample(_stream(stream), graph.h, cache.h if cache else None, memorypool.h,
                                      C.c_int32(count), C.c_int32(dev_id), C.c_int32(op_id),
                                      C.c_int32(int(is_presc)), C.c_int32(dyn_cache)))


def FeatureCacheLookup(stream, cache, memorypool, op_id, dev_id, dyn_cache=0):
    _check(lib().legion_feature_cache_lookup(_stream(stream), cache.h if cache else None, memorypool.h,
                                             C.c_int32(op_id), C.c_int32(dev_id), C.c_int32(dyn_cache)))


def IOSubmit(stream, feature, memorypool, op_id, dev_id):
    _check(lib().legion_io_submit(_stream(stream), feature.h, memorypool.h, C.c_int32(op_id), C.c_int32(dev_id)))


def IOComplete(stream, cache, memorypool, dev_id, mode):
    _check(lib().legion_io_complete(_stream(stream), cache.h if cache else None, memorypool.h, C.c_int32(dev_id),
                                    C.c_int32(mode)))


def run_batch(stream, graph, feature, cache, pool, dev_id):
    _check(lib().legion_run_batch(_stream(stream), graph.h, feature.h, cache.h if cache else None, pool.h,
                                  C.c_int32(dev_id)))


def run_batch_host(graph, feature, cache, pool, dev_id, seeds, labels, ids_out, labels_out, agg_src_out,
                   agg_dst_out, nc_out, ec_out, features_out=None):
    """Host-buffer call: numpy int32 arrays in and out; returns (n_nodes, n_edges)."""
    _check(lib().legion_run_batch_host(graph.h, feature.h if feature else None, cache.h if cache else None, pool.h,
                                       C.c_int32(dev_id), _ptr(seeds), _ptr(labels), C.c_int32(len(seeds)),
                                       _ptr(ids_out), _ptr(labels_out), _ptr(agg_src_out), _ptr(agg_dst_out),
                                       _ptr(nc_out), _ptr(ec_out), _ptr(features_out)))
    hops = int(nc_out[INTRABATCH_CON * 3 - 1])
    return int(nc_out[INTRABATCH_CON * 3 + hops]), int(ec_out[0] + ec_out[1])


NOALLOC_MAX_ROWS = 1 << 18


def gather_rows_noalloc(stream, dev_id, ids_dev, lut_ptr, capacity, kg, ki, partition_ptrs, host_table, n_nodes,
                        row_bytes, out_dev):
    """Lookup + gather of one id list through the entry point that allocates nothing (its scratch is a
    fixed array inside the library).  For callers that must not allocate device memory when they call in;
    at most NOALLOC_MAX_ROWS ids per call, calls on one GPU must not overlap.  Makes dev_id the current device."""
    if lut_ptr and len(partition_ptrs) < kg:
        raise LegionError("gather_rows_noalloc: %d partition pointers for a clique of %d" % (len(partition_ptrs), kg))
    parts = (C.c_void_p * max(1, len(partition_ptrs)))(*partition_ptrs)
    _check(lib().legion_gather_rows_noalloc(_stream(stream), C.c_int32(dev_id), _ptr(ids_dev),
                                            C.c_int64(ids_dev.numel()), C.c_void_p(lut_ptr), C.c_int32(capacity),
                                            C.c_int32(kg), C.c_int32(ki), parts, _ptr(host_table), C.c_int64(n_nodes),
                                            C.c_int32(row_bytes), _ptr(out_dev)))


class IPCEnv:
    """Shared segment + semaphores of the server <-> trainer hand-off (engine/ipc_service.h:6-35)."""

    def __init__(self, device_count, shm_name=None):
        self.h = C.c_void_p()
        name = shm_name.encode() if shm_name else None
        _check(lib().legion_ipc_create(C.byref(self.h), C.c_int32(device_count), name))

    def publish_counters(self, dev_id, pipe, node_counter, edge_counter):
        """Counter words of a finished batch into the companion host segment (the runner does this itself)."""
        nc = (C.c_int32 * 16)(*[int(v) for v in node_counter])
        ec = (C.c_int32 * 16)(*[int(v) for v in edge_counter])
        _check(lib().legion_ipc_publish_counters(self.h, C.c_int32(dev_id), C.c_int32(pipe), nc, ec))

    def Coordinate(self, train_num, valid_num, test_num, raw_batch_size, epochs):
        n = len(train_num)
        arr = lambda v: (C.c_int32 * n)(*v)
        _check(lib().legion_ipc_coordinate(self.h, arr(train_num), arr(valid_num), arr(test_num), C.c_int32(n),
                                           C.c_int32(raw_batch_size), C.c_int32(epochs)))

    def steps(self):
        a = (C.c_int32 * 3)()
        _check(lib().legion_ipc_steps(self.h, a))
        return list(a)

    def GetMaxStep(self):
        return lib().legion_ipc_max_step(self.h)

    def GetCurrentMode(self, global_batch_id):
        return lib().legion_ipc_current_mode(self.h, C.c_int32(global_batch_id))

    def GetLocalBatchId(self, global_batch_id):
        return lib().legion_ipc_local_batch_id(self.h, C.c_int32(global_batch_id))

    def GetCurrentBatchsize(self, dev_id, mode):
        return lib().legion_ipc_current_batchsize(self.h, C.c_int32(dev_id), C.c_int32(mode))

    def publish_pool(self, pool, dev_id):
        _check(lib().legion_ipc_publish_pool(self.h, pool.h, C.c_int32(dev_id)))

    def open_semaphores(self, dev_id, pipes=2):
        _check(lib().legion_ipc_open_semaphores(self.h, C.c_int32(dev_id), C.c_int32(pipes)))

    def IPCWait(self, dev_id, pipe, timeout_ms=-1):
        _check(lib().legion_ipc_wait(self.h, C.c_int32(dev_id), C.c_int32(pipe), C.c_int32(timeout_ms)))

    def IPCPost(self, dev_id, pipe):
        _check(lib().legion_ipc_post(self.h, C.c_int32(dev_id), C.c_int32(pipe)))

    def Finalize(self):
        if self.h:
            lib().legion_ipc_destroy(self.h)
            self.h = C.c_void_p()


def ipc_layout():
    a, b, c = C.c_int64(), C.c_int64(), C.c_int64()
    _check(lib().legion_ipc_layout(C.byref(a), C.byref(b), C.byref(c)))
    return dict(segment_bytes=a.value, handle_bytes=b.value, handles_offset=c.value)


class Runner:
    """GPURunner (engine/server.cu:176-416): runs batches, rotates pipes, hands them off."""

    def __init__(self, dev_id, graph, feature, cache, pool, env=None):
        self.dev_id = dev_id
        self._keep = (graph, feature, cache, pool, env)
        self.h = C.c_void_p()
        _check(lib().legion_runner_create(C.byref(self.h), C.c_int32(dev_id), graph.h, feature.h,
                                          cache.h if cache else None, pool.h, env.h if env else None))

    def RunOnce(self, global_batch_id, mode=TRAINMODE, local_batch_id=None, timeout_ms=-1):
        lb = global_batch_id if local_batch_id is None else local_batch_id
        _check(lib().legion_runner_run_once(self.h, C.c_int32(global_batch_id), C.c_int32(mode), C.c_int32(lb),
                                            C.c_int32(timeout_ms)))

    def enqueue(self, global_batch_id, mode=TRAINMODE, local_batch_id=None):
        lb = global_batch_id if local_batch_id is None else local_batch_id
        _check(lib().legion_runner_enqueue(self.h, C.c_int32(global_batch_id), C.c_int32(mode), C.c_int32(lb)))

    def sync(self):
        _check(lib().legion_runner_sync(self.h))

    def submit_host(self, seeds, labels, global_batch_id):
        """Start one batch from host seed / label arrays (numpy int32)."""
        _check(lib().legion_runner_submit_host(self.h, _ptr(seeds), _ptr(labels), C.c_int32(len(seeds)),
                                               C.c_int32(global_batch_id)))

    def submit_host_to(self, seeds, labels, global_batch_id, ids_out, labels_out, agg_src_out, agg_dst_out):
        """submit_host with the (page-locked) output arrays named up front: the batch writes ids, labels and
        edge lists into them itself; the matching collect_host(None, None, None, None, nc, ec) only waits."""
        _check(lib().legion_runner_submit_host_to(self.h, _ptr(seeds), _ptr(labels), C.c_int32(len(seeds)),
                                                  C.c_int32(global_batch_id), _ptr(ids_out), _ptr(labels_out),
                                                  _ptr(agg_src_out), _ptr(agg_dst_out)))

    def collect_host(self, ids_out, labels_out, agg_src_out, agg_dst_out, nc_out, ec_out, features_out=None):
        """Wait for the oldest submitted batch and copy it out; returns (n_nodes, n_edges)."""
        _check(lib().legion_runner_collect_host(self.h, _ptr(ids_out), _ptr(labels_out), _ptr(agg_src_out),
                                                _ptr(agg_dst_out), _ptr(nc_out), _ptr(ec_out), _ptr(features_out)))
        hops = int(nc_out[INTRABATCH_CON * 3 - 1])
        return int(nc_out[INTRABATCH_CON * 3 + hops]), int(ec_out[0] + ec_out[1])

    def serve(self, first_global_batch, count, timeout_ms=-1):
        _check(lib().legion_runner_serve(self.h, C.c_int32(first_global_batch), C.c_int32(count),
                                         C.c_int32(timeout_ms)))

    def presample(self, first_batch, count, counts_dev):
        """RunPreSc: sample only, count node accesses into counts_dev (uint32 per node)."""
        _check(lib().legion_runner_presample(self.h, C.c_int32(first_batch), C.c_int32(count), _ptr(counts_dev)))

    def stage_seeds(self, mode=TRAINMODE):
        """Rows of the uncached nodes of a mode's seed list into page-locked memory, in list order: the copy
        engine then brings each batch's block in while the batch samples.  Returns the rows staged."""
        n = C.c_int64()
        _check(lib().legion_runner_stage_seeds(self.h, C.c_int32(mode), C.byref(n)))
        return n.value

    def register_host_seeds(self, seeds):
        """The same for a seed list in host memory (numpy int32): submit_host[_to] calls that pass a slice
        of this very array are staged.  The array must stay alive and unchanged."""
        self._keep = self._keep + (seeds,)
        n = C.c_int64()
        _check(lib().legion_runner_register_host_seeds(self.h, _ptr(seeds), C.c_int32(len(seeds)), C.byref(n)))
        return n.value

    def staged_rows(self):
        n = C.c_int64()
        _check(lib().legion_runner_staged_rows(self.h, C.byref(n)))
        return n.value

    def set_edge_counts(self, on):
        """The host-buffer calls deliver per-destination edge counts (bytes) in the place of agg_dst."""
        _check(lib().legion_runner_set_edge_counts(self.h, C.c_int32(1 if on else 0)))

    def host_times(self):
        """Host microseconds inside submit / collect since the last call: dict(submit, collect, collect_wait, batches)."""
        a = (C.c_double * 4)()
        _check(lib().legion_runner_host_times(self.h, a))
        return dict(submit_us=a[0], collect_us=a[1], collect_wait_us=a[2], batches=a[3])

    def current_pipe(self):
        return lib().legion_runner_current_pipe(self.h)

    def timing(self):
        a, b, m, n, t = C.c_float(), C.c_float(), C.c_float(), C.c_int32(), C.c_int32()
        _check(lib().legion_runner_timing(self.h, C.byref(a), C.byref(b), C.byref(m), C.byref(n), C.byref(t)))
        return dict(batch_ms=a.value, gather_ms=b.value, miss_ms=m.value, batches=n.value, timed=t.value)

    def trace(self, max_batches=4096):
        """[[samp_begin, samp_end, gather_begin, gather_end, miss_begin, miss_end], ...] of the last timed window (ms)."""
        buf = (C.c_float * (6 * max_batches))()
        n = lib().legion_runner_trace(self.h, buf, C.c_int32(max_batches))
        if n < 0:
            raise LegionError("legion_runner_trace failed")
        return [list(buf[6 * i:6 * i + 6]) for i in range(n)]

    def set_options(self, use_graph=True, time_kernels=False):
        _check(lib().legion_runner_set_options(self.h, C.c_int32(int(use_graph)), C.c_int32(int(time_kernels))))

    def Finalize(self):
        if self.h:
            lib().legion_runner_destroy(self.h)
            self.h = C.c_void_p()


class MetaConfig(C.Structure):
    """The line of ./meta_config (legion_server.py:45-46, storage/storage_management.cu:33-68)."""
    _fields_ = [("dataset_path", C.c_char * 512), ("feature_path", C.c_char * 512), ("raw_batch_size", C.c_int32),
                ("node_num", C.c_int64), ("edge_num", C.c_int64), ("float_feature_len", C.c_int32),
                ("training_set_num", C.c_int32), ("validation_set_num", C.c_int32), ("testing_set_num", C.c_int32),
                ("cache_memory", C.c_int64), ("epoch", C.c_int32)]

    @staticmethod
    def read(path="./meta_config"):
        m = MetaConfig()
        _check(lib().legion_meta_config_read(path.encode(), C.byref(m)))
        return m

    def write(self, path="./meta_config"):
        _check(lib().legion_meta_config_write(path.encode(), C.byref(self)))


class Dataset:
    """A Legion-format dataset in host memory (StorageManagement::LoadGraph / LoadFeature,
    storage/storage_management.cu:106-279).  Arrays are numpy views of the loader's memory."""

    def __init__(self, meta, pin=True, load_features=True):
        import numpy as np
        self.meta = meta
        self.h = C.c_void_p()
        _check(lib().legion_dataset_load(C.byref(self.h), C.byref(meta), C.c_int32(int(pin)),
                                         C.c_int32(int(load_features))))
        ip, ix, ft, lb = C.c_void_p(), C.c_void_p(), C.c_void_p(), C.c_void_p()
        _check(lib().legion_dataset_arrays(self.h, C.byref(ip), C.byref(ix), C.byref(ft), C.byref(lb)))
        n, e, f = meta.node_num, meta.edge_num, meta.float_feature_len

        def view(ptr, count, ctype, dtype):
            if not ptr.value or count == 0:
                return np.empty(0, dtype)
            return np.ctypeslib.as_array(C.cast(ptr, C.POINTER(ctype)), shape=(count,)).view(dtype)

        self.indptr = view(ip, n + 1, C.c_int64, np.int64)
        self.indices = view(ix, e, C.c_int32, np.int32)
        self.features = view(ft, n * f, C.c_float, np.float32).reshape(-1, f) if load_features else None
        self.labels = view(lb, n, C.c_int32, np.int32)
        self.features_ptr = ft.value

    def pack_features(self, dev_id, order_dev, n_cached):
        """Rewrites the loaded table in packed order: rows of the nodes of rank >= n_cached by rising rank, then
        the rows of the cached nodes.  The features view and pointer are those of the new table afterwards."""
        import numpy as np
        _check(lib().legion_dataset_pack_features(self.h, C.c_int32(dev_id), _ptr(order_dev), C.c_int64(n_cached)))
        ft = C.c_void_p()
        _check(lib().legion_dataset_arrays(self.h, None, None, C.byref(ft), None))
        n, f = self.meta.node_num, self.meta.float_feature_len
        self.features = np.ctypeslib.as_array(C.cast(ft, C.POINTER(C.c_float)), shape=(n * f,)).view(np.float32).reshape(-1, f)
        self.features_ptr = ft.value

    def split(self, mode, partition_count, part_id):
        """(ids, labels) of one GPU: partition file or id % partition_count (storage_management.cu:214-250)."""
        import numpy as np
        cnt = C.c_int32()
        _check(lib().legion_dataset_split(self.h, C.c_int32(mode), C.c_int32(partition_count), C.c_int32(part_id),
                                          None, None, C.byref(cnt)))
        ids = np.empty(cnt.value, np.int32)
        lab = np.empty(cnt.value, np.int32)
        _check(lib().legion_dataset_split(self.h, C.c_int32(mode), C.c_int32(partition_count), C.c_int32(part_id),
                                          _ptr(ids), _ptr(lab), C.byref(cnt)))
        return ids, lab

    def close(self):
        if self.h:
            self.indptr = self.indices = self.features = self.labels = None
            lib().legion_dataset_destroy(self.h)
            self.h = C.c_void_p()


class BatchView(C.Structure):
    _fields_ = [("hop_num", C.c_int32), ("n_ids", C.c_int32), ("n_labels", C.c_int32), ("ids", C.c_void_p),
                ("features", C.c_void_p), ("labels", C.c_void_p), ("agg_src", C.c_void_p * 3),
                ("agg_dst", C.c_void_p * 3), ("n_edges", C.c_int32 * 3), ("block_src", C.c_int32 * 3),
                ("block_dst", C.c_int32 * 3), ("node_counter", C.c_int32 * 16), ("edge_counter", C.c_int32 * 16)]


class ipc_service:
    """Trainer side of the hand-off with the function names of the trainers' torch extension
    (training_backend/ipc_service.cpp:93-100): initialize, get_next, get_block_size, get_steps,
    synchronize, finalize.  get_next returns device pointers and counts instead of torch tensors."""

    def __init__(self, dev_id, shm_name=None):
        self.h = C.c_void_p()
        self.view = BatchView()
        name = shm_name.encode() if shm_name else None
        _check(lib().legion_client_open(C.byref(self.h), C.c_int32(dev_id), name))

    initialize = __init__

    def get_steps(self):
        a = (C.c_int32 * 3)()
        _check(lib().legion_client_steps(self.h, a))
        return list(a)

    def get_next(self, timeout_ms=-1):
        _check(lib().legion_client_get_next(self.h, C.c_int32(timeout_ms), C.byref(self.view)))
        return self.view

    def get_block_size(self):
        v = self.view
        out = []
        for j in range(v.hop_num):
            out += [v.block_src[j], v.block_dst[j]]
        return out

    def counters_on_host(self):
        """True when get_next reads the counters from the server's host segment (no device copy)."""
        return bool(lib().legion_client_counters_on_host(self.h))

    def synchronize(self):
        _check(lib().legion_client_synchronize(self.h))

    def finalize(self):
        if self.h:
            lib().legion_client_close(self.h)
            self.h = C.c_void_p()


def agg_dst_from_counts(counts, node_counter):
    """agg_dst of a batch from its per-destination edge counts (Runner.set_edge_counts): within hop h the
    destinations run 0 .. node_counter[9 + h] - 1, each repeated count times."""
    import numpy as np
    hops = int(node_counter[INTRABATCH_CON * 3 - 1])
    out, pos = [], 0
    for h in range(hops):
        n = int(node_counter[INTRABATCH_CON * 3 + h])
        out.append(np.repeat(np.arange(n, dtype=np.int32), counts[pos:pos + n]))
        pos += n
    return np.concatenate(out) if out else np.zeros(0, np.int32)
