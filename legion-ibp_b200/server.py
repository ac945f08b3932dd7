"""One rank of the sampling server: the Server interface of the reference
(sampling_server/src/engine/server.h:5-21: Initialize / PreSc / Run / Finalize) for one process per GPU.

The reference runs one host thread per GPU inside one process (engine/server.cu:46-170) and shares
raw pointers between the threads; here every GPU has its own process, so the two things the threads
shared travel through ``torch.distributed`` once at start-up:
  * the per-GPU seed counts that the step arithmetic needs (IPCEnv::Coordinate), and
  * the cache partitions, exported as file descriptors of shareable device memory and mapped by
    every peer, from which each rank builds the pointer table that its gather kernel reads peers
    through (plain loads over NVLink; no collective on the data path).
"""
import ctypes as C

import torch

from . import (CODEC_RAW, TRAINMODE, VALIDMODE, TESTMODE, FeatureStorage, GraphStorage, IPCEnv, LegionError,
               MemoryPool, Runner, UnifiedCache, lib)


def split_seeds(ids, world, rank):
    """Seeds of one GPU: ``id % ngpu`` (storage/storage_management.cu:214-250, no partition file)."""
    return ids[(ids % world) == rank].contiguous()


def plan_cache_rows(n_nodes, per_gpu_rows, world):
    """Rows each clique member holds: the requested budget, capped so that the clique never holds
    more rows than the table has (rank t lives on GPU t % world at row t // world)."""
    per_gpu_rows = max(0, min(int(per_gpu_rows), int(n_nodes)))
    if per_gpu_rows * world >= n_nodes:
        per_gpu_rows = (n_nodes + world - 1) // world
    return per_gpu_rows


# Relative cost of serving one row from this GPU's memory, from a peer over NVLink and from the host
# table over the host link (measured on B200: ~4 TB/s, ~640 GB/s and ~43 GB/s of random 512-byte rows).
ROW_COST = (0.16, 1.0, 15.0)


def plan_clique_cache(mass, n_nodes, budget_rows, world, cost=ROW_COST, steps=64):
    """Splits one GPU's row budget into its stripe of the clique's cache and private copies of hot rows
    held by peers.  `mass(x)` is the fraction of all row accesses that go to the x hottest nodes (any
    monotone estimate; `degree_mass` below).  Returns (stripe_rows, replica_rows).

    With R replica rows and S = budget - R stripe rows per GPU the clique holds C = min(n, S * world)
    nodes; the T = R * world / (world - 1) hottest of them are local on every GPU (own stripe or
    replica), the others are local with probability 1 / world.  The plan minimises
    host * (1 - mass(C)) + peer * (mass(C) - mass(T)) * (world - 1) / world + local * (the rest).
    The reference stripes only (cache/cache_impl.cuh:104-109), which is the R = 0 plan."""
    budget_rows = max(0, min(int(budget_rows), int(n_nodes)))
    full = (n_nodes + world - 1) // world
    if world == 1 or budget_rows == 0:
        return min(budget_rows, n_nodes), 0
    c_local, c_peer, c_host = cost
    best = None
    for i in range(steps + 1):
        r = budget_rows // 2 * i // steps
        stripe = min(budget_rows - r, full)
        r = min(r, stripe)
        covered = min(n_nodes, stripe * world)
        local_top = min(covered, r * world // (world - 1))
        m_c, m_t = mass(covered), mass(local_top)
        t = (c_host * (1.0 - m_c) + c_peer * (m_c - m_t) * (world - 1) / world +
             c_local * (m_t + (m_c - m_t) / world))
        if best is None or t < best[0] - 1e-12:
            best = (t, stripe, r)
    # memory left over once the stripes cover the table goes to replicas
    _, stripe, r = best
    if stripe == full:
        r = max(r, min(budget_rows - stripe, stripe))
    return stripe, r


def weight_mass(weights, order):
    """mass(x) for plan_clique_cache: share of the total weight held by the x first nodes of `order`
    (weights: one non-negative number per node, e.g. presampled access counts)."""
    w = weights[order.long()].to(torch.float64)
    cum = torch.cumsum(w, 0)
    total = float(cum[-1].item()) if cum.numel() else 0.0
    n = int(cum.numel())

    def mass(x):
        x = int(min(max(x, 0), n))
        if x == 0 or total <= 0.0:
            return 0.0
        return float(cum[x - 1].item()) / total
    return mass


def degree_mass(indptr, order):
    """mass(x) from node degrees: a node is sampled as a neighbour in proportion to its degree, and
    neighbours are ~96% of the rows of a [25, 10] batch."""
    return weight_mass(indptr[1:] - indptr[:-1], order)


def all_gather_ints(values, dist, device="cpu"):
    """[[values of rank 0], [values of rank 1], ...]; works with gloo (cpu) and nccl (cuda)."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return [list(values)]
    t = torch.tensor(list(values), dtype=torch.int64, device=device)
    out = [torch.empty_like(t) for _ in range(dist.get_world_size())]
    dist.all_gather(out, t)
    return [[int(v) for v in o.cpu().tolist()] for o in out]


def all_gather_bytes(blob, dist, device="cpu"):
    """Every rank's fixed-size byte string, in rank order."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return [bytes(blob)]
    t = torch.tensor(list(blob), dtype=torch.uint8, device=device)
    out = [torch.empty_like(t) for _ in range(dist.get_world_size())]
    dist.all_gather(out, t)
    return [bytes(o.cpu().tolist()) for o in out]


def exchange_partitions(cache, rank, world, dist, device="cuda", tag=None):
    """Builds the clique's pointer table (d_float_feature_cache_ptr_ of cache/cache.cu:601-622) across
    processes: every rank exports its partition as a file descriptor, hands it to every peer over a
    unix socket (SCM_RIGHTS) and maps the descriptors it receives.  Peers are then read by plain loads
    over NVLink.  Falls back to legacy CUDA IPC handles when the partition is not shareable memory."""
    import os
    import socket
    import struct
    try:
        fd, nbytes = cache.export_partition()
    except LegionError:
        return _exchange_partitions_ipc(cache, rank, world, dist, device)
    tag = tag or "%s_%d" % (os.environ.get("MASTER_PORT", "0"), os.getuid())
    name = "\0legion_b200_%s_%d"
    srv = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    srv.bind(name % (tag, rank))
    srv.listen(world)
    dist.barrier()
    for k in range(world):
        if k == rank:
            continue
        s = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        s.connect(name % (tag, k))
        socket.send_fds(s, [struct.pack("iq", rank, nbytes)], [fd])
        s.close()
    for _ in range(world - 1):
        conn, _addr = srv.accept()
        msg, fds, _flags, _a = socket.recv_fds(conn, 64, 1)
        peer, peer_bytes = struct.unpack("iq", msg[:struct.calcsize("iq")])
        cache.import_peer(peer, fds[0], peer_bytes)
        os.close(fds[0])
        conn.close()
    os.close(fd)
    srv.close()
    dist.barrier()
    return "vmm"


def _exchange_partitions_ipc(cache, rank, world, dist, device="cuda"):
    ptr, _ = cache.partition()
    handle = (C.c_char * 64)()
    if ptr:
        rc = lib().legion_ipc_get_handle(C.c_void_p(ptr), handle)
        if rc != 0:
            raise LegionError(lib().legion_last_error().decode())
    blobs = all_gather_bytes(handle.raw, dist, device)
    for k in range(world):
        if k == rank or not ptr:
            continue
        p = C.c_void_p()
        rc = lib().legion_ipc_open_handle(blobs[k], C.byref(p))
        if rc != 0:
            raise LegionError(lib().legion_last_error().decode())
        cache.set_peer(k, p.value)
    return "ipc"


class Server:
    """Builds and runs one rank.  Arguments mirror what GPUServer::Initialize pulls out of
    ``meta_config`` and argv (engine/server.cu:48-92, storage/storage_management.cu:33-68)."""

    def __init__(self, dist=None):
        self.dist = dist
        self.rank = dist.get_rank() if dist is not None and dist.is_initialized() else 0
        self.world = dist.get_world_size() if dist is not None and dist.is_initialized() else 1
        self.runner = None

    def Initialize(self, dev_id, indptr, indices, host_table, row_bytes, train_ids, labels, batch_size, fanout,
                   cache_rows_per_gpu, valid_ids=None, test_ids=None, epochs=1, codec=CODEC_RAW, use_ipc=False,
                   shm_name=None, rng_seed=0):
        self.dev_id = dev_id
        n = int(indptr.numel()) - 1
        self.graph = GraphStorage(dev_id, indptr, indices)
        self.feature = FeatureStorage(dev_id, n, row_bytes, host_table)
        self.splits = {}
        counts = []
        for mode, ids in ((TRAINMODE, train_ids), (VALIDMODE, valid_ids), (TESTMODE, test_ids)):
            if ids is None or ids.numel() == 0:
                counts.append(1)
                continue
            mine = split_seeds(ids, self.world, self.rank)
            mine_labels = labels[mine.long()].contiguous()
            self.feature.set_split(mode, mine, mine_labels)
            self.splits[mode] = (mine, mine_labels)
            counts.append(int(mine.numel()))
        dev = "cuda" if indptr.is_cuda else "cpu"
        per_rank = all_gather_ints(counts, self.dist, dev)
        self.env = None
        if use_ipc:
            self.env = IPCEnv(self.world, shm_name)
            self.env.Coordinate([c[0] for c in per_rank], [c[1] for c in per_rank], [c[2] for c in per_rank],
                                batch_size, epochs)
        self.train_step = (min(c[0] for c in per_rank) - 1) // batch_size
        self.cache_budget = max(0, min(int(cache_rows_per_gpu), n))
        cap = plan_cache_rows(n, cache_rows_per_gpu, self.world)
        self.cache = UnifiedCache(dev_id, n, row_bytes, cap, kg=self.world, ki=self.rank, codec=codec)
        self.replica_rows = 0
        return cap

    def PreSc(self, indptr, host_table):
        """Cache build.  The reference presamples an epoch to rank nodes by hotness
        (engine/server.cu:94-122, cache/cache.cu:354-447); here the ranking is by degree."""
        n = int(indptr.numel()) - 1
        order = torch.empty(n, dtype=torch.int32, device=indptr.device)
        UnifiedCache.degree_order(self.dev_id, indptr, order)
        self.cache.fill_static(order, host_table)
        if self.world > 1:
            # memory of the budget that the stripe does not need holds copies of the hottest rows of the peers
            self.replica_rows = min(self.cache_budget - self.cache.capacity, self.cache.capacity)
            if self.replica_rows > 0:
                self.cache.add_replicas(order, self.replica_rows)
            exchange_partitions(self.cache, self.rank, self.world, self.dist)
        del order
        print("System is ready for serving", flush=True)  # engine/server.cu:121, scripts/wait_file.sh:3

    def make_runner(self, batch_size, fanout, row_bytes_out, rng_seed=0):
        self.pool = MemoryPool(self.dev_id, batch_size, fanout, row_bytes_out, 2)
        self.pool.set_rng(rng_seed, 64)
        if self.env is not None:
            self.env.publish_pool(self.pool, self.dev_id)
        self.runner = Runner(self.dev_id, self.graph, self.feature, self.cache, self.pool, self.env)
        return self.runner

    def Run(self, timeout_ms=-1):
        """Serves every batch of the schedule (engine/server.cu:124-143)."""
        self.runner.serve(0, self.env.GetMaxStep(), timeout_ms)

    def Finalize(self):
        if self.runner is not None:
            self.runner.Finalize()
        if self.env is not None:
            self.env.Finalize()
