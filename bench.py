#!/usr/bin/env python
"""Mini-batch throughput of the sampling-server hot path on seeded synthetic graphs.

    python bench.py --gpus N --steps K --warmup W            # CUDA path (this repository)
    python bench.py --impl reference --steps K --warmup W     # CPU pipeline on the host cores

A step is one mini-batch per GPU: seeds -> neighbour sampling (all hops) -> dedup / relabel ->
cache lookup -> feature gather, outputs left in the hand-off buffers.
`value` = batches of all ranks / device time (CUDA events on the runner's streams, max over ranks)
with all inputs resident: windows of K batches, each bracketed by a barrier and a synchronize, are
repeated until half a second has been timed, and the median window is reported.
`e2e` = the same batches through the host-buffer C-ABI call, seeds copied in from pinned host memory
and the block structure copied back inside the timed region.
One JSON line on stdout (rank 0).
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Workloads.  elt: element type of a feature row ("f32" / "f16"); table: "host" = whole table in pinned
# host memory with a per-GPU cache in front of it, "striped" = no host copy at all, the table is spread
# over the clique's caches (every rank makes the rows of its own stripe).
CONFIGS = {
    # products-shaped (configs[0]); whole table cached
    "c1": dict(name="products-shaped RMAT", n_nodes=2449029, n_pairs=34000000, feat_len=100, classes=47,
               train_frac=0.08, batch=800, fanout=[25, 10], cache_frac=1.0),
    # paper100M-shaped (configs[1]): the configuration the metric is quoted on
    "c2": dict(name="paper100M-shaped RMAT", n_nodes=111059956, n_pairs=900000000, feat_len=128, classes=172,
               train_frac=0.011, batch=8000, fanout=[25, 10], cache_frac=0.2),
    # c2 scaled down to a few GB (inputs still larger than L2) for profiler captures
    "mid": dict(name="mid RMAT (profiler capture)", n_nodes=8000000, n_pairs=64000000, feat_len=128, classes=172,
                train_frac=0.05, batch=8000, fanout=[25, 10], cache_frac=0.2),
    # MAG240M-shaped (configs[2]): 768 x fp16 rows, 375 GB spread over the caches of 8 GPUs, no host copy;
    # 7 of 8 rows are read from peer partitions over NVLink
    "c3": dict(name="MAG240M-shaped RMAT", n_nodes=244160499, n_pairs=875000000, feat_len=768, elt="f16", classes=153,
               train_frac=0.0046, batch=1024, fanout=[25, 15], table="striped"),
    # the same layout on a graph that 1-2 GPUs can hold (profiler captures, tests of the harness)
    "c3s": dict(name="MAG240M-shaped rows on a small RMAT", n_nodes=6000000, n_pairs=48000000, feat_len=768, elt="f16",
                classes=153, train_frac=0.02, batch=1024, fanout=[25, 15], table="striped"),
    # compressed-cache variant of configs[0] (configs[3]): int8 codes + fp32 row scale in the byte budget of c1
    "c4": dict(name="products-shaped RMAT, int8 cache", n_nodes=2449029, n_pairs=34000000, feat_len=100, classes=47,
               train_frac=0.08, batch=800, fanout=[25, 10], cache_frac=1.0, codec="int8"),
    # the same codec in front of the paper100M-shaped table, where the cache does not hold everything
    "c2-int8": dict(name="paper100M-shaped RMAT, int8 cache", n_nodes=111059956, n_pairs=900000000, feat_len=128,
                    classes=172, train_frac=0.011, batch=8000, fanout=[25, 10], cache_frac=0.2, codec="int8"),
    "mid-int8": dict(name="mid RMAT, int8 cache", n_nodes=8000000, n_pairs=64000000, feat_len=128, classes=172,
                     train_frac=0.05, batch=8000, fanout=[25, 10], cache_frac=0.2, codec="int8"),
    "mid-e4m3": dict(name="mid RMAT, fp8 e4m3 cache", n_nodes=8000000, n_pairs=64000000, feat_len=128, classes=172,
                     train_frac=0.05, batch=8000, fanout=[25, 10], cache_frac=0.2, codec="e4m3"),
    # compressed rows in the host table too: a miss moves 144 instead of 512 bytes over the host link
    "c2-int8-host": dict(name="paper100M-shaped RMAT, int8 cache and int8 host table", n_nodes=111059956,
                         n_pairs=900000000, feat_len=128, classes=172, train_frac=0.011, batch=8000, fanout=[25, 10],
                         cache_frac=0.2, codec="int8", host_codec=True),
    "mid-int8-host": dict(name="mid RMAT, int8 cache and int8 host table", n_nodes=8000000, n_pairs=64000000,
                          feat_len=128, classes=172, train_frac=0.05, batch=8000, fanout=[25, 10], cache_frac=0.2,
                          codec="int8", host_codec=True),
    # dynamic-LRU stress (configs[4]): Zipf(1.1) seeds, three hops, per-GPU set-associative LRU cache of 10% of
    # the table; the 256 GB host table needs a box with that much memory (else a window of it, see host_window)
    "c5": dict(name="LRU stress RMAT", n_nodes=500000000, n_pairs=2100000000, feat_len=128, classes=172,
               train_frac=0.0, batch=4096, fanout=[15, 10, 5], cache_frac=0.1, lru_ways=8, zipf=1.1, zipf_batches=96),
    # the same workload scaled 1:25 (host table 10 GB)
    "c5s": dict(name="LRU stress RMAT scaled 1:25", n_nodes=20000000, n_pairs=80000000, feat_len=128,
                classes=172, train_frac=0.0, batch=4096, fanout=[15, 10, 5], cache_frac=0.1, lru_ways=8,
                zipf=1.1, zipf_batches=160),
    # reduced copy of c2 for checking the harness itself on small machines (never the default)
    "tiny": dict(name="tiny RMAT (harness check)", n_nodes=200000, n_pairs=2000000, feat_len=128, classes=172,
                 train_frac=0.2, batch=2000, fanout=[25, 10], cache_frac=0.2),
}

# dram__bytes_read.sum + dram__bytes_write.sum of gather_vec_kernel per 512-byte row served from GPU memory, from
# a profiler capture of the "mid" config (the full-size workload is too large for a multi-pass capture)
NCU_DRAM_BYTES_PER_HIT_ROW = 811
RNG_SEED = 0x5EED


def load_pkg():
    import __graft_entry__ as ge
    return ge._package()


def load_oracle():
    import __graft_entry__ as ge
    return ge._oracle()


def elt_of(cfg):
    import torch
    return {"f32": (torch.float32, 4), "f16": (torch.float16, 2)}[cfg.get("elt", "f32")]


class ClockSampler:
    """SM clock and throttle reasons while the timed region runs, polled from the driver library in a
    thread (a sample every millisecond or so); `nvidia-smi -lms` stands in when it cannot be loaded."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")
    BITS = {"sw_power_cap": 0x4, "hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}

    def __init__(self, gpu_index=0):
        self.rows, self.proc, self.gpu = [], None, gpu_index
        self.nv, self.handle, self.polling, self.samples, self.t = None, None, False, [], None

    def _nvml_handle(self):
        import pynvml
        pynvml.nvmlInit()
        try:
            import torch
            pr = torch.cuda.get_device_properties(self.gpu)
            bus = "%08x:%02x:%02x.0" % (pr.pci_domain_id, pr.pci_bus_id, pr.pci_device_id)
            return pynvml, pynvml.nvmlDeviceGetHandleByPciBusId(bus.encode())
        except Exception:
            return pynvml, pynvml.nvmlDeviceGetHandleByIndex(self.gpu)

    def start(self):
        try:
            self.nv, self.handle = self._nvml_handle()
            self.nv.nvmlDeviceGetClockInfo(self.handle, self.nv.NVML_CLOCK_SM)
            self.polling = True
            self.t = threading.Thread(target=self._poll, daemon=True)
            self.t.start()
            return
        except Exception:
            self.nv = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _poll(self):
        nv, h = self.nv, self.handle
        mx = 0.0
        try:
            mx = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
        except Exception:
            pass
        while self.polling:
            try:
                sm = nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)
                why = nv.nvmlDeviceGetCurrentClocksEventReasons(h)
                self.samples.append((float(sm), float(mx), int(why)))
            except Exception:
                pass
            time.sleep(0.001)

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.nv is not None:
            self.polling = False
            self.t.join(timeout=2)
            sm = sorted(s[0] for s in self.samples)
            reasons = sorted(n for n, bit in self.BITS.items() if any(s[2] & bit for s in self.samples))
            return {"sm_mhz": sm[len(sm) // 2] if sm else None,
                    "sm_max_mhz": max(s[1] for s in self.samples) if self.samples else None,
                    "reasons": reasons, "samples": len(sm), "source": "nvml"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm = sorted(float(r[1]) for r in self.rows if len(r) > 8 and r[1].replace(".", "").isdigit())
        mx = [float(r[2]) for r in self.rows if len(r) > 8 and r[2].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = set()
        for r in self.rows:
            if len(r) > 8:
                for i, nm in enumerate(names):
                    if r[5 + i].lower().startswith("active"):
                        reasons.add(nm)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "source": "nvidia-smi"}


def make_graph(cfg, device, seed=0):
    from legion_ibp_b200 import synth
    return synth.rmat_csr(cfg["n_nodes"], cfg["n_pairs"], seed=seed, device=device)


def bind_near_gpu(gpu_index):
    """Keeps this process next to its GPU: on the CPUs that the driver library reports for the device, and with
    the memory node of the GPU's PCIe slot as the preferred node of its allocations (set_mempolicy), so that the
    page-locked arrays it allocates are on the memory that the GPU's host link is attached to.  With eight ranks
    on two sockets the copies of half of them otherwise cross the socket link, whatever CPUs the container
    allows.  Returns (CPUs in the mask, preferred node); 0 / -1 for a part that could not be applied (the
    process then stays as it was)."""
    n_bound, node = 0, -1
    try:
        import torch
        pr = torch.cuda.get_device_properties(gpu_index)
        bus = "%08x:%02x:%02x.0" % (pr.pci_domain_id, pr.pci_bus_id, pr.pci_device_id)
    except Exception:
        return 0, -1
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByPciBusId(bus.encode())
        n_cpu = os.cpu_count() or 1
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (n_cpu + 63) // 64)
        cpus = {64 * w + b for w, word in enumerate(words) for b in range(64) if (int(word) >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
            n_bound = len(cpus)
    except Exception:
        pass
    try:
        import ctypes
        with open("/sys/bus/pci/devices/%s/numa_node" % bus[-12:].lower()) as fh:
            want = int(fh.read().strip())
        if want >= 0:
            mask = (ctypes.c_ulong * 16)()
            mask[want // 64] = 1 << (want % 64)
            libc = ctypes.CDLL(None, use_errno=True)
            MPOL_PREFERRED, SYS_set_mempolicy = 1, 238        # x86-64
            if os.uname().machine == "x86_64" and libc.syscall(SYS_set_mempolicy, MPOL_PREFERRED, mask, 16 * 64 + 1) == 0:
                node = want
    except Exception:
        pass
    return n_bound, node


def host_memory_bytes():
    try:
        return os.sysconf("SC_PAGE_SIZE") * os.sysconf("SC_PHYS_PAGES")
    except (ValueError, OSError):
        return 1 << 62


def host_buffer(n_bytes, shared_name, rank, world, dev=0, barrier=None):
    """uint8 buffer in host memory that every rank's GPU will read: pinned (one rank) or one POSIX shared
    segment that rank 0 creates and every rank maps.  Not initialised; a shared segment is page-locked later,
    by host_buffer_lock, once it has been filled (the driver may register a large range in pieces, and a copy
    must not straddle two of them)."""
    import torch
    if world == 1:
        return torch.empty(n_bytes, dtype=torch.uint8, pin_memory=True)
    path = "/dev/shm/" + shared_name
    if rank == 0:
        t = torch.from_file(path, shared=True, size=n_bytes, dtype=torch.uint8)
    barrier()
    if rank != 0:
        t = torch.from_file(path, shared=True, size=n_bytes, dtype=torch.uint8)
    barrier()
    if rank == 0:
        os.unlink(path)  # the mappings stay valid
    return t


def host_buffer_lock(t, rank, world, dev, barrier):
    """Page-locks a filled shared segment for this rank's GPU."""
    if world == 1:
        return
    L = load_pkg()
    barrier()
    L.host_register(dev, t)
    barrier()


def fill_host_rows(table2d, rank, world, barrier, node_of_row=None):
    """Every rank writes its share of the rows of a shared table: row r holds the features of node r, or of
    node_of_row[r]."""
    from legion_ibp_b200 import synth
    n = table2d.shape[0]
    lo, hi = n * rank // world, n * (rank + 1) // world
    synth.features_into(table2d, seed=0, row_ids=node_of_row, first=lo, last=hi)
    if barrier is not None:
        barrier()


def copy_peak(kind, n_bytes=1 << 30):
    """GB/s of a plain pinned copy over the host link: kind "h2d" (the ceiling for zero-copy reads of the
    host table) or "d2h" (the ceiling for the export of the block structure)."""
    import torch
    host = torch.empty(n_bytes, dtype=torch.uint8, pin_memory=True)
    devt = torch.empty(n_bytes, dtype=torch.uint8, device="cuda")
    src, dst = (host, devt) if kind == "h2d" else (devt, host)
    for _ in range(2):
        dst.copy_(src, non_blocking=True)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    for _ in range(3):
        dst.copy_(src, non_blocking=True)
    b.record()
    torch.cuda.synchronize()
    return 3 * n_bytes / (a.elapsed_time(b) * 1e-3) / 1e9


def presampled_counts(L, dev, indptr, indices, n, row_bytes, cfg, seeds, seed_labels, rank, world):
    """Visits per node (int32, device) over one presampling epoch of every rank's training batches."""
    import torch
    import torch.distributed as dist
    g0 = L.GraphStorage(dev, indptr, indices)
    f0 = L.FeatureStorage(dev, n, row_bytes, None)
    f0.set_split(L.TRAINMODE, seeds, seed_labels)
    pool0 = L.MemoryPool(dev, cfg["batch"], cfg["fanout"], 16, 1)   # rows are not gathered: a token row size
    pool0.set_rng(RNG_SEED + 7919 * (rank + 1), 64)                  # not the stream of the timed batches
    r0 = L.Runner(dev, g0, f0, None, pool0, None)
    counts = torch.zeros(n, dtype=torch.int32, device="cuda")
    r0.presample(0, (seeds.numel() + cfg["batch"] - 1) // cfg["batch"], counts)
    torch.cuda.synchronize()
    r0.Finalize(); pool0.close(); f0.close(); g0.close()
    if world > 1:
        dist.all_reduce(counts)
    return counts


def host_rows_seeds_first(order, seeds, n_cached):
    """(row_of[id], node_of[row]) for a host table that holds, in this order: the uncached seed nodes, the
    other uncached nodes by falling degree, and last the nodes whose rows live in the GPU caches (read
    once, at fill time)."""
    import torch
    n = order.numel()
    rank_of = torch.empty(n, dtype=torch.int64, device=order.device)
    rank_of[order.long()] = torch.arange(n, dtype=torch.int64, device=order.device)
    cls = torch.ones(n, dtype=torch.int64, device=order.device)
    cls[seeds.long()] = 0
    cls[order[:min(n, n_cached)].long()] = 2
    node_of = torch.argsort(cls * n + rank_of)
    del cls, rank_of
    row_of = torch.empty(n, dtype=torch.int32, device=order.device)
    row_of[node_of] = torch.arange(n, dtype=torch.int32, device=order.device)
    return row_of, node_of.to(torch.int32)


def zipf_batches(n_nodes, batch, n_batches, s, world=1, rank=0, device="cuda"):
    """Seed sequence of one rank for the LRU stress workload: Zipf(s) draws over node id, those with
    id % world == rank, made distinct inside every window of `batch` seeds (a mini-batch holds a node once)."""
    import torch
    from legion_ibp_b200 import synth
    # the hottest ids take a large share of the draws (of a rank's share all the more when the ranks split them), so
    # the window that has to hold `batch` distinct ids is doubled until every batch finds them
    mult = 1
    while True:
        draws = synth.zipf_seeds(n_nodes, 4 * mult * batch * n_batches * world, s=s, seed=0, device=device)
        draws = draws[(draws % world) == rank]
        win = 3 * mult * batch
        assert draws.numel() >= win * n_batches
        draws = draws[:win * n_batches].view(n_batches, win)
        out = []
        for i in range(n_batches):
            row = draws[i]
            srt, idx = torch.sort(row, stable=True)
            keep = torch.ones_like(srt, dtype=torch.bool)
            keep[1:] = srt[1:] != srt[:-1]
            first = torch.sort(idx[keep]).values  # positions of first appearances, in draw order
            uniq = row[first][:batch]
            if uniq.numel() < batch:
                break
            out.append(uniq.to(torch.int32))
        if len(out) == n_batches:
            break
        mult *= 2
        assert mult <= 64, "not enough distinct Zipf draws for a batch"
    return torch.cat(out)


def runner_counts(nc, ec):
    hops = int(nc[8])
    return int(nc[9 + hops]), int(ec[0] + ec[1])


def bounds(batch, fanout):
    nodes, edges = batch, 0
    for k in fanout:
        e = nodes * k
        edges += e
        nodes += e
    return nodes, edges


def workload_config(cfg, n_gpus):
    elt = cfg.get("elt", "f32")
    if cfg.get("table") == "striped":
        kind = "whole table striped over the caches of the %d GPU(s) (no host copy), peer rows by NVLink loads" % n_gpus
    elif cfg.get("lru_ways"):
        kind = ("%d-way set-associative LRU cache of %d%% of the table per GPU, Zipf(%.1f) seeds, misses by zero-copy "
                "from pinned host memory" % (cfg["lru_ways"], int(cfg["cache_frac"] * 100), cfg.get("zipf", 0.0)))
    elif cfg.get("codec", "raw") != "raw":
        kind = "static degree-ordered %s cache (codes + fp32 row scale) in %d%% of the table's bytes per GPU" % (
            cfg["codec"], int(cfg["cache_frac"] * 100))
        kind += (", host table held as the same compressed rows" if cfg.get("host_codec") else
                 ", misses by zero-copy from pinned host memory")
    else:
        kind = "static degree-ordered cache %d%% of the table per GPU, misses by zero-copy from pinned host memory" % int(
            cfg["cache_frac"] * 100)
    return {"workload": "%s: %d nodes, %s dim %d, batch %d, fanout %s, %s" % (
                cfg["name"], cfg["n_nodes"], elt, cfg["feat_len"], cfg["batch"], cfg["fanout"], kind),
            "batch_per_gpu": cfg["batch"], "fanout": cfg["fanout"], "feat_len": cfg["feat_len"],
            "parallelism": "dp%d, cache striped over %d GPU(s)" % (n_gpus, n_gpus),
            "l2": "inputs larger than L2 (topology, cache partition and host table are each GBs)"}


def time_cpu(fn, cores, first_guess, target_s=3.0):
    """Runs fn(first_batch, n_batches) once to warm up, then with growing batch counts until one run lasts
    about target_s seconds; returns (batches/s, batches, seconds) of that run."""
    fn(0, cores)
    first, nb = cores, first_guess
    while True:
        t0 = time.perf_counter()
        fn(first, nb)
        dt = time.perf_counter() - t0
        if dt >= 0.6 * target_s or nb >= (1 << 20):
            return nb / dt, nb, dt
        first += nb
        nb = max(nb + cores, int(nb * target_s / max(dt, 1e-3)) // cores * cores)


def cpu_arms(O, indptr, indices, seeds, labels, batch, fanout, table, cores, target_s=3.0):
    """Both CPU pipelines on the same workload: the sampler written for a CPU (Floyd's algorithm, a
    reusable relabelling map per thread) and the lock-step replay of the GPU's algorithm that the parity
    tests use.  The faster one is the baseline."""
    n_iters = max(1, (len(seeds) - 1) // batch)

    def run(fn):
        return lambda first, nb: fn(indptr, indices, seeds, labels, batch, first % n_iters, nb, fanout, 1, table, cores)
    native = time_cpu(run(O.cpu_pipeline_native), cores, 2 * cores, target_s)
    lockstep = time_cpu(run(O.cpu_pipeline), cores, 2 * cores, target_s / 2)
    best = max(native, lockstep, key=lambda r: r[0])
    which = "cpu-native" if best is native else "lock-step"
    return {"value": best[0], "unit": "batches/s", "cores": cores, "kind": "port", "sampler": which,
            "values": {"cpu-native sampler (Floyd, reusable map per thread)": native[0],
                       "lock-step replay of the GPU algorithm (the parity checker)": lockstep[0]},
            "sample": "%d batches of the same workload (sample + relabel + gather), %d threads, %.1f s" % (
                best[1], cores, best[2])}


def reference_table(cfg):
    """Host table of the CPU arm: the whole table in node-id order, or a window of it (row = id % rows) when
    the whole table does not fit the box."""
    import torch
    from legion_ibp_b200 import synth
    dtype, esz = elt_of(cfg)
    n, f = cfg["n_nodes"], cfg["feat_len"]
    rows = min(n, int(host_memory_bytes() * 0.4) // (f * esz))
    table = torch.empty((rows, f), dtype=dtype)
    synth.features_into(table, seed=0)
    return table.view(torch.uint8).view(rows, f * esz).numpy(), rows


def run_reference(args, cfg):
    """CPU arm: the DGL CPU pipeline restated in oracle/ (sample -> relabel -> gather), one batch
    per host thread, on the same synthetic workload."""
    import torch
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    O = load_oracle()
    load_pkg()
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    ip, ix = make_graph(cfg, dev)
    indptr, indices = ip.cpu().numpy(), ix.cpu().numpy()
    del ip, ix
    from legion_ibp_b200 import synth
    n = cfg["n_nodes"]
    if cfg.get("zipf"):
        assert dev == "cuda", "the Zipf seed generator of this config runs on a GPU"
        train = zipf_batches(n, cfg["batch"], cfg["zipf_batches"], cfg["zipf"]).cpu().numpy()
        tl = (train % cfg["classes"]).astype("int32")
    else:
        labels, train, _, _ = synth.labels_and_split(n, cfg["classes"], cfg["train_frac"], device=dev)
        train = train.cpu().numpy()
        tl = labels.cpu().numpy()[train]
    if dev == "cuda":
        torch.cuda.empty_cache()
    table, rows = reference_table(cfg)
    cores = O.num_threads()
    batch, fanout = cfg["batch"], cfg["fanout"]
    per_step = 4 * cores  # four batches per thread and step: the threads finish within a few percent of one another
    n_iters = (len(train) - 1) // batch
    results = {}
    for name, fn in (("cpu-native", O.cpu_pipeline_native), ("lock-step", O.cpu_pipeline)):
        it = 0
        for _ in range(args.warmup):
            fn(indptr, indices, train, tl, batch, it % max(1, n_iters - per_step), per_step, fanout, 1, table, cores)
            it += per_step
        t0 = time.perf_counter()
        for _ in range(args.steps):
            fn(indptr, indices, train, tl, batch, it % max(1, n_iters - per_step), per_step, fanout, 1, table, cores)
            it += per_step
        dt = time.perf_counter() - t0
        results[name] = (args.steps * per_step / dt, dt)
    which = max(results, key=lambda k: results[k][0])
    value, dt = results[which]
    line = {"impl": "reference", "metric": "sampled+gathered mini-batches/sec", "value": value, "unit": "batches/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": cfg.get("elt", "f32"),
            "data": "synthetic", "config": workload_config(cfg, args.gpus),
            "cpu_baseline": {"value": value, "unit": "batches/s", "cores": cores, "kind": "port", "sampler": which,
                             "values": {k: v[0] for k, v in results.items()},
                             "sample": "%d batches per step (four per thread), %d steps; host table of %d rows in "
                                       "node-id order" % (per_step, args.steps, rows)},
            "e2e": {"value": value, "unit": "batches/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="c2", choices=sorted(CONFIGS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-cpu-binding", action="store_true",
                    help="leave the process on whatever CPUs it was started on (default: the CPUs next to its GPU)")
    ap.add_argument("--cache-order", choices=["degree", "hotness"], default="degree",
                    help="ranking that fills the static caches: node degree, or the visits counted in a presampling "
                         "epoch over the training batches (the reference's PreSc)")
    ap.add_argument("--no-edge-counts", action="store_true",
                    help="skip the second host-buffer loop, which delivers per-destination edge counts in the place of "
                         "agg_dst (extra key e2e_edge_counts)")
    ap.add_argument("--edge-counts", action="store_true", help=argparse.SUPPRESS)  # the loop runs by default
    ap.add_argument("--cache-frac", type=float, default=None, help="override the cached fraction of the table")
    ap.add_argument("--pipes", type=int, default=0,
                    help="batches in flight on the device (0: 4 for static caches, 2 for the LRU cache; the hand-off to "
                         "trainer processes uses 2)")
    ap.add_argument("--slots", type=int, default=2,
                    help="hand-off buffer sets of the device-resident leg (the trainers' segment holds 2); pipes beyond "
                         "them sample ahead into private buffers")
    ap.add_argument("--host-layout", default="packed", choices=["id", "packed", "seeds_first"],
                    help="row order of the pinned host table: node-id order (the feature file's); packed = the rows of "
                         "uncached nodes by falling degree, cached rows last (what the sampling_server binary does at "
                         "load time: the likeliest misses next to each other); seeds_first = uncached seed nodes, then "
                         "packed (only matters without seed staging)")
    ap.add_argument("--no-replicas", action="store_true",
                    help="N > 1: stripe the whole per-GPU budget over the clique (the reference's placement) instead "
                         "of planning private copies of the hottest peer rows")
    ap.add_argument("--no-seed-staging", action="store_true",
                    help="fetch the rows of uncached seeds like any other miss instead of staging them by the copy engine")
    ap.add_argument("--topology", default="device", choices=["device", "host"],
                    help="where the CSR lives: in this GPU's memory (default), or in pinned host memory read in place by "
                         "zero-copy loads (what a graph that does not fit beside the cache falls back to)")
    ap.add_argument("--tunable", action="append", default=[], metavar="NAME=VALUE",
                    help="launch-shape knob passed to legion_set_tunable")
    ap.add_argument("--profile-only", action="store_true",
                    help="set-up, warm-up and one timed window only (for runs under a profiler); prints no bench line")
    args = ap.parse_args()
    cfg = dict(CONFIGS[args.config])
    if args.cache_frac is not None:
        cfg["cache_frac"] = args.cache_frac
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args, cfg)
        return

    import numpy as np
    import torch
    L = load_pkg()
    L.lib()  # fails loudly when the CUDA library is missing
    for kv in args.tunable:
        name, _, val = kv.partition("=")
        L._check(L.lib().legion_set_tunable(name.encode(), int(val)))
    from legion_ibp_b200 import synth
    assert torch.cuda.is_available(), "bench.py needs a GPU (use --impl reference for the CPU arm)"
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, "--gpus must equal the number of launched ranks"
    # (one rank keeps all CPUs: the CPU baseline of the same run uses every core)
    near_cpus, near_node = (0, -1) if (args.no_cpu_binding or world == 1) else bind_near_gpu(local_rank)
    torch.cuda.set_device(local_rank)
    dev = local_rank
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    t_setup = time.perf_counter()

    def barrier0():
        if dist is not None:
            dist.barrier()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        if dist is None:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def sum_over_ranks(x):
        if dist is None:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t)
        return float(t.item())

    # ---- synthetic inputs -------------------------------------------------------------------
    indptr, indices = make_graph(cfg, "cuda")
    torch.cuda.empty_cache()
    n, f = cfg["n_nodes"], cfg["feat_len"]
    dtype, esz = elt_of(cfg)
    row_bytes = f * esz
    n_edges = int(indices.numel())
    striped = cfg.get("table") == "striped"
    lru_ways = cfg.get("lru_ways", 0)
    if cfg.get("zipf"):
        train = zipf_batches(n, cfg["batch"], cfg["zipf_batches"], cfg["zipf"], world, rank)
        mine = train
        mine_labels = (mine % cfg["classes"]).to(torch.int32).contiguous()
    else:
        labels, train, _, _ = synth.labels_and_split(n, cfg["classes"], max(cfg["train_frac"], 1e-6), device="cuda")
        mine = train[(train % world) == rank].contiguous()  # id % ngpu split, storage_management.cu:214-250
        mine_labels = labels[mine.long()].contiguous()
        del labels

    # ---- ranking and cache plan -----------------------------------------------------------------
    codec_name = cfg.get("codec", "raw")
    codec = {"raw": L.CODEC_RAW, "int8": L.CODEC_INT8, "e4m3": L.CODEC_E4M3}[codec_name]
    slot_bytes = row_bytes if codec == L.CODEC_RAW else (f + 4 + 15) // 16 * 16
    order = None
    replica_rows = 0
    access_counts = None
    if not lru_ways:
        order = torch.empty(n, dtype=torch.int32, device="cuda")
        if args.cache_order == "hotness" and not striped:
            # the reference's presampling epoch (GPUServer::PreSc, engine/server.cu:94-122): every training batch
            # is sampled once with a random stream of its own, the visits of all ranks are added up
            # (cache/cache.cu:354-447) and the nodes are ranked by them
            access_counts = presampled_counts(L, dev, indptr, indices, n, row_bytes, cfg, mine, mine_labels, rank, world)
            L.UnifiedCache.hotness_order(dev, access_counts, order)
        else:
            L.UnifiedCache.degree_order(dev, indptr, order)
    if striped:
        cap = (n + world - 1) // world
        need = cap * row_bytes + 8 * (n + 1) + 4 * n_edges + 4 * n
        free_b, _ = torch.cuda.mem_get_info()
        assert need < free_b + 4 * n, ("the table striped over %d GPU(s) needs %.0f GB per GPU next to the topology; "
                                       "run this config on more GPUs" % (world, need / 1e9))
    else:
        budget = cap = min(n, int(n * cfg["cache_frac"] * row_bytes / slot_bytes))
        if cap * world >= n:
            cap = (n + world - 1) // world
        if world > 1 and not args.no_replicas and not lru_ways:
            from legion_ibp_b200 import server
            mass = server.degree_mass(indptr, order) if access_counts is None else server.weight_mass(access_counts, order)
            cap, replica_rows = server.plan_clique_cache(mass, n, budget, world)
            del mass

    # ---- host table ----------------------------------------------------------------------------------
    table = None           # [rows, row_bytes] uint8 view of the pinned host table
    table_rows = 0
    row_of = None
    stored = None          # compressed copy of the host table (configs with host_codec)
    host_layout = "none" if striped else ("id" if lru_ways else args.host_layout)
    if not striped:
        table_rows = n
        whole = n * row_bytes
        if whole > 0.8 * host_memory_bytes():
            # the box cannot hold the table: a window of it stands in (row = id % rows), sized to half the memory
            table_rows = int(host_memory_bytes() * 0.5) // row_bytes
            assert lru_ways, "only the LRU cache addresses a window of the table (row = id % rows)"
        node_of = None
        if host_layout == "seeds_first":
            row_of, node_of = host_rows_seeds_first(order, train, cap * world)
        elif host_layout == "packed":
            n_cached = min(n, cap * world)
            row_of = torch.empty(n, dtype=torch.int32, device="cuda")
            L.UnifiedCache.pack_order(dev, order, n_cached, row_of)
            node_of = torch.cat([order[n_cached:], order[:n_cached]])
        table = host_buffer(table_rows * row_bytes, "legion_b200_bench_features", rank, world, dev, barrier0)
        fill_host_rows(table.view(dtype).view(table_rows, f), rank, world, barrier0, node_of)
        host_buffer_lock(table, rank, world, dev, barrier0)
        table = table.view(table_rows, row_bytes)
        del node_of

    def expected_rows(ids_t):
        """Rows that a gather of these node ids must return (device tensor [len, row_bytes] of bytes)."""
        src = ids_t.long() if table_rows in (0, n) else ids_t.long() % table_rows
        return synth.feature_rows(src, f, 0, dtype).view(torch.uint8).view(-1, row_bytes)

    # ---- storage, cache, pool, runner ------------------------------------------------------------
    if args.topology == "host":
        topo = (indptr.cpu().pin_memory(), indices.cpu().pin_memory())
        g = L.GraphStorage(dev, topo[0], topo[1])
    else:
        g = L.GraphStorage(dev, indptr, indices)
    fs = L.FeatureStorage(dev, table_rows if table_rows else n, row_bytes, table)
    fs.set_split(L.TRAINMODE, mine, mine_labels)
    if lru_ways:
        # every GPU keeps its own LRU cache (no clique: the contents change every batch)
        cap = cap // lru_ways * lru_ways
        cache = L.UnifiedCache(dev, table_rows, row_bytes, 0, lru=(cap // lru_ways, lru_ways))
        cache.set_host_table(table)
    elif striped:
        cache = L.UnifiedCache(dev, n, row_bytes, cap, kg=world, ki=rank, codec=codec)
        cache.place_static(order)
        chunk = 1 << 17
        for s0 in range(0, cap, chunk):
            s1 = min(cap, s0 + chunk)
            t_idx = torch.arange(s0, s1, device="cuda", dtype=torch.int64) * world + rank
            t_idx = t_idx[t_idx < n]
            if t_idx.numel():
                cache.write_partition_rows(s0, synth.feature_rows(order[t_idx], f, 0, dtype))
        torch.cuda.synchronize()
    else:
        if cfg.get("host_codec"):
            stored = host_buffer(n * slot_bytes, "legion_b200_bench_codes", rank, world, dev, barrier0)
            host_buffer_lock(stored, rank, world, dev, barrier0)   # written in place by rank 0's kernel, row by row
            stored = stored.view(n, slot_bytes)
            if rank == 0:
                L.quantize_table(dev, codec, table, n, f, stored)
            barrier0()
        cache = L.UnifiedCache(dev, n, row_bytes, cap, kg=world, ki=rank, codec=codec)
        if stored is not None:
            cache.set_host_codec(codec)
        cache.fill_static(order, table if stored is None else stored, row_of_id=row_of)
        if replica_rows > 0:
            cache.add_replicas(order, replica_rows, row_of_id=row_of)
    del order, access_counts
    share = None
    if world > 1 and not lru_ways:
        from legion_ibp_b200 import server
        share = server.exchange_partitions(cache, rank, world, dist)
    pipes = args.pipes or (2 if lru_ways else 4)
    # The device-resident leg leaves its batches in two hand-off slots, the number the trainers' segment holds;
    # behind a static cache the other pipes sample ahead of them into private buffers.  The host-buffer leg has a
    # pool of its own whose pipes are its slots (every batch in flight is exported to its own host arrays).
    slots = min(pipes, args.slots) if not lru_ways else pipes
    pool = L.MemoryPool(dev, cfg["batch"], cfg["fanout"], row_bytes, pipes, slots=slots)
    pool.set_rng(RNG_SEED + rank, 64)
    runner = L.Runner(dev, g, fs, cache, pool, None)
    if slots < pipes:
        pool_h = L.MemoryPool(dev, cfg["batch"], cfg["fanout"], row_bytes, pipes)
        pool_h.set_rng(RNG_SEED + rank, 64)
        runner_h = L.Runner(dev, g, fs, cache, pool_h, None)
    else:
        pool_h, runner_h = pool, runner
    n_iters = (int(mine.numel()) - 1) // cfg["batch"]
    seeds_h = mine.cpu().numpy()
    labels_h = mine_labels.cpu().numpy()
    staging = None
    if not args.no_seed_staging and hasattr(runner, "stage_seeds") and not lru_ways and not striped and codec == L.CODEC_RAW:
        staging = {"list": runner.stage_seeds(L.TRAINMODE), "host": runner_h.register_host_seeds(seeds_h)}
    torch.cuda.synchronize()
    setup_s = time.perf_counter() - t_setup

    # ---- full-size checks (outside every timed region) --------------------------------------------
    O = load_oracle() if rank == 0 else None
    h_indptr = h_indices = None
    if rank == 0:
        h_indptr, h_indices = indptr.cpu().numpy(), indices.cpu().numpy()

    def check_batch(pipe, global_batch, it, what, pool=pool):
        """The batch that sits in `pipe`: every gathered row against the table's generator on all ranks, and on
        rank 0 ids, labels, both edge lists and both counter arrays against the CPU checker's batch."""
        torch.cuda.synchronize()
        nc = pool.read(L.BUF_NODE_COUNTER, pipe, 16, np.int32)
        ec = pool.read(L.BUF_EDGE_COUNTER, pipe, 16, np.int32)
        nn, ne = runner_counts(nc, ec)
        ids_np = pool.read(L.BUF_IDS, pipe, nn, np.int32)
        ids_t = torch.from_numpy(ids_np).cuda()
        fptr, _ = pool.buffer(L.BUF_FEATURES, pipe)
        got = torch.empty(nn * row_bytes, dtype=torch.uint8, device="cuda")
        L._check(L.lib().legion_copy(ctypes.c_void_p(got.data_ptr()), ctypes.c_void_p(fptr), ctypes.c_int64(nn * row_bytes),
                                     ctypes.c_int32(3)))
        got = got.view(nn, row_bytes)
        bad = 0
        for r0 in range(0, nn, 1 << 17):
            r1 = min(nn, r0 + (1 << 17))
            want = expected_rows(ids_t[r0:r1])
            if codec == L.CODEC_RAW:
                bad += int((got[r0:r1] != want).any(dim=1).sum().item())
            else:
                # rows served by the compressed cache: |x - x^| <= absmax / 254 for int8 (half a code step); half an
                # e4m3 step (2^-4 relative) of the scaled value for fp8; rows that missed are exact
                w, x = want.view(torch.float32), got[r0:r1].view(torch.float32)
                amax = w.abs().amax(dim=1, keepdim=True)
                tol = amax / 254.0 * 1.001 if codec == L.CODEC_INT8 else torch.maximum(w.abs() / 16.0, amax / 448.0 / 1024.0) * 1.001
                bad += int(((x - w).abs() > tol).any(dim=1).sum().item())
        assert bad == 0, "%s: %d of %d gathered rows differ from the table" % (what, bad, nn)
        res = {"rows_checked": nn}
        if rank == 0:
            ref = O.run_batch(h_indptr, h_indices, seeds_h, labels_h, cfg["batch"], it, cfg["fanout"], global_batch,
                              RNG_SEED + rank)
            assert np.array_equal(nc, ref["node_counter"]) and np.array_equal(ec, ref["edge_counter"]), what
            assert np.array_equal(ids_np, ref["ids"]), what
            assert np.array_equal(pool.read(L.BUF_LABELS, pipe, int(nc[9]), np.int32), ref["labels"]), what
            assert np.array_equal(pool.read(L.BUF_AGG_SRC, pipe, ne, np.int32), ref["agg_src"]), what
            assert np.array_equal(pool.read(L.BUF_AGG_DST, pipe, ne, np.int32), ref["agg_dst"]), what
            res.update(ids=nn, edges=ne, against="CPU checker: ids, labels, agg_src, agg_dst, node_counter, edge_counter bit-exact")
        return res

    # ---- value: inputs resident, device-timed ----------------------------------------------------
    step = 0
    for _ in range(args.warmup):
        runner.enqueue(step, L.TRAINMODE, step % n_iters)
        step += 1
    lru_warm = 0
    if lru_ways and not args.profile_only:
        # an LRU cache starts empty: one pass over the seed batches fills it before anything is timed, so that
        # `value` is the rate of a warm cache like `e2e`, which runs later, and not of the compulsory misses
        lru_warm = n_iters
        for _ in range(lru_warm):
            runner.enqueue(step, L.TRAINMODE, step % n_iters)
            step += 1
    runner.sync()
    checks = {"value_path": check_batch((step - 1) % pipes % slots, step - 1, (step - 1) % n_iters, "device-resident batch")}
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    windows = []
    timed_s, budget_s = 0.0, (0.0 if args.profile_only else 0.5)
    while True:
        barrier()
        for _ in range(args.steps):
            runner.enqueue(step, L.TRAINMODE, step % n_iters)
            step += 1
        runner.sync()
        barrier()
        ms = max_over_ranks(runner.timing()["batch_ms"])
        windows.append(ms)
        timed_s += ms * 1e-3
        if timed_s >= budget_s or len(windows) >= 400:
            break
    wsorted = sorted(windows)
    ms_total = wsorted[len(wsorted) // 2]
    value = args.steps * world / (ms_total * 1e-3)
    assert pool.device_error() == 0, "device-side error flag set"
    if args.profile_only:
        if rank == 0:
            sampler.stop()
            print(json.dumps({"profile_only": True, "ms_per_step": ms_total / args.steps, "value": value}), flush=True)
        runner.Finalize()
        return

    # ---- kernel durations: the same graph replay with CUDA events around the gather launches, one
    # batch at a time (the events of a pipe's graph are overwritten by its next launch) ----------------
    runner.set_options(use_graph=True, time_kernels=True)
    for _ in range(2):
        runner.enqueue(step, L.TRAINMODE, step % n_iters)
        step += 1
    runner.sync()
    stats0 = cache.stats()
    staged0 = runner.staged_rows() if staging else 0
    tm = {"gather_ms": 0.0, "miss_ms": 0.0, "timed": 0}
    k_steps = max(args.steps, 40)
    for _ in range(k_steps):
        runner.enqueue(step, L.TRAINMODE, step % n_iters)
        step += 1
        runner.sync()
        t1 = runner.timing()
        for k in tm:
            tm[k] += t1[k]
    stats1 = cache.stats()
    staged = (runner.staged_rows() - staged0) if staging else 0
    # the same events with batches in flight: how busy the host-link stream is in steady state
    for _ in range(k_steps):
        runner.enqueue(step, L.TRAINMODE, step % n_iters)
        step += 1
    runner.sync()
    tp = runner.timing()
    pipeline = {"window_ms_per_batch": tp["batch_ms"] / k_steps, "miss_ms_per_batch": tp["miss_ms"] / k_steps,
                "miss_stream_busy_frac": tp["miss_ms"] / tp["batch_ms"] if tp["batch_ms"] > 0 else None}
    runner.set_options(use_graph=True, time_kernels=False)
    clocks = sampler.stop() if rank == 0 else None

    # ---- roofline of the gather ---------------------------------------------------------------------
    # Algorithmic bytes per gathered row: the row read from its source + the row written + 4 B id +
    # 4 B lookup-table entry.  Rows served from GPU memory are moved by the hit kernel (HBM bound; rows of
    # uncached seeds that the copy engine staged in device memory count among them); rows that miss the cache
    # are moved by the miss kernel over the host link, for which the hit kernel still reads id + table entry
    # and writes an 8-byte list entry.
    d = {k: stats1[k] - stats0[k] for k in stats0}
    hits = d["local_hits"] + d["peer_hits"] + staged
    rows = hits + d["misses"]
    gather_launches = tm["timed"]  # one lookup + gather launch per batch
    hit_read = slot_bytes + (4 * lru_ways + 4 if lru_ways else 0)
    hit_bytes = (hits - staged) * (hit_read + row_bytes + 8) + staged * (2 * row_bytes + 12) + d["misses"] * 16
    host_row_bytes = slot_bytes if stored is not None else row_bytes   # bytes a miss moves over the host link
    miss_bytes = d["misses"] * (host_row_bytes + row_bytes + 8)
    gather_s = tm["gather_ms"] * 1e-3
    miss_s = tm["miss_ms"] * 1e-3
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    hbm_peak = float(peaks.get("hbm_gbs", 6650.0))
    achieved = hit_bytes / gather_s / 1e9 if gather_s > 0 else 0.0
    traffic = traffic_source = None
    if codec == L.CODEC_RAW and not lru_ways and row_bytes == 512 and world == 1:
        traffic = NCU_DRAM_BYTES_PER_HIT_ROW * hits / max(1, gather_launches)
        traffic_source = ("ncu dram__bytes_read.sum + dram__bytes_write.sum of the mid config (%d B per row served "
                          "from GPU memory; part of the written rows is still in L2 when the kernel ends), scaled "
                          "by the rows per launch" % NCU_DRAM_BYTES_PER_HIT_ROW)
    kname = ("gather_lru_kernel (set probe + gather of rows held in the LRU cache)" if lru_ways else
             "gather_quant_kernel<%s> (cache lookup + gather with in-kernel dequantisation)" % codec_name
             if codec != L.CODEC_RAW else "gather_vec_kernel (cache lookup + gather of rows held in GPU memory)")
    peer_frac = d["peer_hits"] / max(1, rows)
    roofline = {"bound": "hbm", "kernel": kname,
                "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                "peak_source": "of measured (MEASURED_PEAKS.json hbm_gbs)" if peaks else "of fallback 6650 GB/s",
                "traffic": traffic, "traffic_source": traffic_source, "launches": gather_launches,
                "avg_launch_ms": tm["gather_ms"] / max(1, gather_launches),
                "rows_per_batch": rows / k_steps, "staged_seed_rows_per_batch": staged / k_steps,
                "source_split": {k: d[k] / max(1, rows) for k in ("local_hits", "peer_hits", "misses")},
                "measured": "CUDA events around each launch on its stream, %d batches run one at a time right "
                            "after the timed region" % tm["timed"]}
    roofline_nvlink = None
    if d["peer_hits"] > 0:
        # rows read from peer partitions cross NVLink inside the same kernel; 770 GB/s per direction is the
        # peer copy measured on this pool (900 nominal)
        nv = d["peer_hits"] * slot_bytes / gather_s / 1e9 if gather_s > 0 else 0.0
        roofline_nvlink = {"bound": "nvlink", "kernel": kname, "achieved": nv, "peak": 770.0, "unit": "GB/s",
                           "frac": nv / 770.0, "peak_source": "peer copy measured on this pool, per direction",
                           "peer_rows_per_batch": d["peer_hits"] / k_steps, "peer_row_frac": peer_frac}
        if peer_frac > 0.5:
            # most rows cross NVLink: that link, not HBM, bounds the launch
            roofline = dict(roofline_nvlink, hbm=roofline, traffic=None, launches=gather_launches,
                            avg_launch_ms=tm["gather_ms"] / max(1, gather_launches))
    # one rank at a time: the ranks' host links share the host's memory and root ports
    link_peak = 0.0
    for k in range(world):
        if k == rank:
            link_peak = copy_peak("h2d")
        barrier()
    roofline_host = None
    if table is not None:
        link_achieved = d["misses"] * host_row_bytes / miss_s / 1e9 if miss_s > 0 else 0.0
        roofline_host = {"bound": "host_link", "kernel": "gather_miss_kernel (zero-copy fetch of missed rows)",
                         "achieved": link_achieved, "peak": link_peak, "unit": "GB/s",
                         "frac": link_achieved / link_peak if link_peak else None,
                         "peak_source": "pinned host->device cudaMemcpy of 1 GiB measured in this run, one rank at a time",
                         "launches": tm["timed"], "avg_launch_ms": tm["miss_ms"] / max(1, tm["timed"]),
                         "rows_per_batch": d["misses"] / k_steps, "algorithmic_bytes": miss_bytes,
                         "copy_engine_bytes_per_batch": staged * row_bytes / k_steps}
    # lower bound of the whole gather step: the slowest of the HBM side, the NVLink side and the host-link side
    t_lb = max(hit_bytes / (hbm_peak * 1e9), d["peer_hits"] * slot_bytes / 770e9,
               (d["misses"] * host_row_bytes + staged * row_bytes) / (link_peak * 1e9) if link_peak else 0.0)
    roofline_path = {"lower_bound_ms_per_batch": t_lb / k_steps * 1e3,
                     "gather_ms_per_batch": (tm["gather_ms"] + tm["miss_ms"]) / max(1, tm["timed"]),
                     "batch_ms": ms_total / args.steps}

    # ---- e2e: host buffers through the C ABI --------------------------------------------------------
    max_nodes, max_edges = bounds(cfg["batch"], cfg["fanout"])
    depth = pipes if lru_ways else pipes + 1   # static caches: one more batch may sample ahead of the pipes
    outs = [dict(ids=torch.empty(max_nodes, dtype=torch.int32).pin_memory().numpy(),
                 lab=torch.empty(cfg["batch"], dtype=torch.int32).pin_memory().numpy(),
                 src=torch.empty(max_edges, dtype=torch.int32).pin_memory().numpy(),
                 dst=torch.empty(max_edges, dtype=torch.int32).pin_memory().numpy()) for _ in range(depth)]
    nc_o, ec_o = np.zeros(16, np.int32), np.zeros(16, np.int32)
    b = cfg["batch"]

    def submit(i, gb_base=0):
        # gb_base: the timed loops draw with batch numbers that nothing before them used (a batch that is run twice
        # finds its rows in an LRU cache the second time)
        it = i % n_iters
        o = outs[i % depth]
        runner_h.submit_host_to(seeds_h[it * b:(it + 1) * b], labels_h[it * b:(it + 1) * b], gb_base + i, o["ids"],
                                o["lab"], o["src"], o["dst"])

    def collect():
        return runner_h.collect_host(None, None, None, None, nc_o, ec_o, None)

    pipe0 = runner_h.current_pipe()
    for i in range(depth):
        submit(i)
    for i in range(depth, depth + 4):
        collect()
        submit(i)
    for _ in range(depth):
        collect()
    # the exported block structure of the last batch is what the device buffers hold, and that batch is right
    last = depth + 3
    nn_chk, ne_chk = runner_counts(nc_o, ec_o)
    chk_pipe = (pipe0 + last) % pipes
    o_chk = outs[last % depth]
    assert np.array_equal(o_chk["ids"][:nn_chk], pool_h.read(L.BUF_IDS, chk_pipe, nn_chk, np.int32))
    assert np.array_equal(o_chk["src"][:ne_chk], pool_h.read(L.BUF_AGG_SRC, chk_pipe, ne_chk, np.int32))
    assert np.array_equal(o_chk["dst"][:ne_chk], pool_h.read(L.BUF_AGG_DST, chk_pipe, ne_chk, np.int32))
    checks["host_buffer_path"] = check_batch(chk_pipe, last, last % n_iters, "host-buffer batch", pool_h)
    # wall clock needs a longer window than the device-timed leg: at least 0.5 s of steps
    e2e_steps = max(args.steps, 200, int(0.6 / max(ms_total / args.steps * 1e-3, 1e-6)))
    e2e_steps = min(e2e_steps, 20000)
    def timed_e2e(counts):
        """e2e_steps batches through the host-buffer calls; counts: per-destination edge counts (bytes) leave in
        the place of agg_dst.  Returns (seconds, max over ranks; bytes device -> host; host times)."""
        runner_h.set_edge_counts(counts)
        base = (2 << 20) if counts else (1 << 20)
        for i in range(depth):          # a first round, untimed: sizes the copies that run ahead
            submit(50 + i, base)
        for _ in range(depth):
            collect()
        barrier()
        runner_h.host_times()
        t0 = time.perf_counter()
        d2h = 0
        hops_n = len(cfg["fanout"])

        def out_bytes(nn, ne):
            if counts:
                return 4 * nn + 4 * ne + int(sum(nc_o[9 + h] for h in range(hops_n))) + 4 * b + 128
            return 4 * nn + 8 * ne + 4 * b + 128
        for i in range(depth):
            submit(100 + i, base)
        for i in range(depth, e2e_steps):
            nn, ne = collect()
            d2h += out_bytes(nn, ne)
            submit(100 + i, base)
        for _ in range(depth):
            nn, ne = collect()
            d2h += out_bytes(nn, ne)
        torch.cuda.synchronize()
        sec = max_over_ranks(time.perf_counter() - t0)
        ht = runner_h.host_times()
        barrier()
        runner_h.set_edge_counts(False)
        return sec, d2h, ht

    barrier()
    staged_e2e0 = runner_h.staged_rows() if staging else 0
    e2e_s, d2h, ht = timed_e2e(False)
    staged_e2e = (runner_h.staged_rows() - staged_e2e0) if staging else 0
    # floor of the export: every rank copies device -> pinned host at the same time
    barrier()
    d2h_peak = copy_peak("d2h")
    barrier()
    d2h_peak_min = -max_over_ranks(-d2h_peak)
    e2e_value = e2e_steps * world / e2e_s
    d2h_per_step = d2h // e2e_steps
    floor_s = d2h_per_step / (d2h_peak_min * 1e9)
    e2e = {"value": e2e_value, "unit": "batches/s", "h2d_bytes_per_step": 8 * b + staged_e2e * row_bytes // e2e_steps,
           "d2h_bytes_per_step": d2h_per_step, "steps": e2e_steps,
           "api": "legion_runner_submit_host_to / legion_runner_collect_host, %d batches in flight" % depth,
           "host_us_per_step": {"submit": ht["submit_us"] / max(1.0, ht["batches"]), "collect": ht["collect_us"] / max(1.0, ht["batches"]),
                                "of_which_waiting_for_the_device": ht["collect_wait_us"] / max(1.0, ht["batches"]),
                                "wall": e2e_s / e2e_steps * 1e6},
           "note": "seeds+labels copied in from host memory (and, with seed staging, the rows of uncached seeds by the copy "
                   "engine), ids/labels/edge lists/counters written to page-locked host memory every step; gathered rows "
                   "stay in the device hand-off buffer where the trainer reads them; missed rows cross the host link "
                   "inside the gather"}
    e2e_counts = None
    if not args.no_edge_counts:
        # the same loop with the edge counts in the place of agg_dst, checked on its last batch first
        runner_h.set_edge_counts(True)
        cnt_bufs = [torch.empty(len(cfg["fanout"]) * max_nodes + 16, dtype=torch.uint8).pin_memory().numpy() for _ in range(depth)]
        for o, cb in zip(outs, cnt_bufs):
            o["dst_i32"], o["dst"] = o["dst"], cb
        for i in range(depth):
            submit(i)
        for _ in range(depth):
            collect()
        nn_c, ne_c = runner_counts(nc_o, ec_o)
        last_c = depth - 1
        pipe_c = runner_h.current_pipe()
        pipe_c = (pipe_c + pipes - 1) % pipes
        n_cnt = int(sum(nc_o[9 + h] for h in range(len(cfg["fanout"]))))
        dst_c = L.agg_dst_from_counts(outs[last_c % depth]["dst"][:n_cnt], nc_o)
        assert np.array_equal(dst_c, pool_h.read(L.BUF_AGG_DST, pipe_c, ne_c, np.int32)), "edge counts do not give agg_dst"
        sec_c, d2h_c, ht_c = timed_e2e(True)
        e2e_counts = {"value": e2e_steps * world / sec_c, "unit": "batches/s", "d2h_bytes_per_step": d2h_c // e2e_steps,
                      "steps": e2e_steps, "agg_dst_rebuilt_and_checked": True,
                      "floor_ms_per_step": d2h_c / e2e_steps / (d2h_peak_min * 1e9) * 1e3,
                      "achieved_ms_per_step": sec_c / e2e_steps * 1e3,
                      "note": "legion_runner_set_edge_counts(1): one byte per destination and hop leaves in the place of "
                              "agg_dst (4 bytes per edge); everything else as in e2e"}
        for o in outs:
            o["dst"] = o.pop("dst_i32")
    roofline_e2e = {"bound": "host_link_d2h", "peak": d2h_peak_min, "unit": "GB/s",
                    "peak_source": "device -> pinned host cudaMemcpy of 1 GiB, all ranks at the same time, slowest rank",
                    "d2h_bytes_per_step": d2h_per_step, "floor_ms_per_step": floor_s * 1e3,
                    "achieved_ms_per_step": e2e_s / e2e_steps * 1e3,
                    "frac": floor_s / (e2e_s / e2e_steps) if e2e_s > 0 else None}

    # ---- CPU baseline on this box's cores (rank 0, N=1 only) ----------------------------------------
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cores = O.num_threads()
        if table is not None and table_rows == n and row_of is None:
            tnp = table.numpy()
        else:
            # the CPU pipeline reads a table in node-id order (a window of it when the box cannot hold it)
            del table
            tnp, _ = reference_table(cfg)
        cpu = cpu_arms(O, h_indptr, h_indices, seeds_h, labels_h, b, cfg["fanout"], tnp, cores)

    if rank == 0:
        hops = len(cfg["fanout"])
        per_batch = 1 + 4 * hops + 1 + (1 if not striped else 0) + (3 if lru_ways else 0)
        line = {"metric": "sampled+gathered mini-batches/sec", "value": value, "unit": "batches/s",
                "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": cfg.get("elt", "f32"), "data": "synthetic",
                "config": workload_config(cfg, world), "host_table_layout": host_layout, "lru_warm_batches": lru_warm, "cpus_bound_near_gpu": near_cpus, "preferred_memory_node": near_node,
                "cache_order": ("none" if lru_ways else ("degree" if striped else args.cache_order)),
                "host_table_rows": table_rows, "pipes": pipes, "handoff_slots": slots, "topology": args.topology,
                "windows": {"count": len(windows), "timed_s": timed_s, "ms_per_step_min": wsorted[0] / args.steps,
                            "ms_per_step_median": ms_total / args.steps, "ms_per_step_max": wsorted[-1] / args.steps},
                "e2e": e2e, "gpu_launches": args.steps * per_batch,
                "roofline": roofline, "roofline_host_link": roofline_host, "roofline_path": roofline_path,
                "roofline_nvlink": roofline_nvlink, "roofline_e2e": roofline_e2e, "e2e_edge_counts": e2e_counts,
                "pipeline": pipeline, "full_size_checks": checks,
                "cpu_baseline": cpu, "vs_cpu_baseline": {"value": value / cpu["value"], "e2e": e2e_value / cpu["value"]} if cpu else None,
                "clocks": clocks,
                "graph": {"nodes": n, "directed_edges": n_edges, "train_seeds_this_rank": int(mine.numel()),
                          "cache_rows_per_gpu": cap, "replica_rows_per_gpu": replica_rows,
                          "peer_mapping": share, "seed_staging": bool(staging)},
                "setup_s": setup_s, "tunables": args.tunable or None}
        print(json.dumps(line), flush=True)
    assert pool_h.device_error() == 0, "device-side error flag set"
    if runner_h is not runner:
        runner_h.Finalize()
    runner.Finalize()
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
