#!/usr/bin/env python
"""Mini-batch throughput of the sampling-server hot path on seeded synthetic graphs.

    python bench.py --gpus N --steps K --warmup W            # CUDA path (this repository)
    python bench.py --impl reference --steps K --warmup W     # CPU pipeline on the host cores

A step is one mini-batch per GPU: seeds -> neighbour sampling (all hops) -> dedup / relabel ->
cache lookup -> feature gather, outputs left in the double-buffered hand-off buffers.
`value` = batches of all ranks / device time (CUDA events on the runner's streams, max over ranks)
with all inputs resident; `e2e` = the same batches through the host-buffer C-ABI call, seeds copied
in from pinned host memory and the block structure copied back inside the timed region.
One JSON line on stdout (rank 0).
"""
import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CONFIGS = {
    # products-shaped (BASELINE.json configs[0]); whole table cached
    "c1": dict(name="products-shaped RMAT", n_nodes=2449029, n_pairs=34000000, feat_len=100, classes=47,
               train_frac=0.08, batch=800, fanout=[25, 10], cache_frac=1.0),
    # paper100M-shaped (configs[1]): the configuration the metric is quoted on
    "c2": dict(name="paper100M-shaped RMAT", n_nodes=111059956, n_pairs=900000000, feat_len=128, classes=172,
               train_frac=0.011, batch=8000, fanout=[25, 10], cache_frac=0.2),
    # c2 scaled down to a few GB (inputs still larger than L2) for profiler captures
    "mid": dict(name="mid RMAT (profiler capture)", n_nodes=8000000, n_pairs=64000000, feat_len=128, classes=172,
                train_frac=0.05, batch=8000, fanout=[25, 10], cache_frac=0.2),
    # compressed-cache variant of c2 (configs[3]): the same byte budget holds int8 rows + fp32 scale
    "c4": dict(name="paper100M-shaped RMAT, int8 cache", n_nodes=111059956, n_pairs=900000000, feat_len=128,
               classes=172, train_frac=0.011, batch=8000, fanout=[25, 10], cache_frac=0.2, codec="int8"),
    "mid-int8": dict(name="mid RMAT, int8 cache", n_nodes=8000000, n_pairs=64000000, feat_len=128, classes=172,
                     train_frac=0.05, batch=8000, fanout=[25, 10], cache_frac=0.2, codec="int8"),
    "mid-e4m3": dict(name="mid RMAT, fp8 e4m3 cache", n_nodes=8000000, n_pairs=64000000, feat_len=128, classes=172,
                     train_frac=0.05, batch=8000, fanout=[25, 10], cache_frac=0.2, codec="e4m3"),
    # compressed rows in the host table too: a miss moves 144 instead of 512 bytes over the host link
    "c4h": dict(name="paper100M-shaped RMAT, int8 cache and int8 host table", n_nodes=111059956, n_pairs=900000000,
                feat_len=128, classes=172, train_frac=0.011, batch=8000, fanout=[25, 10], cache_frac=0.2, codec="int8",
                host_codec=True),
    "mid-int8-host": dict(name="mid RMAT, int8 cache and int8 host table", n_nodes=8000000, n_pairs=64000000,
                          feat_len=128, classes=172, train_frac=0.05, batch=8000, fanout=[25, 10], cache_frac=0.2,
                          codec="int8", host_codec=True),
    # dynamic-LRU stress (configs[4]) scaled 1:25 so that the host table (10 GB) fits any box: Zipf(1.1)
    # seeds, three hops, set-associative LRU cache of 10% of the table
    "c5s": dict(name="LRU stress RMAT (configs[4] scaled 1:25)", n_nodes=20000000, n_pairs=80000000, feat_len=128,
                classes=172, train_frac=0.0, batch=4096, fanout=[15, 10, 5], cache_frac=0.1, lru_ways=8,
                zipf=1.1, zipf_batches=160),
    # reduced copy of c2 for checking the harness itself on small machines (never the default)
    "tiny": dict(name="tiny RMAT (harness check)", n_nodes=200000, n_pairs=2000000, feat_len=128, classes=172,
                 train_frac=0.2, batch=2000, fanout=[25, 10], cache_frac=0.2),
}


# dram__bytes_read.sum + dram__bytes_write.sum of gather_vec_kernel per row served from GPU memory, from the
# profiler capture of the "mid" config summarised in profiles/gather_kernels_mid_config.md
NCU_DRAM_BYTES_PER_HIT_ROW = 811


def load_pkg():
    import __graft_entry__ as ge
    return ge._package()


def load_oracle():
    import __graft_entry__ as ge
    return ge._oracle()


class ClockSampler:
    """SM clock and throttle reasons while the timed region runs.  The region is a few milliseconds, so
    the driver library is polled from a thread (a sample every millisecond or so); when it cannot be
    loaded, `nvidia-smi -lms` stands in, which manages a sample per 100 ms."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")
    # bits of the driver's clocks-event-reasons mask
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


def host_buffer(n_bytes, shared_name, rank, world, dev=0, fill=None):
    """uint8 buffer in host memory that every rank's GPU can read: pinned (one rank) or one POSIX shared
    segment that rank 0 creates and populates (`fill(buffer)`, else zeros) and every rank page-locks."""
    import torch
    if world == 1:
        t = torch.empty(n_bytes, dtype=torch.uint8, pin_memory=True)
        if fill is not None:
            fill(t)
        return t
    import torch.distributed as dist
    L = load_pkg()
    path = "/dev/shm/" + shared_name
    if rank == 0:
        t = torch.from_file(path, shared=True, size=n_bytes, dtype=torch.uint8)
        if fill is not None:
            fill(t)
        else:
            t.zero_()
    dist.barrier()
    if rank != 0:
        t = torch.from_file(path, shared=True, size=n_bytes, dtype=torch.uint8)
    try:
        L.host_register(dev, t)
    except L.LegionError as e:
        # the driver would not page-lock the shared segment: every rank keeps a pinned copy of its own
        print("rank %d: %s; falling back to a private pinned copy" % (rank, e), file=sys.stderr, flush=True)
        own = torch.empty(n_bytes, dtype=torch.uint8, pin_memory=True)
        own.copy_(t)
        t = own
    dist.barrier()
    if rank == 0:
        os.unlink(path)  # the mappings stay valid
    return t


def host_table(cfg, shared_name=None, rank=0, world=1, dev=0):
    """[N, F] fp32 table in host memory, filled by rank 0; pinned / registered for zero-copy reads."""
    import torch
    from legion_ibp_b200 import synth
    n, f = cfg["n_nodes"], cfg["feat_len"]
    fill = lambda b: synth.features_into(b.view(torch.float32).view(n, f), seed=0)
    return host_buffer(n * f * 4, shared_name, rank, world, dev, fill).view(torch.float32).view(n, f)


def host_link_peak(table):
    """GB/s of a plain pinned host -> device copy, the ceiling for zero-copy reads of the host table."""
    import torch
    n = min(table.numel(), 1 << 28)  # 1 GiB of fp32
    src = table.view(-1)[:n]
    dst = torch.empty(n, dtype=table.dtype, device="cuda")
    for _ in range(2):
        dst.copy_(src, non_blocking=True)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    for _ in range(3):
        dst.copy_(src, non_blocking=True)
    b.record()
    torch.cuda.synchronize()
    return 3 * n * 4 / (a.elapsed_time(b) * 1e-3) / 1e9


def host_rows_seeds_first(order, seeds, n_cached):
    """row_of[id] for a host table that holds, in this order: the uncached seed nodes, the other
    uncached nodes by falling degree, and last the nodes whose rows live in the GPU caches (read once,
    at fill time).  The synthetic table is random, so it can be taken to be in this order already."""
    import torch
    n = order.numel()
    rank_of = torch.empty(n, dtype=torch.int64, device=order.device)
    rank_of[order.long()] = torch.arange(n, dtype=torch.int64, device=order.device)
    cls = torch.ones(n, dtype=torch.int64, device=order.device)
    cls[seeds.long()] = 0
    cls[order[:min(n, n_cached)].long()] = 2
    perm = torch.argsort(cls * n + rank_of)
    del cls, rank_of
    row_of = torch.empty(n, dtype=torch.int32, device=order.device)
    row_of[perm] = torch.arange(n, dtype=torch.int32, device=order.device)
    return row_of


def zipf_batches(n_nodes, batch, n_batches, s, world=1, rank=0):
    """Seed sequence of one rank for the LRU stress workload: Zipf(s) draws over node id, those with
    id % world == rank, made distinct inside every window of `batch` seeds (a mini-batch holds a node once)."""
    import torch
    from legion_ibp_b200 import synth
    draws = synth.zipf_seeds(n_nodes, 4 * batch * n_batches * world, s=s, seed=0, device="cuda")
    draws = draws[(draws % world) == rank]
    assert draws.numel() >= 3 * batch * n_batches
    draws = draws[:3 * batch * n_batches].view(n_batches, 3 * batch)
    out = []
    for i in range(n_batches):
        row = draws[i].long()
        first = torch.full((n_nodes,), 1 << 40, dtype=torch.int64, device=row.device)
        first.scatter_reduce_(0, row, torch.arange(row.numel(), device=row.device), reduce="amin")
        keep = first[row] == torch.arange(row.numel(), device=row.device)
        uniq = row[keep][:batch]
        assert uniq.numel() == batch, "not enough distinct Zipf draws for a batch"
        out.append(uniq.to(torch.int32))
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


def run_reference(args, cfg):
    """CPU arm: the DGL CPU pipeline restated in oracle/ (sample -> relabel -> gather), one batch
    per host thread, on the same synthetic workload."""
    import numpy as np
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
    labels, train, _, _ = synth.labels_and_split(cfg["n_nodes"], cfg["classes"], cfg["train_frac"], device=dev)
    train = train.cpu().numpy()
    tl = labels.cpu().numpy()[train]
    table = torch.empty((cfg["n_nodes"], cfg["feat_len"]), dtype=torch.float32)
    synth.features_into(table, seed=0)
    table = table.numpy()
    if dev == "cuda":
        torch.cuda.empty_cache()
    cores = O.num_threads()
    batch, fanout = cfg["batch"], cfg["fanout"]
    per_step = cores  # one batch per thread and step
    n_iters = (len(train) - 1) // batch
    it = 0
    for _ in range(args.warmup):
        O.cpu_pipeline(indptr, indices, train, tl, batch, it % max(1, n_iters - per_step), per_step, fanout, 1, table, cores)
        it += per_step
    t0 = time.perf_counter()
    for _ in range(args.steps):
        O.cpu_pipeline(indptr, indices, train, tl, batch, it % max(1, n_iters - per_step), per_step, fanout, 1, table, cores)
        it += per_step
    dt = time.perf_counter() - t0
    value = args.steps * per_step / dt
    line = {"impl": "reference", "metric": "sampled+gathered mini-batches/sec", "value": value, "unit": "batches/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(cfg, args.gpus),
            "cpu_baseline": {"value": value, "unit": "batches/s", "cores": cores, "kind": "port",
                             "sample": "%d batches per step (one per thread), %d steps" % (per_step, args.steps)},
            "e2e": {"value": value, "unit": "batches/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def workload_config(cfg, n_gpus):
    if cfg.get("lru_ways"):
        kind = "%d-way set-associative LRU cache of %d%% of the table per GPU, Zipf(%.1f) seeds" % (
            cfg["lru_ways"], int(cfg["cache_frac"] * 100), cfg.get("zipf", 0.0))
    elif cfg.get("codec", "raw") != "raw":
        kind = "static degree-ordered %s cache (codes + fp32 row scale) in %d%% of the table's bytes per GPU" % (
            cfg["codec"], int(cfg["cache_frac"] * 100))
        if cfg.get("host_codec"):
            kind += ", host table held as the same compressed rows"
    else:
        kind = "static %s-ordered cache %d%% of the table per GPU" % (cfg.get("cache_order", "degree"),
                                                                    int(cfg["cache_frac"] * 100))
    return {"workload": "%s: %d nodes, fp32 dim %d, batch %d, fanout %s, %s, misses by zero-copy from pinned host "
                        "memory" % (cfg["name"], cfg["n_nodes"], cfg["feat_len"], cfg["batch"], cfg["fanout"], kind),
            "batch_per_gpu": cfg["batch"], "fanout": cfg["fanout"], "feat_len": cfg["feat_len"],
            "parallelism": "dp%d, cache striped over %d GPU(s)" % (n_gpus, n_gpus),
            "l2": "inputs larger than L2 (topology, cache partition and host table are each GBs)"}



def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="c2", choices=sorted(CONFIGS))
    ap.add_argument("--cpu-sample-batches", type=int, default=0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cache-frac", type=float, default=None, help="override the cached fraction of the table")
    ap.add_argument("--pipes", type=int, default=2, help="batches in flight (the hand-off protocol uses 2)")
    ap.add_argument("--host-layout", default="seeds_first", choices=["id", "seeds_first"],
                    help="row order of the pinned host table: node-id order, or uncached seed nodes first and the "
                         "other uncached nodes by falling degree (shorter spans for the zero-copy misses)")
    ap.add_argument("--no-replicas", action="store_true",
                    help="N > 1: stripe the whole per-GPU budget over the clique (the reference's placement) instead "
                         "of planning private copies of the hottest peer rows")
    ap.add_argument("--cache-order", default="degree", choices=["degree", "hotness", "seeds_degree"],
                    help="ranking behind the static cache: node degree (what the configs name); the reference's own "
                         "policy, access counts of one presampled epoch (engine/server.cu:94-122); or the training "
                         "seeds (every one of them is read once per epoch) followed by the other nodes by degree")
    ap.add_argument("--e2e-outputs", default="bound", choices=["bound", "copy", "none"],
                    help="e2e leg: block structure written by the batch into page-locked arrays named at submit "
                         "time (default), copied out by collect after the batch (two batches in flight), or not "
                         "moved at all (diagnostic)")
    ap.add_argument("--tunable", action="append", default=[], metavar="NAME=VALUE",
                    help="launch-shape knob passed to legion_set_tunable (measurement sweeps)")
    ap.add_argument("--profile-only", action="store_true",
                    help="set-up, warm-up and the timed steps only (for runs under a profiler); prints no bench line")
    args = ap.parse_args()
    cfg = dict(CONFIGS[args.config])
    if args.cache_frac is not None:
        cfg["cache_frac"] = args.cache_frac
    cfg["cache_order"] = args.cache_order
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
    torch.cuda.set_device(local_rank)
    dev = local_rank
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    t_setup = time.perf_counter()

    # ---- synthetic inputs -------------------------------------------------------------------
    indptr, indices = make_graph(cfg, "cuda")
    torch.cuda.empty_cache()
    n, f = cfg["n_nodes"], cfg["feat_len"]
    row_bytes = f * 4
    n_edges = int(indices.numel())
    labels, train, _, _ = synth.labels_and_split(n, cfg["classes"], max(cfg["train_frac"], 1e-6), device="cuda")
    if cfg.get("zipf"):
        train = zipf_batches(n, cfg["batch"], cfg["zipf_batches"], cfg["zipf"], world, rank)
    mine = train[(train % world) == rank].contiguous()  # id % ngpu split, storage_management.cu:214-250
    mine_labels = labels[mine.long()].contiguous()
    table = host_table(cfg, "legion_b200_bench_features", rank, world, dev)

    # ---- storage, cache, pool, runner ------------------------------------------------------------
    g = L.GraphStorage(dev, indptr, indices)
    fs = L.FeatureStorage(dev, n, row_bytes, table)
    fs.set_split(L.TRAINMODE, mine, mine_labels)
    order = torch.empty(n, dtype=torch.int32, device="cuda")
    counts = None
    if args.cache_order == "hotness":
        # PreSc: one epoch of sampling only, every touched node counted; counts of all ranks added up
        pre_pool = L.MemoryPool(dev, cfg["batch"], cfg["fanout"], row_bytes, 2)
        pre_pool.set_rng(0xC0FFEE + rank, 64)  # not the measured runs' stream: those batches must be new to the cache
        pre = L.Runner(dev, g, fs, None, pre_pool, None)
        counts = torch.zeros(n, dtype=torch.int32, device="cuda")
        pre.presample(0, max(1, (int(mine.numel()) - 1) // cfg["batch"]), counts)
        torch.cuda.synchronize()
        pre.Finalize()
        pre_pool.close()
        if dist is not None:
            dist.all_reduce(counts)
        L.UnifiedCache.hotness_order(dev, counts, order)
    else:
        L.UnifiedCache.degree_order(dev, indptr, order)
        if args.cache_order == "seeds_degree":
            is_seed = torch.zeros(n, dtype=torch.bool, device="cuda")
            is_seed[train.long()] = True
            first = is_seed[order.long()]
            order = torch.cat([order[first], order[~first]]).contiguous()
            del is_seed, first
    codec_name = cfg.get("codec", "raw")
    codec = {"raw": L.CODEC_RAW, "int8": L.CODEC_INT8, "e4m3": L.CODEC_E4M3}[codec_name]
    slot_bytes = row_bytes if codec == L.CODEC_RAW else (f + 4 + 15) // 16 * 16
    budget = cap = min(n, int(n * cfg["cache_frac"] * row_bytes / slot_bytes))
    replica_rows = 0
    if cap * world >= n:
        cap = (n + world - 1) // world
    row_of = None
    stored = None  # compressed copy of the host table (configs with host_codec)

    def barrier0():
        if dist is not None:
            dist.barrier()

    lru_ways = cfg.get("lru_ways", 0)
    if lru_ways:
        # every GPU keeps its own LRU cache (no clique: the contents change every batch)
        cap = cap // lru_ways * lru_ways
        cache = L.UnifiedCache(dev, n, row_bytes, 0, lru=(cap // lru_ways, lru_ways))
        cache.set_host_table(table)
        args.host_layout = "id"
    else:
        if cfg.get("host_codec"):
            stored = host_buffer(n * slot_bytes, "legion_b200_bench_codes", rank, world, dev).view(n, slot_bytes)
            if rank == 0:
                L.quantize_table(dev, codec, table, n, f, stored)
            barrier0()
        if world > 1 and not args.no_replicas:
            from legion_ibp_b200 import server
            mass = server.degree_mass(indptr, order) if counts is None else server.weight_mass(counts, order)
            cap, replica_rows = server.plan_clique_cache(mass, n, budget, world)
            del mass
        cache = L.UnifiedCache(dev, n, row_bytes, cap, kg=world, ki=rank, codec=codec)
        if args.host_layout == "seeds_first":
            row_of = host_rows_seeds_first(order, train, cap * world)
        if stored is not None:
            cache.set_host_codec(codec)
        cache.fill_static(order, table if stored is None else stored, row_of_id=row_of)
        if replica_rows > 0:
            cache.add_replicas(order, replica_rows, row_of_id=row_of)
    del order, counts
    share = None
    if world > 1 and not lru_ways:
        from legion_ibp_b200 import server
        share = server.exchange_partitions(cache, rank, world, dist)
    pool = L.MemoryPool(dev, cfg["batch"], cfg["fanout"], row_bytes, args.pipes)
    pool.set_rng(0x5EED + rank, 64)
    runner = L.Runner(dev, g, fs, cache, pool, None)
    n_iters = (int(mine.numel()) - 1) // cfg["batch"]
    torch.cuda.synchronize()
    setup_s = time.perf_counter() - t_setup

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

    # ---- value: inputs resident, device-timed ----------------------------------------------------
    step = 0
    for _ in range(args.warmup):
        runner.enqueue(step, L.TRAINMODE, step % n_iters)
        step += 1
    runner.sync()
    # full-size spot check: gathered rows of the last warm-up batch are bit copies of their host rows
    last_pipe = (step - 1) % args.pipes
    nc_chk = pool.read(L.BUF_NODE_COUNTER, last_pipe, 16, np.int32)
    n_chk = int(nc_chk[9 + int(nc_chk[8])])
    ids_chk = torch.from_numpy(pool.read(L.BUF_IDS, last_pipe, n_chk, np.int32))
    pick = torch.randint(0, n_chk, (min(2000, n_chk),))
    fptr, _ = pool.buffer(L.BUF_FEATURES, last_pipe)
    rows_chk = np.empty((n_chk, f), np.float32)
    import ctypes
    L._check(L.lib().legion_copy(ctypes.c_void_p(rows_chk.ctypes.data), ctypes.c_void_p(fptr), ctypes.c_int64(rows_chk.nbytes),
                                 ctypes.c_int32(2)))
    src_rows = ids_chk[pick].long() if row_of is None else row_of.cpu()[ids_chk[pick].long()].long()
    want_rows = table[src_rows].numpy()
    if codec == L.CODEC_RAW:
        assert np.array_equal(rows_chk[pick.numpy()], want_rows), "gathered rows differ from the host table"
    else:
        # rows served by the compressed cache: |x - x^| <= absmax / 254 for int8 (half a code step);
        # half an e4m3 step (2^-4 relative) of the scaled value for fp8
        amax = np.abs(want_rows).max(axis=1, keepdims=True)
        tol = amax / 254.0 * 1.001 if codec == L.CODEC_INT8 else np.maximum(np.abs(want_rows) / 16.0, amax / 448.0 / 1024.0) * 1.001
        assert np.all(np.abs(rows_chk[pick.numpy()] - want_rows) <= tol), "dequantised rows out of tolerance"
    del rows_chk
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(args.steps):
        runner.enqueue(step, L.TRAINMODE, step % n_iters)
        step += 1
    runner.sync()
    barrier()
    ms_total = max_over_ranks(runner.timing()["batch_ms"])
    value = args.steps * world / (ms_total * 1e-3)
    assert pool.device_error() == 0, "device-side error flag set"

    # ---- kernel durations: the same graph replay with CUDA events around the gather launches, one
    # batch at a time (the events of a pipe's graph are overwritten by its next launch) ----------------
    runner.set_options(use_graph=True, time_kernels=True)
    for _ in range(2):
        runner.enqueue(step, L.TRAINMODE, step % n_iters)
        step += 1
    runner.sync()
    stats0 = cache.stats()
    tm = {"gather_ms": 0.0, "miss_ms": 0.0, "timed": 0}
    for _ in range(args.steps):
        runner.enqueue(step, L.TRAINMODE, step % n_iters)
        step += 1
        runner.sync()
        t1 = runner.timing()
        for k in tm:
            tm[k] += t1[k]
    stats1 = cache.stats()
    # the same events with batches in flight: how busy the host-link stream is in steady state
    for _ in range(args.steps):
        runner.enqueue(step, L.TRAINMODE, step % n_iters)
        step += 1
    runner.sync()
    tp = runner.timing()
    pipeline = {"window_ms_per_batch": tp["batch_ms"] / args.steps, "miss_ms_per_batch": tp["miss_ms"] / args.steps,
                "miss_stream_busy_frac": tp["miss_ms"] / tp["batch_ms"] if tp["batch_ms"] > 0 else None}
    runner.set_options(use_graph=True, time_kernels=False)
    # the timed region is a few milliseconds: the clock samples run on through the kernel-timing passes
    # above, which replay the same batches
    clocks = sampler.stop() if rank == 0 else None
    if args.profile_only:
        if rank == 0:
            print(json.dumps({"profile_only": True, "ms_per_step": ms_total / args.steps, "value": value}), flush=True)
        runner.Finalize()
        return

    # ---- roofline of the gather ---------------------------------------------------------------------
    # Algorithmic bytes per gathered row: the row read from its source + the row written + 4 B id +
    # 4 B lookup-table entry.  Rows served from GPU memory are moved by the hit kernel (HBM bound);
    # rows that miss the cache are moved by the miss kernel over the host link, for which the hit
    # kernel still reads id + table entry and writes an 8-byte list entry.
    d = {k: stats1[k] - stats0[k] for k in stats0}
    hits = d["local_hits"] + d["peer_hits"]
    rows = hits + d["misses"]
    gather_launches = tm["timed"]  # one lookup + gather launch per batch
    # a hit reads its cache slot (the raw row; codes + scale; for the LRU cache also the keys of its set
    # and one stamp) and writes the fp32 row
    hit_read = slot_bytes + (4 * lru_ways + 4 if lru_ways else 0)
    hit_bytes = hits * (hit_read + row_bytes + 8) + d["misses"] * 16
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
    # DRAM bytes per launch: the full-size workload is too large for a multi-pass profiler capture, so the
    # figure of the captured "mid" case (profiles/gather_kernels_mid_config.md: dram read + write bytes per
    # row served from GPU memory) is scaled by the rows one launch serves here; raw 512-byte rows only
    traffic = traffic_source = None
    if codec == L.CODEC_RAW and not lru_ways and row_bytes == 512 and world == 1:
        traffic = NCU_DRAM_BYTES_PER_HIT_ROW * hits / max(1, gather_launches)
        traffic_source = ("ncu dram__bytes_read.sum + dram__bytes_write.sum of the mid config (%d B per row served "
                          "from GPU memory; part of the written rows is still in L2 when the kernel ends), scaled "
                          "by the rows per launch" % NCU_DRAM_BYTES_PER_HIT_ROW)
    kname = ("gather_lru_kernel (set probe + gather of rows held in the LRU cache)" if lru_ways else
             "gather_quant_kernel<%s> (cache lookup + gather with in-kernel dequantisation)" % codec_name
             if codec != L.CODEC_RAW else "gather_vec_kernel (cache lookup + gather of rows held in GPU memory)")
    roofline = {"bound": "hbm", "kernel": kname,
                "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                "peak_source": "of measured (MEASURED_PEAKS.json hbm_gbs)" if peaks else "of fallback 6650 GB/s",
                "traffic": traffic, "traffic_source": traffic_source, "launches": gather_launches,
                "avg_launch_ms": tm["gather_ms"] / max(1, gather_launches),
                "rows_per_batch": rows / args.steps,
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
                           "peer_rows_per_batch": d["peer_hits"] / args.steps}
    # one rank at a time: the ranks' host links share the host's memory and root ports
    link_peak = 0.0
    for k in range(world):
        if k == rank:
            link_peak = host_link_peak(table)
        barrier()
    link_achieved = d["misses"] * host_row_bytes / miss_s / 1e9 if miss_s > 0 else 0.0
    roofline_host = {"bound": "host_link", "kernel": "gather_miss_kernel (zero-copy fetch of missed rows)",
                     "achieved": link_achieved, "peak": link_peak, "unit": "GB/s",
                     "frac": link_achieved / link_peak if link_peak else None,
                     "peak_source": "pinned host->device cudaMemcpy of 1 GiB measured in this run (the same kernel "
                                    "alone reaches 50.6 GB/s on random rows of a 1 GB table and 26 GB/s over 48 GB)",
                     "launches": tm["timed"], "avg_launch_ms": tm["miss_ms"] / max(1, tm["timed"]),
                     "rows_per_batch": d["misses"] / args.steps, "algorithmic_bytes": miss_bytes}
    # lower bound of the whole gather step: the slowest of the HBM side, the NVLink side and the host-link side
    t_lb = max(hit_bytes / (hbm_peak * 1e9), d["peer_hits"] * slot_bytes / 770e9,
               d["misses"] * host_row_bytes / (link_peak * 1e9) if link_peak else 0.0)
    roofline_path = {"lower_bound_ms_per_batch": t_lb / args.steps * 1e3,
                     "gather_ms_per_batch": (tm["gather_ms"] + tm["miss_ms"]) / max(1, tm["timed"]),
                     "batch_ms": ms_total / args.steps}

    # ---- e2e: host buffers through the C ABI --------------------------------------------------------
    max_nodes, max_edges = bounds(cfg["batch"], cfg["fanout"])
    seeds_h = mine.cpu().numpy()
    labels_h = mine_labels.cpu().numpy()
    # one set of page-locked output arrays per batch in flight; the batch itself writes into them
    outs = [dict(ids=torch.empty(max_nodes, dtype=torch.int32).pin_memory().numpy(),
                 lab=torch.empty(cfg["batch"], dtype=torch.int32).pin_memory().numpy(),
                 src=torch.empty(max_edges, dtype=torch.int32).pin_memory().numpy(),
                 dst=torch.empty(max_edges, dtype=torch.int32).pin_memory().numpy()) for _ in range(3)]
    nc_o, ec_o = np.zeros(16, np.int32), np.zeros(16, np.int32)
    b = cfg["batch"]

    mode = args.e2e_outputs

    def submit(i):
        it = i % n_iters
        o = outs[i % 3]
        if mode == "bound":
            runner.submit_host_to(seeds_h[it * b:(it + 1) * b], labels_h[it * b:(it + 1) * b], i, o["ids"], o["lab"],
                                  o["src"], o["dst"])
        else:
            runner.submit_host(seeds_h[it * b:(it + 1) * b], labels_h[it * b:(it + 1) * b], i)

    def collect():
        if mode == "copy":
            o = outs[0]
            return runner.collect_host(o["ids"], o["lab"], o["src"], o["dst"], nc_o, ec_o, None)
        return runner.collect_host(None, None, None, None, nc_o, ec_o, None)

    # two batches in flight plus, for static caches, a third that samples ahead (the API's limit); a
    # batch counts as done when its collect returns
    depth = 3 if (mode == "bound" and not lru_ways) else 2
    pipe0 = runner.current_pipe()
    for i in range(depth):
        submit(i)
    for i in range(depth, depth + 4):
        collect()
        submit(i)
    for _ in range(depth):
        collect()
    # the exported block structure of the last batch is what the device buffers hold
    last = depth + 3
    nn_chk, ne_chk = runner_counts(nc_o, ec_o)
    chk_pipe = (pipe0 + last) % 2
    if mode != "none":
        o_chk = outs[last % 3] if mode == "bound" else outs[0]
        assert np.array_equal(o_chk["ids"][:nn_chk], pool.read(L.BUF_IDS, chk_pipe, nn_chk, np.int32))
        assert np.array_equal(o_chk["src"][:ne_chk], pool.read(L.BUF_AGG_SRC, chk_pipe, ne_chk, np.int32))
    # wall clock needs a longer window than the device-timed leg: 40 steps of 0.2 ms are 8 ms, which one
    # descheduled rank out of eight distorts; the steps are the same steps
    e2e_steps = max(args.steps, 200)
    barrier()
    t0 = time.perf_counter()
    d2h = 0
    for i in range(depth):
        submit(100 + i)
    for i in range(depth, e2e_steps):
        nn, ne = collect()
        d2h += 4 * nn + 8 * ne + 4 * b + 128
        submit(100 + i)
    for _ in range(depth):
        nn, ne = collect()
        d2h += 4 * nn + 8 * ne + 4 * b + 128
    torch.cuda.synchronize()
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    barrier()
    e2e = {"value": e2e_steps * world / e2e_s, "unit": "batches/s", "h2d_bytes_per_step": 8 * b,
           "d2h_bytes_per_step": d2h // e2e_steps, "steps": e2e_steps,
           "api": "legion_runner_submit_host%s / legion_runner_collect_host, %d batches in flight, outputs: %s" % (
               "_to" if mode == "bound" else "", depth, mode),
           "note": "seeds+labels copied in from host memory, ids/labels/edge lists/counters written to page-locked host "
                   "memory every step; gathered rows stay in the device hand-off buffer where the trainer reads "
                   "them; missed rows cross the host link inside the gather"}

    # ---- CPU baseline on this box's cores (rank 0, N=1 only) ----------------------------------------
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        O = load_oracle()
        cores = O.num_threads()
        nb = args.cpu_sample_batches or 2 * cores
        h_indptr, h_indices = indptr.cpu().numpy(), indices.cpu().numpy()
        tnp = table.numpy()
        O.cpu_pipeline(h_indptr, h_indices, seeds_h, labels_h, b, 0, cores, cfg["fanout"], 1, tnp, cores)
        t0 = time.perf_counter()
        O.cpu_pipeline(h_indptr, h_indices, seeds_h, labels_h, b, cores, nb, cfg["fanout"], 1, tnp, cores)
        dt = time.perf_counter() - t0
        cpu = {"value": nb / dt, "unit": "batches/s", "cores": cores, "kind": "port",
               "sample": "%d batches of the same workload (sample + relabel + gather), %d threads, %.1f s" %
                         (nb, cores, dt)}

    if rank == 0:
        hops = len(cfg["fanout"])
        line = {"metric": "sampled+gathered mini-batches/sec", "value": value, "unit": "batches/s",
                "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": dict(workload_config(cfg, world), host_table_layout=args.host_layout),
                "e2e": e2e, "gpu_launches": args.steps * (1 + 4 * hops + 1 + 1 + (3 if lru_ways else 0)),
                "roofline": roofline, "roofline_host_link": roofline_host, "roofline_path": roofline_path, "roofline_nvlink": roofline_nvlink,
                "pipeline": pipeline,
                "cpu_baseline": cpu, "clocks": clocks,
                "graph": {"nodes": n, "directed_edges": n_edges, "train_seeds_this_rank": int(mine.numel()),
                          "cache_rows_per_gpu": cap, "replica_rows_per_gpu": replica_rows,
                          "peer_mapping": share}, "setup_s": setup_s, "tunables": args.tunable or None}
        print(json.dumps(line), flush=True)
    runner.Finalize()
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
