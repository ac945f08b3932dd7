"""Two ranks, one process per GPU (torchrun + NCCL for the start-up exchange only): seeds split by
id % 2, cache striped over both GPUs, partitions exchanged as file descriptors, peer rows read over
NVLink from inside the gather kernel.  Every rank compares its batches with the host replay.
Skipped on a box with one GPU."""
import os
import socket
import subprocess
import sys
import textwrap

import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu

WORKER = textwrap.dedent(r'''
    import os, sys
    import numpy as np
    import torch
    import torch.distributed as dist
    sys.path.insert(0, os.path.join(sys.argv[1], "tests"))
    import conftest
    import legion_ibp_b200 as L
    from legion_ibp_b200 import server
    import oracle as O
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    indptr, indices = conftest.small_graph(20000, 300000, 31)
    n, F = len(indptr) - 1, 128
    rng = np.random.default_rng(0)
    table = rng.standard_normal((n, F)).astype(np.float32)
    train = rng.permutation(n)[:2000].astype(np.int32)
    labels = rng.integers(0, 47, n).astype(np.int32)
    d_ip, d_ix = torch.from_numpy(indptr).cuda(), torch.from_numpy(indices).cuda()
    h_table = torch.from_numpy(table).pin_memory()
    srv = server.Server(dist)
    cap = srv.Initialize(rank, d_ip, d_ix, h_table, F * 4, torch.from_numpy(train).cuda(),
                         torch.from_numpy(labels).cuda(), 64, [25, 10], n // 4)
    srv.PreSc(d_ip, h_table)
    runner = srv.make_runner(64, [25, 10], F * 4, rng_seed=100 + rank)
    mine = train[train % world == rank]
    for it in range(0, 4, 2):
        runner.enqueue(it, L.TRAINMODE, it)
        runner.enqueue(it + 1, L.TRAINMODE, it + 1)
        runner.sync()
        for pipe in (0, 1):
            ref = O.run_batch(indptr, indices, mine, labels[mine], 64, it + pipe, [25, 10], it + pipe, 100 + rank)
            ids = srv.pool.read(L.BUF_IDS, pipe, len(ref["ids"]), np.int32)
            assert (ids == ref["ids"]).all()
            assert (srv.pool.read(L.BUF_AGG_SRC, pipe, len(ref["agg_src"]), np.int32) == ref["agg_src"]).all()
            feat = srv.pool.read(L.BUF_FEATURES, pipe, len(ids) * F, np.float32).reshape(-1, F)
            assert (feat == table[ref["ids"]]).all()
    st = srv.cache.stats()
    assert st["peer_hits"] > 0 and st["local_hits"] > 0 and st["misses"] > 0, st
    assert srv.pool.device_error() == 0
    dist.barrier()
    srv.Finalize()
    dist.destroy_process_group()
    print("rank %d ok %s" % (rank, st))
''')


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def test_two_ranks_share_a_striped_cache(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(_free_port()), str(script), ROOT]
    r = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, timeout=600)
    out = r.stdout.decode()
    assert r.returncode == 0, out[-4000:]
    assert "rank 0 ok" in out and "rank 1 ok" in out
