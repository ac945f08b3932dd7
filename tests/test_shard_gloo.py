"""The one-process-per-GPU start-up exchange with two gloo ranks on the CPU: seed split,
count gathering for the step arithmetic, fixed-size handle exchange, cache planning."""
import os
import socket
import subprocess
import sys
import textwrap

import numpy as np

from conftest import ROOT

WORKER = textwrap.dedent(r'''
    import os, sys, json
    import numpy as np
    import torch
    import torch.distributed as dist
    sys.path.insert(0, os.path.join(sys.argv[1], "tests"))
    import conftest
    from legion_ibp_b200 import server
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    g = torch.Generator().manual_seed(0)
    train = torch.randperm(10000, generator=g)[:1237].to(torch.int32)
    mine = server.split_seeds(train, world, rank)
    counts = server.all_gather_ints([int(mine.numel()), 11 + rank, 7], dist)
    blob = bytes([rank] * 64)
    blobs = server.all_gather_bytes(blob, dist)
    out = dict(rank=rank, world=world, mine=mine.tolist(), counts=counts, blobs=[list(b[:2]) for b in blobs],
               cap=[server.plan_cache_rows(1000, 200, world), server.plan_cache_rows(1000, 600, world),
                    server.plan_cache_rows(1001, 5000, world)])
    json.dump(out, open(sys.argv[2] + ".%d" % rank, "w"))
    dist.barrier()
    dist.destroy_process_group()
''')


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def test_two_rank_startup_exchange(tmp_path):
    import json
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    out = str(tmp_path / "out.json")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), str(script), ROOT, out]
    env = dict(os.environ, OMP_NUM_THREADS="1")
    r = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, timeout=300)
    assert r.returncode == 0, r.stdout.decode()[-3000:]
    res = [json.load(open(out + ".%d" % k)) for k in range(2)]
    import torch
    g = torch.Generator().manual_seed(0)
    train = torch.randperm(10000, generator=g)[:1237].numpy()
    # the split is by id % world, keeps list order, and is a partition of the seed list
    for k in range(2):
        np.testing.assert_array_equal(res[k]["mine"], train[train % 2 == k])
        assert res[k]["world"] == 2 and res[k]["rank"] == k
    assert sorted(res[0]["mine"] + res[1]["mine"]) == sorted(train.tolist())
    # every rank sees every rank's counts and handles, in rank order
    exp_counts = [[len(res[0]["mine"]), 11, 7], [len(res[1]["mine"]), 12, 7]]
    for k in range(2):
        assert res[k]["counts"] == exp_counts
        assert res[k]["blobs"] == [[0, 0], [1, 1]]
        assert res[k]["cap"] == [200, 500, 501]
