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


SERVER_CLIENT = textwrap.dedent(r'''
    import os, sys, ctypes as C
    import numpy as np
    sys.path.insert(0, os.path.join(sys.argv[1], "tests"))
    import conftest
    import legion_ibp_b200 as L
    dev, shm, total, feat_len, out_path = int(sys.argv[2]), sys.argv[3], int(sys.argv[4]), int(sys.argv[5]), sys.argv[6]
    import torch
    torch.cuda.set_device(dev)
    svc = L.ipc_service(dev, shm)
    def d2h(ptr, count, dtype):
        out = np.empty(count, dtype)
        if out.nbytes:
            L._check(L.lib().legion_copy(C.c_void_p(out.ctypes.data), C.c_void_p(ptr), C.c_int64(out.nbytes), C.c_int32(2)))
        return out
    res = {}
    for b in range(total):
        v = svc.get_next(timeout_ms=120000)
        res["ids%d" % b] = d2h(v.ids, v.n_ids, np.int32)
        res["feat%d" % b] = d2h(v.features, v.n_ids * feat_len, np.float32)
        res["nc%d" % b] = np.array(v.node_counter[:], np.int32)
        res["ec%d" % b] = np.array(v.edge_counter[:], np.int32)
        svc.synchronize()
    svc.finalize()
    np.savez(out_path, **res)
''')


@pytest.mark.parametrize("no_vmm", [False, True])
def test_server_binary_on_two_gpus_plans_replicas_and_stages_seeds(oracle_mod, tmp_path, no_vmm):
    """`sampling_server 2 0 0`: one thread per GPU, the per-GPU budget planned into stripe + private copies,
    peers read in place (shareable memory, or plain allocations with peer access when the platform has no
    virtual memory management), seed rows staged for the copy engine; two trainer processes, one per GPU,
    compare every batch with the host replay."""
    import select
    import time
    import numpy as np
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from test_dataset_cpu import meta_for, write_dataset
    feat_len, batch, seed = 16, 32, 11
    ref = write_dataset(tmp_path / "ds", n=6000, f=feat_len, seed=13)
    meta = meta_for(tmp_path / "ds", ref, f=feat_len)
    meta.raw_batch_size = batch
    meta.epoch = 1
    meta.cache_memory = feat_len * 4 * 1500
    meta.write(str(tmp_path / "meta_config"))
    shm = "legion_b200_srv2_%d_%d" % (os.getpid(), int(no_vmm))
    # the run with plain allocations also ranks by presampled hotness (the reference's policy): every GPU must then
    # rank by the access counts of ALL GPUs, or the members of the clique would disagree on where a row lives
    env = dict(os.environ, LEGION_SHM_NAME=shm, LEGION_ORDER="hotness" if no_vmm else "degree", LEGION_SEED=str(seed),
               LEGION_TIMEOUT_MS="120000")
    if no_vmm:
        env["LEGION_NO_VMM"] = "1"
    binary = os.path.join(ROOT, "legion-ibp_b200", "sampling_server")
    server = subprocess.Popen([binary, "2", "0", "0"], cwd=str(tmp_path), env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    clients = []
    try:
        seen, deadline = b"", time.time() + 180
        while b"System is ready for serving" not in seen:
            assert time.time() < deadline and server.poll() is None, seen.decode()[-2000:]
            if select.select([server.stdout], [], [], 1.0)[0]:
                seen += os.read(server.stdout.fileno(), 4096)
        assert b"private copies" in seen and b"Seed rows staged" in seen, seen.decode()[-2000:]
        train, valid, test = ref["train"], ref["valid"], ref["test"]
        parts = [[ids[ids % 2 == g] for ids in (train, valid, test)] for g in range(2)]
        steps, vbs, tbs = oracle_mod.coordinate([len(p[0]) for p in parts], [len(p[1]) for p in parts], [len(p[2]) for p in parts], batch)
        total = steps[0] + steps[1] + steps[2]
        script = tmp_path / "client.py"
        script.write_text(SERVER_CLIENT)
        for g in range(2):
            clients.append(subprocess.Popen([sys.executable, str(script), ROOT, str(g), shm, str(total), str(feat_len),
                                             str(tmp_path / ("client%d.npz" % g))], stdout=subprocess.PIPE, stderr=subprocess.STDOUT))
        for c in clients:
            out, _ = c.communicate(timeout=300)
            assert c.returncode == 0, out.decode()[-3000:]
        s_out, _ = server.communicate(timeout=60)
        assert server.returncode == 0, (seen + s_out).decode()[-2000:]
    finally:
        for p in clients + [server]:
            if p.poll() is None:
                p.kill()
    for g in range(2):
        got = np.load(tmp_path / ("client%d.npz" % g))
        lists = {0: (parts[g][0], batch), 1: (parts[g][1], int(vbs[g])), 2: (parts[g][2], int(tbs[g]))}
        for b in range(total):
            mode, local = oracle_mod.mode_of_batch(b, steps[0], steps[1], steps[2], 1)
            ids_all, bs = lists[mode]
            want = oracle_mod.run_batch(ref["indptr"], ref["indices"], ids_all, ref["labels"][ids_all], bs, local, [25, 10], b, seed + g)
            np.testing.assert_array_equal(got["ids%d" % b], want["ids"], err_msg="gpu %d batch %d" % (g, b))
            np.testing.assert_array_equal(got["nc%d" % b], want["node_counter"])
            np.testing.assert_array_equal(got["ec%d" % b], want["edge_counter"])
            np.testing.assert_array_equal(got["feat%d" % b].reshape(len(want["ids"]), -1), ref["feats"][want["ids"]])
