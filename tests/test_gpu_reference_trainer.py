"""The REFERENCE's own trainer-side extension consuming batches from this repository's sampling_server.

oracle/_ref/ipc_service.so is training_backend/ipc_service.cpp + helper_multiprocess.cpp +
ipc_cuda_kernel.cu of the reference, compiled unmodified by oracle/build_ref_trainer.py (where the
reference tree is present; without the built module the test skips).  A second process imports it and
does what training_backend/legion_graphsage.py:87-126 does per step: initialize(), get_steps(), then
get_next(feature_dim) / get_block_size() / synchronize() for every batch of the schedule.  The seven
tensors it returns must equal the CPU checker's batch and the rows of the feature file, bit for bit.
The server runs under the names the extension has compiled in (segment simpleIPCshm, semaphores
sem_r_0_* / sem_w_0_*), started the way the reference starts it.
"""
import glob
import os
import select
import subprocess
import sys
import time

import numpy as np
import pytest

import legion_ibp_b200 as L
from conftest import ROOT

pytestmark = pytest.mark.gpu

EXT = os.path.join(ROOT, "oracle", "_ref", "ipc_service.so")

TRAINER = r'''
import faulthandler, importlib.util, sys, numpy as np, torch
faulthandler.enable()
ext_path, feat_len, total, out_path = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), sys.argv[4]
torch.cuda.set_device(0)
torch.zeros(1, device="cuda")          # the extension expects a live context on the trainer's device
spec = importlib.util.spec_from_file_location("ipc_service", ext_path)
ipc_service = importlib.util.module_from_spec(spec)
spec.loader.exec_module(ipc_service)
print("initialize", flush=True)
ipc_service.initialize()
print("initialized", flush=True)
res = {"steps": np.array(ipc_service.get_steps(), np.int32)}
for b in range(total):
    print("get_next", b, flush=True)
    t = ipc_service.get_next(feat_len)          # ids, features, labels, then (src, dst) per hop, last hop first
    res["blocks%d" % b] = np.array(ipc_service.get_block_size(), np.int32)
    res["n%d" % b] = np.array([len(t)], np.int32)
    for k, x in enumerate(t):
        res["t%d_%d" % (b, k)] = x.cpu().numpy()
    ipc_service.synchronize()
ipc_service.finalize()
np.savez(out_path, **res)
'''


def _clear_stale_names():
    for p in glob.glob("/dev/shm/sem.sem_[rw]_0_*") + glob.glob("/dev/shm/simpleIPCshm*"):
        try:
            os.unlink(p)
        except OSError:
            pass


@pytest.mark.skipif(not os.path.exists(EXT), reason="the reference's trainer extension is not built (needs the reference tree)")
def test_reference_trainer_extension_consumes_served_batches(oracle_mod, tmp_path):
    from test_dataset_cpu import meta_for, write_dataset
    feat_len, batch, fanout, seed = 16, 24, [25, 10], 7
    ref = write_dataset(tmp_path / "ds", n=3000, f=feat_len, seed=9)
    meta = meta_for(tmp_path / "ds", ref, f=feat_len)
    meta.raw_batch_size = batch
    meta.epoch = 1
    meta.cache_memory = feat_len * 4 * 600
    meta.write(str(tmp_path / "meta_config"))
    _clear_stale_names()
    env = dict(os.environ, LEGION_ORDER="degree", LEGION_SEED=str(seed), LEGION_TIMEOUT_MS="120000")
    env.pop("LEGION_SHM_NAME", None)
    binary = os.path.join(ROOT, "legion-ibp_b200", "sampling_server")
    server = subprocess.Popen([binary, "1", "0", "0"], cwd=str(tmp_path), env=env, stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT)
    trainer = None
    try:
        seen, deadline = b"", time.time() + 120
        while b"System is ready for serving" not in seen:
            assert time.time() < deadline and server.poll() is None, seen.decode()[-2000:]
            if select.select([server.stdout], [], [], 1.0)[0]:
                seen += os.read(server.stdout.fileno(), 4096)
        train, valid, test = ref["train"], ref["valid"], ref["test"]
        steps, vbs, tbs = oracle_mod.coordinate([len(train)], [len(valid)], [len(test)], batch)
        total = (steps[0] + steps[1]) * 1 + steps[2]
        script = tmp_path / "trainer.py"
        script.write_text(TRAINER)
        out = tmp_path / "trainer.npz"
        trainer = subprocess.Popen([sys.executable, str(script), EXT, str(feat_len), str(total), str(out)],
                                   stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
        t_out, _ = trainer.communicate(timeout=300)
        assert trainer.returncode == 0, t_out.decode()[-3000:]
        s_out, _ = server.communicate(timeout=60)
        assert server.returncode == 0, (seen + s_out).decode()[-2000:]
        assert b"System finalized" in s_out
    finally:
        for p in (trainer, server):
            if p is not None and p.poll() is None:
                p.kill()
        _clear_stale_names()
    got = np.load(out)
    assert list(got["steps"]) == list(steps)
    lists = {0: (train, batch), 1: (valid, int(vbs[0])), 2: (test, int(tbs[0]))}
    for b in range(total):
        mode, local = oracle_mod.mode_of_batch(b, steps[0], steps[1], steps[2], 1)
        ids_all, bs = lists[mode]
        want = oracle_mod.run_batch(ref["indptr"], ref["indices"], ids_all, ref["labels"][ids_all], bs, local, fanout, b, seed)
        nc, ec = want["node_counter"], want["edge_counter"]
        assert int(got["n%d" % b][0]) == 3 + 2 * len(fanout)        # the 7 tensors legion_graphsage.py unpacks
        np.testing.assert_array_equal(got["t%d_0" % b], want["ids"], err_msg="batch %d mode %d" % (b, mode))
        np.testing.assert_array_equal(got["t%d_1" % b], ref["feats"][want["ids"]])
        np.testing.assert_array_equal(got["t%d_2" % b], want["labels"])
        for j, hop in enumerate(range(len(fanout), 0, -1)):
            lo, cnt = int(ec[12 + hop]), int(ec[9 + hop])
            np.testing.assert_array_equal(got["t%d_%d" % (b, 3 + 2 * j)], want["agg_src"][lo:lo + cnt])
            np.testing.assert_array_equal(got["t%d_%d" % (b, 4 + 2 * j)], want["agg_dst"][lo:lo + cnt])
        assert list(got["blocks%d" % b]) == [nc[11], nc[10], nc[10], nc[9]]
