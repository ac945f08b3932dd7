"""Host side of the hand-off without a GPU: segment layout, step arithmetic, semaphore protocol,
bounded waits and clean-up (failure detection is exercised on the host only)."""
import mmap
import multiprocessing as mp
import os
import time

import numpy as np
import pytest

import legion_ibp_b200 as L


def _name(tag):
    return "legion_b200_cpu_%s_%d" % (tag, os.getpid())


def test_segment_layout_and_steps(oracle_mod):
    name = _name("lay")
    env = L.IPCEnv(2, name)
    try:
        train, valid, test = [24491, 24490], [4900, 4899], [276630, 276629]
        env.Coordinate(train, valid, test, 8000, 3)
        steps, vbs, tbs = oracle_mod.coordinate(train, valid, test, 8000)
        assert env.steps() == list(steps)
        # the trainer reads steps[3] straight from the segment (ipc_cuda_kernel.cu:50-52)
        fd = os.open("/dev/shm/" + name, os.O_RDONLY)
        assert os.fstat(fd).st_size == L.ipc_layout()["segment_bytes"]
        raw = mmap.mmap(fd, 12, prot=mmap.PROT_READ)
        assert list(np.frombuffer(raw, np.int32, 3)) == list(steps)
        assert env.GetMaxStep() == (steps[0] + steps[1]) * 3 + steps[2]
        for b in range(env.GetMaxStep()):
            mode, local = oracle_mod.mode_of_batch(b, steps[0], steps[1], steps[2], 3)
            assert env.GetCurrentMode(b) == mode and env.GetLocalBatchId(b) == local
        for d in range(2):
            assert env.GetCurrentBatchsize(d, L.TRAINMODE) == 8000
            assert env.GetCurrentBatchsize(d, L.VALIDMODE) == vbs[d]
            assert env.GetCurrentBatchsize(d, L.TESTMODE) == tbs[d]
    finally:
        env.Finalize()
    assert not os.path.exists("/dev/shm/" + name)


def test_counters_are_published_in_a_companion_host_segment():
    """Next to the reference's segment the server keeps "<name>_ctr": int32 [8][2][32], node_counter then
    edge_counter of the last batch finished on (device, pipe); it goes away with the environment."""
    name = _name("ctr")
    env = L.IPCEnv(2, name)
    try:
        path = "/dev/shm/" + name + "_ctr"
        assert os.path.getsize(path) == 8 * 2 * 32 * 4
        seg = np.memmap(path, dtype=np.int32, mode="r", shape=(8, 2, 32))
        assert not seg.any()
        nc, ec = np.arange(16, dtype=np.int32) + 100, np.arange(16, dtype=np.int32) + 200
        env.publish_counters(1, 0, nc, ec)
        env.publish_counters(0, 1, ec, nc)
        np.testing.assert_array_equal(seg[1, 0], np.concatenate([nc, ec]))
        np.testing.assert_array_equal(seg[0, 1], np.concatenate([ec, nc]))
        assert not seg[0, 0].any() and not seg[1, 1].any()
        import pytest
        with pytest.raises(L.LegionError):
            env.publish_counters(0, 2, nc, ec)
        del seg
    finally:
        env.Finalize()
    assert not os.path.exists("/dev/shm/" + name + "_ctr")


def _trainer(name, n_batches, q):
    """The trainer's half of the protocol (ipc_cuda_kernel.cu:70-106): post sem_r once per pipe,
    then wait sem_w / post sem_r while rotating the pipe."""
    import ctypes as C
    libc = C.CDLL("libc.so.6", use_errno=True)
    libc.sem_open.restype = C.c_void_p
    libc.sem_open.argtypes = [C.c_char_p, C.c_int, C.c_uint, C.c_uint]
    libc.sem_wait.argtypes = [C.c_void_p]
    libc.sem_post.argtypes = [C.c_void_p]
    semr = [libc.sem_open(("%s_sem_r_0_%d" % (name, i)).encode(), os.O_CREAT | os.O_RDWR, 0o666, 0) for i in range(2)]
    semw = [libc.sem_open(("%s_sem_w_0_%d" % (name, i)).encode(), os.O_CREAT | os.O_RDWR, 0o666, 0) for i in range(2)]
    for s in semr:
        libc.sem_post(s)
    pipe, order = 0, []
    for b in range(n_batches):
        libc.sem_wait(semw[pipe])
        order.append(pipe)
        libc.sem_post(semr[pipe])
        pipe = (pipe + 1) % 2
    q.put(order)


def test_semaphore_protocol_with_a_trainer_process():
    name = _name("sem")
    env = L.IPCEnv(1, name)
    try:
        env.open_semaphores(0, 2)
        q = mp.get_context("fork").Queue()
        p = mp.get_context("fork").Process(target=_trainer, args=(name, 7, q))
        p.start()
        pipe = 0
        for b in range(7):
            env.IPCWait(0, pipe, timeout_ms=20000)   # slot free
            env.IPCPost(0, pipe)                     # slot full
            pipe = (pipe + 1) % 2
        assert q.get(timeout=20) == [0, 1, 0, 1, 0, 1, 0]
        p.join(20)
        assert p.exitcode == 0
        # two credits are left (one initial post per pipe was never used up for pipe 1, and the last
        # release of pipe 0); after them a lost trainer shows as a timeout, not a hang
        env.IPCWait(0, 1, timeout_ms=1000)
        env.IPCWait(0, 0, timeout_ms=1000)
        t0 = time.time()
        with pytest.raises(L.LegionError, match="did not release"):
            env.IPCWait(0, 1, timeout_ms=200)
        assert 0.15 < time.time() - t0 < 5
    finally:
        env.Finalize()
    left = [f for f in os.listdir("/dev/shm") if name in f]
    assert left == [], left


def test_wait_needs_open_semaphores():
    name = _name("arg")
    env = L.IPCEnv(1, name)
    try:
        with pytest.raises(L.LegionError):
            env.IPCWait(0, 0, timeout_ms=10)
        with pytest.raises(L.LegionError):
            env.open_semaphores(9, 2)
    finally:
        env.Finalize()


def test_default_names_are_the_reference_names():
    """Default segment and semaphore names are the ones the trainer extension hard-codes."""
    if os.path.exists("/dev/shm/simpleIPCshm"):
        pytest.skip("a sampling server seems to be running on this machine")
    env = L.IPCEnv(1, None)
    try:
        env.open_semaphores(3, 2)
        names = set(os.listdir("/dev/shm"))
        assert "simpleIPCshm" in names
        for nm in ("sem.sem_r_3_0", "sem.sem_r_3_1", "sem.sem_w_3_0", "sem.sem_w_3_1"):
            assert nm in names
    finally:
        env.Finalize()
    assert "simpleIPCshm" not in os.listdir("/dev/shm")
