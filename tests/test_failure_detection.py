"""Failure detection without any GPU fault: failures are made on the host.

* a rank that leaves between steps: the surviving rank's next collective ends with an error inside the process-group
  timeout instead of hanging (Gloo ranks on CPU);
* a failing launcher return code and a non-zero kernel status word are turned into exceptions by the loader
  (`ops/_lib.check_rc`, `check_status` semantics exercised on a fake status buffer);
* on a GPU, a device-side bounded wait is made to run out (a flag that nothing sets, a limit of milliseconds): the
  kernel returns, the status word names the wait, the kernels that depend on it skip their work.
The reference has no failure handling at all (its collectives use the default 10-minute NCCL timeout, train.py:956).
"""
import os
import socket
import sys
import time

import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    from slowrun_b200.parallel.comm import TorchComm, init_distributed
    init_distributed(device="cpu", timeout_s=4)
    comm = TorchComm()
    t = torch.ones(4)
    comm.all_reduce_sum(t, async_op=False)          # step 1: both ranks take part
    assert float(t[0]) == world
    if rank == 1:
        os._exit(0)                                 # leaves between steps, nothing in flight
    t0 = time.time()
    try:
        comm.all_reduce_sum(torch.ones(4), async_op=False)   # step 2: the peer is gone
        outcome = "completed"
    except Exception as e:  # noqa: BLE001
        outcome = f"error:{type(e).__name__}"
    with open(os.path.join(out, "rank0.txt"), "w") as f:
        f.write(f"{outcome} {time.time() - t0:.1f}")
    os._exit(0)


@pytest.mark.timeout(120)
def test_rank_that_leaves_is_detected_within_the_timeout(tmp_path):
    ctx = mp.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, str(tmp_path))) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(90)
        assert not p.is_alive(), "a rank hung instead of reporting the lost peer"
    outcome, secs = open(tmp_path / "rank0.txt").read().split()
    assert outcome.startswith("error:"), outcome
    assert float(secs) < 60


def test_launcher_codes_and_status_word_raise():
    from slowrun_b200.ops import _lib
    _lib.check_rc(0, "ok")
    with pytest.raises(RuntimeError, match="returned -5"):
        _lib.check_rc(-5, "sr_fake_launch")
    # the status word a kernel writes when a bounded wait runs out: [code, site, block, detail]
    fake = torch.tensor([2, 900, 0, 3], dtype=torch.int32)
    saved = _lib.status_buffer
    try:
        _lib.status_buffer = lambda device=None: fake
        with pytest.raises(_lib.KernelStatusError, match="code=2 site=900"):
            _lib.check_status()
        assert int(fake[0]) == 0, "the word is cleared after it has been reported"
        _lib.check_status()
    finally:
        _lib.status_buffer = saved


def test_reference_arm_reports_unavailable_without_a_gpu():
    """`bench.py --impl reference` must print one JSON line and exit 0 even where the reference cannot run."""
    import json
    import subprocess
    if torch.cuda.is_available():
        pytest.skip("a GPU is present: the arm would run the reference")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "1"],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "unavailable" in line


@pytest.mark.gpu
def test_device_side_peer_wait_runs_out_and_the_step_is_skipped():
    """A peer that never arrives, on ONE GPU and without any fault: the barrier is launched for a world of two whose
    second flag word nobody writes, with a wait limit of a few milliseconds. The kernel must return by itself, the
    status word must say which wait gave up (code 2 = peer wait, site 900, detail = the missing peer), a consumer
    kernel launched after it must not touch its output, and once the word is cleared the next launches work."""
    import ctypes
    from slowrun_b200.ops import _lib
    dev = torch.device("cuda", 0)
    torch.cuda.synchronize()
    _lib.check_status(dev)
    flags0 = torch.zeros(64, dtype=torch.int32, device=dev)     # "rank 0" (this process)
    flags1 = torch.zeros(64, dtype=torch.int32, device=dev)     # stands in for a peer that is never launched
    ptrs = (ctypes.c_ulonglong * 2)(flags0.data_ptr(), flags1.data_ptr())
    status = _lib.status_buffer(dev)
    barrier = _lib.fn("sr_peer_barrier", [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_uint, ctypes.c_void_p,
                                          ctypes.c_ulonglong, ctypes.c_void_p])
    t0 = time.time()
    assert barrier(ctypes.cast(ptrs, ctypes.c_void_p), 0, 2, 1, status.data_ptr(), 5_000_000, _lib.stream_ptr()) == 0
    # a consumer of the "collective": sums two sources into `out`; it must see the failed barrier and leave `out` alone
    src = torch.ones(1024, device=dev)
    out = torch.full((1024,), -7.0, device=dev)
    sptrs = (ctypes.c_ulonglong * 2)(src.data_ptr(), src.data_ptr())
    reduce = _lib.fn("sr_reduce_multi", [ctypes.c_void_p, ctypes.c_int, ctypes.c_long, ctypes.c_void_p, ctypes.c_long,
                                         ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p])
    assert reduce(ctypes.cast(sptrs, ctypes.c_void_p), 2, 0, out.data_ptr(), 1024, 0, status.data_ptr(), _lib.stream_ptr()) == 0
    torch.cuda.synchronize()
    assert time.time() - t0 < 5.0, "the wait limit was not honoured"
    assert int(flags1[0]) == 1, "this rank did announce itself to the peer"
    assert float(out[0]) == -7.0 and float(out[-1]) == -7.0, "a consumer ran after a failed barrier"
    with pytest.raises(_lib.KernelStatusError, match="code=2 site=900") as ei:
        _lib.check_status(dev)
    assert "detail=1" in str(ei.value)
    # cleared: the same launches now go through (the peer's flag is written by hand, as its barrier kernel would)
    flags0[1] = 2
    assert barrier(ctypes.cast(ptrs, ctypes.c_void_p), 0, 2, 2, status.data_ptr(), 5_000_000, _lib.stream_ptr()) == 0
    assert reduce(ctypes.cast(sptrs, ctypes.c_void_p), 2, 0, out.data_ptr(), 1024, 0, status.data_ptr(), _lib.stream_ptr()) == 0
    torch.cuda.synchronize()
    _lib.check_status(dev)
    assert float(out[0]) == 2.0
