"""Failure paths of the communicator set-up, driven on the host: no kernel is launched and no GPU is needed.

The attention library loads NCCL with dlopen and creates its communicator in non-blocking mode, polling
ncclCommGetAsyncError with a wall-clock limit, so that a rank that never joins ends in DT_TIMEOUT instead of a
hang.  These tests point the library at a stand-in libnccl (tests/fake/fake_nccl.c, built here with gcc) whose
communicator never becomes ready, reports an asynchronous error, or becomes ready after a few polls, and check
the status codes, the time the wait takes and that a communicator that timed out is aborted.  Each case runs in
a child process because the library resolves NCCL once per process.
"""
import os
import subprocess
import sys
import time

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
FAKE_SRC = os.path.join(ROOT, "tests", "fake", "fake_nccl.c")

CHILD = r"""
import ctypes, os, sys, time
sys.path.insert(0, os.path.join(sys.argv[1], "draw-things-community_b200"))
import dtattn
lib = dtattn.lib()
ident = ctypes.create_string_buffer(128)
assert lib.dt_comm_unique_id(ident) == dtattn.DT_OK
comm = ctypes.c_void_p()
t0 = time.monotonic()
st = lib.dt_comm_init(ctypes.byref(comm), 0, 2, ident, int(sys.argv[2]))
print("RESULT", st, round(time.monotonic() - t0, 3), int(bool(comm.value)))
if comm.value:
    lib.dt_comm_destroy(comm)
"""


@pytest.fixture(scope="module")
def fake_nccl(tmp_path_factory):
    out = tmp_path_factory.mktemp("fake_nccl") / "libfake_nccl.so"
    subprocess.check_call(["gcc", "-O1", "-shared", "-fPIC", "-o", str(out), FAKE_SRC])
    return str(out)


def run_child(fake_nccl, mode, timeout_ms, tmp_path):
    log = tmp_path / f"calls_{mode}.txt"
    env = dict(os.environ, DTATTN_NCCL_LIB=fake_nccl, FAKE_NCCL_MODE=mode, FAKE_NCCL_LOG=str(log))
    t0 = time.monotonic()
    r = subprocess.run([sys.executable, "-c", CHILD, ROOT, str(timeout_ms)], env=env, capture_output=True, text=True,
                       timeout=120)
    assert r.returncode == 0, r.stderr[-2000:]
    line = [ln for ln in r.stdout.splitlines() if ln.startswith("RESULT")][0].split()
    calls = log.read_text().split() if log.exists() else []
    return int(line[1]), float(line[2]), int(line[3]), calls, time.monotonic() - t0


def test_rank_that_never_joins_ends_in_timeout(dtattn, fake_nccl, tmp_path):
    st, waited, have_comm, calls, _ = run_child(fake_nccl, "never", 700, tmp_path)
    assert st == dtattn.DT_TIMEOUT and have_comm == 0
    assert 0.65 <= waited < 10.0, waited          # the limit is honoured, and the call does come back
    assert calls.count("CommInitRankConfig") == 1 and calls.count("CommAbort") == 1  # the half-made communicator is torn down
    assert "CommDestroy" not in calls


def test_asynchronous_error_is_reported_as_nccl_failure(dtattn, fake_nccl, tmp_path):
    st, waited, have_comm, calls, _ = run_child(fake_nccl, "error", 5000, tmp_path)
    assert st == dtattn.DT_NCCL and have_comm == 0 and waited < 4.0
    assert calls.count("CommAbort") == 1


def test_communicator_that_becomes_ready_is_accepted(dtattn, fake_nccl, tmp_path):
    import torch
    st, waited, have_comm, calls, _ = run_child(fake_nccl, "ready", 5000, tmp_path)
    if torch.cuda.is_available():
        assert st == dtattn.DT_OK and have_comm == 1 and "CommDestroy" in calls
    else:  # the polling succeeded; creating the side stream then fails for want of a device
        assert st == dtattn.DT_CUDA and have_comm == 0
    assert "CommAbort" not in calls or st != dtattn.DT_OK
    assert waited < 4.0
