"""A bounded device-side wait really ends.

Every wait in the kernels gives up after a wall-clock limit, stores a code in the device status word and lets the
kernel return.  This test makes one run out ON PURPOSE WITHOUT FAULTING ANYTHING: it loads a bring-up build of the
library (lib/libdtattn_waittest.so: waits limited to 5 ms, and a host switch that tells the decode kernel's producer
lane to issue no loads).  The consumers then wait for data that never comes, give up after 5 ms, the kernel returns,
dt_device_status reports DT_TIMEOUT with code 1, and the next ordinary call on the same workspace is correct.  Nothing
traps, faults or waits without a limit.  Runs in a child process because the product library is already loaded here.
"""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "draw-things-community_b200", "lib", "libdtattn_waittest.so")

CHILD = r"""
import ctypes, os, sys, time
root = sys.argv[1]
sys.path.insert(0, root); sys.path.insert(0, os.path.join(root, "draw-things-community_b200"))
os.environ["DTATTN_LIB"] = sys.argv[2]
import torch, dtattn
from oracle import sdpa_oracle as so
lib = dtattn.lib()
dev = "cuda:0"
q = so.seeded_normal((1, 1, 8, 128), 1).half().to(dev)
k = so.seeded_normal((1, 4096, 2, 128), 2).half().to(dev)
v = so.seeded_normal((1, 4096, 2, 128), 3).half().to(dev)
ws = dtattn.Workspace(torch.device(dev))
good = dtattn.sdpa_forward(q, k, v, 128 ** -0.5, True, workspace=ws)
torch.cuda.synchronize()
assert dtattn.device_status() == 0
lib.dt_internal_set_decode_skip_loads(1)          # the failure, made on the host
t0 = time.monotonic()
dtattn.sdpa_forward(q, k, v, 128 ** -0.5, True, workspace=ws)
torch.cuda.synchronize()                           # returns: the waits ran out, nothing hangs
waited = time.monotonic() - t0
lib.dt_internal_set_decode_skip_loads(0)
code = ctypes.c_int(0)
st = lib.dt_device_status(None, ctypes.byref(code))
print("STATUS", st, code.value, round(waited, 4))
assert st == dtattn.DT_TIMEOUT and code.value == 1, (st, code.value)
assert 0.004 < waited < 1.0, waited
assert dtattn.device_status() == 0                 # the word was cleared by the read
# the workspace's ticket counters are in an unknown state after a failed call: reset them, then all is well again
lib.dt_sdpa_workspace_init(ctypes.c_void_p(ws.buf.data_ptr()), ws.buf.numel(), None)
again = dtattn.sdpa_forward(q, k, v, 128 ** -0.5, True, workspace=ws)
torch.cuda.synchronize()
assert dtattn.device_status() == 0
assert torch.equal(again, good)
print("RECOVERED")
"""


def test_a_wait_that_runs_out_returns_and_reports():
    if not os.path.exists(LIB):
        pytest.skip("lib/libdtattn_waittest.so is not built (python draw-things-community_b200/build.py --all)")
    r = subprocess.run([sys.executable, "-c", CHILD, ROOT, LIB], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-1500:]
    assert "RECOVERED" in r.stdout
