"""dt_sdpa_decode_noalloc: the decode entry point for hosts that cannot allocate device memory when they call
(a runtime that gave the whole GPU to its own allocator at start-up, or a token loop that must not stall on
an allocation).  Its scratch is a fixed array inside the library image, so consecutive calls reuse the same
bytes: this test runs two calls in a row on different inputs through the C ABI and checks each against the
workspace-based entry point (dt_sdpa_forward).  Collected last (file name) so that a failure here cannot hide
another test when a run stops at the first failure."""
import ctypes
import os

import pytest
import torch

from oracle import sdpa_oracle as so

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _case(seed, B, Sk, Hq, Hkv, D, dtype):
    q = so.seeded_normal((B, 1, Hq, D), seed).to(dtype).to(DEV)
    k = so.seeded_normal((B, Sk, Hkv, D), seed + 1).to(dtype).to(DEV)
    v = so.seeded_normal((B, Sk, Hkv, D), seed + 2).to(dtype).to(DEV)
    return q, k, v


def test_noalloc_matches_workspace_entry_point_twice(dtattn):
    lib = dtattn.lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    # two different requests back to back: the second must not see anything of the first in the shared array
    cases = [_case(301, 2, 3000, 32, 8, 128, torch.float16), _case(311, 1, 8192, 32, 8, 128, torch.float16),
             _case(321, 3, 777, 8, 8, 64, torch.bfloat16)]
    for q, k, v in cases:
        D = q.shape[-1]
        want = dtattn.sdpa_forward(q, k, v, D ** -0.5, True)
        torch.cuda.synchronize()
        got = torch.full_like(q, float("nan"))
        p = dtattn.make_params(q, k, v, got, D ** -0.5, True)
        assert dtattn.kernel_name(p) == "decode_splitkv" and dtattn.workspace_size(p) > 0
        before = torch.cuda.memory_allocated()
        assert lib.dt_sdpa_decode_noalloc(ctypes.byref(p), stream) == dtattn.DT_OK
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        mx, mean = so.error_stats(got.float().cpu(), want.float().cpu())
        assert mx <= so.TOL_MAX_ABS and mean <= so.TOL_MEAN_ABS, (mx, mean)
        ref = so.sdpa_explicit(q.cpu(), k.cpu(), v.cpu(), D ** -0.5, True)
        mx, mean = so.error_stats(got.float().cpu(), ref)
        assert mx <= so.TOL_MAX_ABS + 2 ** -8 * float(ref.abs().max()) and mean <= 2 * so.TOL_MEAN_ABS, (mx, mean)


def test_noalloc_rejects_requests_beyond_its_array(dtattn):
    lib = dtattn.lib()
    q, k, v = _case(331, 1, 256, 32, 8, 128, torch.float16)
    o = torch.empty_like(q)
    p = dtattn.make_params(q, k, v, o, 128 ** -0.5, True)
    p.B, p.Sq, p.Sk = 16, 4, 8192  # sizes only: the request is refused before any pointer is used
    # the library's own split choice keeps the partials small; a forced split count (tuning override) does not
    os.environ["DTATTN_DECODE_SPLITS"] = "128"
    try:
        assert dtattn.workspace_size(p) > dtattn.NOALLOC_SCRATCH_BYTES
        assert lib.dt_sdpa_decode_noalloc(ctypes.byref(p), None) == dtattn.DT_SCRATCH_LIMIT
    finally:
        del os.environ["DTATTN_DECODE_SPLITS"]
    assert "scratch" in dtattn.status_string(dtattn.DT_SCRATCH_LIMIT)
    # shapes the decode kernel does not serve are refused as well
    p2 = dtattn.make_params(torch.empty(1, 64, 8, 128, dtype=torch.float16, device=DEV), k[:1], v[:1],
                            torch.empty(1, 64, 8, 128, dtype=torch.float16, device=DEV), 0.1, True)
    assert lib.dt_sdpa_decode_noalloc(ctypes.byref(p2), None) == dtattn.DT_UNSUPPORTED
