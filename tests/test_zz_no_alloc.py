"""dt_sdpa_decode_noalloc: the decode entry point for hosts that cannot allocate device memory when they call
(a runtime that gave the whole GPU to its own allocator at start-up, or a token loop that must not stall on
an allocation).  Its scratch is a fixed array inside the library image, so consecutive calls reuse the same
bytes: this test runs two calls in a row on different inputs through the C ABI and checks each against the
workspace-based entry point (dt_sdpa_forward).  Collected last (file name) so that a failure here cannot hide
another test when a run stops at the first failure."""
import ctypes

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
    # (inputs, split count): with up to 8 splits per KV head the CTAs combine inside a thread-block cluster and
    # need no scratch, so most cases fix a larger or an odd count, which makes the partials go through the scratch
    # array; the batch-1 shapes (the last but one) do so by the library's own choice
    cases = [(_case(301, 2, 3000, 32, 8, 128, torch.float16), 48), (_case(311, 1, 8192, 32, 8, 128, torch.float16), 64),
             (_case(321, 3, 777, 8, 8, 64, torch.bfloat16), 5), (_case(341, 1, 8192, 16, 4, 256, torch.bfloat16), 0),
             (_case(351, 2, 3000, 32, 8, 128, torch.float16), 0)]
    code = ctypes.c_int(-1)
    for (q, k, v), splits in cases:
        D = q.shape[-1]
        flags = dtattn.DT_FLAG_DECODE_SPLITS(splits)
        want = dtattn.sdpa_forward(q, k, v, D ** -0.5, True, flags=flags)
        torch.cuda.synchronize()
        got = torch.full_like(q, float("nan"))
        p = dtattn.make_params(q, k, v, got, D ** -0.5, True, flags=flags)
        assert dtattn.kernel_name(p) == "decode_splitkv" and (dtattn.workspace_size(p) > 0 or splits == 0)
        # memory the driver reports free on the device: unlike torch's own counters it would see a cudaMalloc made
        # inside the library.  The first call on a device does the one-time set-up, so it is measured on a repeat.
        assert lib.dt_sdpa_decode_noalloc(ctypes.byref(p), stream) == dtattn.DT_OK
        torch.cuda.synchronize()
        got.fill_(float("nan"))
        free_before = torch.cuda.mem_get_info()[0]
        assert lib.dt_sdpa_decode_noalloc(ctypes.byref(p), stream) == dtattn.DT_OK
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before
        assert lib.dt_sdpa_decode_noalloc_status(stream, ctypes.byref(code)) == dtattn.DT_OK and code.value == 0
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
    # the library's own split choice keeps the partials small; a fixed split count (tuning flag) that forms no
    # cluster does not: 255 partials x 128 (batch, KV head) pairs x 16 rows x 128 floats
    p.flags = dtattn.DT_FLAG_DECODE_SPLITS(255)
    assert dtattn.workspace_size(p) > dtattn.NOALLOC_SCRATCH_BYTES
    assert lib.dt_sdpa_decode_noalloc(ctypes.byref(p), None) == dtattn.DT_SCRATCH_LIMIT
    p.flags = 0
    assert "scratch" in dtattn.status_string(dtattn.DT_SCRATCH_LIMIT)
    # shapes the decode kernel does not serve are refused as well
    p2 = dtattn.make_params(torch.empty(1, 64, 8, 128, dtype=torch.float16, device=DEV), k[:1], v[:1],
                            torch.empty(1, 64, 8, 128, dtype=torch.float16, device=DEV), 0.1, True)
    assert lib.dt_sdpa_decode_noalloc(ctypes.byref(p2), None) == dtattn.DT_UNSUPPORTED


def test_noalloc_checks_arguments_like_the_workspace_entry_point(dtattn):
    """Nothing is launched for a request dt_sdpa_forward would refuse: a NaN scale, a negative window, output or
    sink pointers that are not aligned to the element size, a misaligned log-sum-exp pointer."""
    lib = dtattn.lib()
    q, k, v = _case(361, 1, 512, 8, 2, 128, torch.float16)
    o = torch.empty_like(q)
    sinks = torch.zeros(8, dtype=torch.float16, device=DEV)
    lse = torch.empty(1, 8, 1, dtype=torch.float32, device=DEV)

    def params():
        return dtattn.make_params(q, k, v, o, 128 ** -0.5, True, sinks=sinks, lse=lse)

    for name, value in (("scale", float("nan")), ("sliding_window", -1), ("sinks", sinks.data_ptr() + 1),
                        ("lse", lse.data_ptr() + 2), ("Hkv", 3)):
        p = params()
        setattr(p, name, value)
        assert lib.dt_sdpa_decode_noalloc(ctypes.byref(p), None) == dtattn.DT_BAD_ARG, name
        assert lib.dt_sdpa_forward(ctypes.byref(p), None, 0, None) == dtattn.DT_BAD_ARG, name
    p = params()
    p.o.ptr = o.data_ptr() + 1
    assert lib.dt_sdpa_decode_noalloc(ctypes.byref(p), None) == dtattn.DT_BAD_ARG
    assert lib.dt_sdpa_decode_noalloc_status(None, None) == dtattn.DT_BAD_ARG
    code = ctypes.c_int(-1)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.dt_sdpa_decode_noalloc(ctypes.byref(params()), stream) == dtattn.DT_OK
    assert lib.dt_sdpa_decode_noalloc_status(stream, ctypes.byref(code)) == dtattn.DT_OK and code.value == 0
