"""The CUDA kernels against the COMMITTED fixtures (tests/golden/*.json, written by tests/golden/make_golden.py from
the float64 oracle), through the C ABI: the fixture files, not a freshly evaluated oracle, are the yardstick here, so
a drift of the oracle and of the kernels in the same direction cannot go unnoticed.

Each attention case runs three times: fp32 tensors (CUDA-core kernels, fp32 arithmetic: the sampled values must agree
to 2e-5), fp16 and bf16 tensors (whatever kernel the library picks: tensor-core prefill, split-KV decode; the tolerance
is the one of the other parity tests plus the rounding of the 16-bit inputs, which the fixture did not see).
"""
import json
import os

import pytest
import torch

from oracle import sdpa_oracle as so

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")

with open(os.path.join(GOLDEN, "sdpa_golden.json")) as _f:
    CASES = json.load(_f)
with open(os.path.join(GOLDEN, "variants_golden.json")) as _f:
    VARIANTS = json.load(_f)


def inputs_of(cfg):
    q = so.seeded_normal((cfg["B"], cfg["Sq"], cfg["Hq"], cfg["D"]), cfg["seed"])
    k = so.seeded_normal((cfg["B"], cfg["Sk"], cfg["Hkv"], cfg["D"]), cfg["seed"] + 1)
    v = so.seeded_normal((cfg["B"], cfg["Sk"], cfg["Hkv"], cfg["D"]), cfg["seed"] + 2)
    return q, k, v


@pytest.mark.parametrize("n", range(len(CASES)))
def test_fp32_kernels_reproduce_the_fixture(dtattn, n):
    case = CASES[n]
    cfg = case["cfg"]
    q, k, v = inputs_of(cfg)
    out = dtattn.sdpa_forward(q.to(DEV), k.to(DEV), v.to(DEV), cfg["scale"], cfg["causal"])
    torch.cuda.synchronize()
    assert dtattn.device_status() == 0
    got = out.cpu().flatten()[case["index"]].double()
    want = torch.tensor(case["values"], dtype=torch.float64)
    assert (got - want).abs().max() < 2e-5, cfg
    assert abs(float(out.double().sum()) - case["sum"]) < 1e-3 * max(1.0, abs(case["sum"])), cfg


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("n", range(len(CASES)))
def test_half_precision_kernels_against_the_fixture(dtattn, n, dtype):
    """The tensors are rounded to 16 bits before the call, the fixture was computed from the unrounded ones: the
    bound adds what that rounding does to a softmax-weighted mean of unit-normal values (a few ulp of 16-bit)."""
    case = CASES[n]
    cfg = case["cfg"]
    q, k, v = (t.to(dtype) for t in inputs_of(cfg))
    p = dtattn.make_params(q.to(DEV), k.to(DEV), v.to(DEV), q.to(DEV), cfg["scale"], cfg["causal"])
    assert dtattn.kernel_name(p) in ("prefill_tcgen05", "decode_splitkv", "crossattn_short")
    out = dtattn.sdpa_forward(q.to(DEV), k.to(DEV), v.to(DEV), cfg["scale"], cfg["causal"])
    torch.cuda.synchronize()
    assert dtattn.device_status() == 0
    got = out.float().cpu().flatten()[case["index"]].double()
    want = torch.tensor(case["values"], dtype=torch.float64)
    ulp = 2.0 ** -11 if dtype == torch.float16 else 2.0 ** -8
    bound = so.TOL_MAX_ABS + 8 * ulp * max(1.0, float(want.abs().max()))
    assert (got - want).abs().max() < bound, (cfg, float((got - want).abs().max()), bound)
    assert (got - want).abs().mean() < bound / 4, cfg


def test_sinks_and_window_fixture(dtattn):
    q, k, v = (so.seeded_normal(s, 200 + i) for i, s in enumerate([(1, 40, 8, 64), (1, 40, 2, 64), (1, 40, 2, 64)]))
    sinks = so.seeded_normal((8,), 203) * 2.0
    fx = VARIANTS["sinks_window"]
    want = torch.tensor(fx["values"], dtype=torch.float64)
    out = dtattn.sdpa_forward(q.to(DEV), k.to(DEV), v.to(DEV), 0.125, True, sinks=sinks.to(DEV), sliding_window=16)
    torch.cuda.synchronize()
    assert (out.cpu().flatten()[fx["index"]].double() - want).abs().max() < 2e-5  # fp32: CUDA-core kernel
    h = torch.bfloat16
    out = dtattn.sdpa_forward(q.to(h).to(DEV), k.to(h).to(DEV), v.to(h).to(DEV), 0.125, True, sinks=sinks.to(h).to(DEV),
                              sliding_window=16)
    torch.cuda.synchronize()
    assert dtattn.device_status() == 0
    assert (out.float().cpu().flatten()[fx["index"]].double() - want).abs().max() < so.TOL_MAX_ABS + 8 * 2.0 ** -8 * 3


def test_variable_length_fixture(dtattn):
    q, k, v = (so.seeded_normal(s, 200 + i) for i, s in enumerate([(1, 40, 8, 64), (1, 40, 2, 64), (1, 40, 2, 64)]))
    off_q, off_k = [0, 5, 5, 30, 40], [0, 7, 10, 35, 40]
    fx = VARIANTS["varlen"]
    want = torch.tensor(fx["values"], dtype=torch.float64)
    oq = torch.tensor(off_q, dtype=torch.int32, device=DEV)
    ok = torch.tensor(off_k, dtype=torch.int32, device=DEV)
    for dtype, bound in ((torch.float32, 2e-5), (torch.float16, so.TOL_MAX_ABS + 8 * 2.0 ** -11 * 3)):
        out = torch.zeros(q.shape, dtype=dtype, device=DEV)
        dtattn.sdpa_forward(q.to(dtype).to(DEV), k.to(dtype).to(DEV), v.to(dtype).to(DEV), 0.125, False, out=out,
                            seq_offsets_q=oq, seq_offsets_k=ok, max_seq_q=25, max_seq_k=25)
        torch.cuda.synchronize()
        assert dtattn.device_status() == 0
        assert (out.float().cpu().flatten()[fx["index"]].double() - want).abs().max() < bound, dtype
