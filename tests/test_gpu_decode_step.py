"""Fused decode step (dt_sdpa_decode_step): rotary cmul on the new queries and keys, KV-cache append and causal
attention in one launch, against the oracle's restatement of the reference's separate nodes
(Qwen3_5.swift:167-196).  The cache rows the call writes are compared bit for bit (cmul is three fp32
operations and one rounding on both sides); the attention output within the stated tolerance
(max-abs <= 2e-3, mean-abs <= 2e-4, plus the 16-bit output's own rounding on small shapes)."""
import ctypes

import pytest
import torch

from oracle import sdpa_oracle as so
from test_gpu_parity import DEV, check

pytestmark = pytest.mark.gpu


def make_case(B, cached, Tn, Sq, Hq, Hkv, D, dtype, seed, rotary_dim=None, capacity=None, per_batch_rotary=False,
              with_rotary=True):
    capacity = capacity or cached + Tn + 5
    q = so.seeded_normal((B, Sq, Hq, D), seed).to(dtype)
    k_new = so.seeded_normal((B, Tn, Hkv, D), seed + 1).to(dtype)
    v_new = so.seeded_normal((B, Tn, Hkv, D), seed + 2).to(dtype)
    k_cache = so.seeded_normal((B, capacity, Hkv, D), seed + 3).to(dtype)
    v_cache = so.seeded_normal((B, capacity, Hkv, D), seed + 4).to(dtype)
    rot = None
    if with_rotary:
        rot = so.qwen_rotary_table(Tn, cached, D, rotary_dim).to(dtype)
        if per_batch_rotary:  # a table per batch item (different positions per sequence)
            rot = torch.cat([so.qwen_rotary_table(Tn, cached + 7 * i, D, rotary_dim) for i in range(B)]).to(dtype)
    return q, k_cache, v_cache, k_new, v_new, rot


def run_step(dtattn, case, cached, scale, dtype, what, flags=0):
    q, k_cache, v_cache, k_new, v_new, rot = case
    Tn = k_new.shape[1]
    kc_ref, vc_ref = k_cache.clone(), v_cache.clone()
    rot_ref = rot if rot is None or rot.shape[0] > 1 else rot
    ref = so.decode_step_explicit(q, kc_ref, vc_ref, k_new, v_new, rot_ref, scale, cached, dtype)
    kc, vc = k_cache.to(DEV), v_cache.to(DEV)
    out = dtattn.decode_step(q.to(DEV), kc, vc, k_new.to(DEV), v_new.to(DEV), None if rot is None else rot.to(DEV),
                             scale, cached, flags=flags)
    torch.cuda.synchronize()
    assert dtattn.device_status() == 0, "a device-side wait ran out"
    # the whole cache, not only the appended rows: nothing else may have been touched
    assert torch.equal(kc.cpu().view(torch.int16), kc_ref.view(torch.int16)), f"{what}: key cache differs"
    assert torch.equal(vc.cpu().view(torch.int16), vc_ref.view(torch.int16)), f"{what}: value cache differs"
    check(out, ref, dtype, what)
    return out


STEPS = [
    # B, cached, T_new, Sq, Hq, Hkv, D, dtype, rotary_dim
    (1, 4095, 1, 1, 16, 4, 256, torch.bfloat16, 64),    # Qwen3.5 attention shape, one token per step
    (1, 2000, 1, 1, 16, 4, 256, torch.float16, 64),
    (2, 1000, 4, 4, 32, 8, 128, torch.bfloat16, None),  # 4 new tokens x group of 4 = 16 rows
    (1, 517, 3, 1, 64, 8, 64, torch.float16, None),     # keys for 3 new tokens, queries for the last one only
    (2, 0, 5, 5, 8, 4, 128, torch.float16, None),       # empty cache: the prompt's first rows
    (1, 16, 16, 2, 8, 8, 64, torch.bfloat16, 32),       # a full unit of new rows
    (3, 33, 2, 2, 4, 4, 256, torch.bfloat16, 64),       # streamed range ends inside a unit (zero-filled tail masked)
]


@pytest.mark.parametrize("case", STEPS)
def test_decode_step_matches_separate_nodes(dtattn, case):
    B, cached, Tn, Sq, Hq, Hkv, D, dtype, rdim = case
    c = make_case(B, cached, Tn, Sq, Hq, Hkv, D, dtype, 701, rdim)
    run_step(dtattn, c, cached, D ** -0.5, dtype, str(case))


def test_decode_step_per_batch_table_and_no_table(dtattn):
    c = make_case(3, 300, 2, 2, 16, 4, 128, torch.float16, 711, per_batch_rotary=True)
    run_step(dtattn, c, 300, 128 ** -0.5, torch.float16, "per-batch rotary")
    c = make_case(2, 300, 2, 2, 16, 4, 128, torch.bfloat16, 713, with_rotary=False)
    run_step(dtattn, c, 300, 128 ** -0.5, torch.bfloat16, "no rotary")


@pytest.mark.parametrize("splits", [1, 3, 4, 8, 16, 48])
def test_decode_step_split_counts(dtattn, splits):
    """The appended rows are attended by the last split only, whatever the split count (fixed here with
    DT_FLAG_DECODE_SPLITS): one CTA, an odd count, clusters of 4 and 8 that combine through distributed shared
    memory, and counts whose partials go through the workspace."""
    c = make_case(2, 1234, 2, 2, 8, 2, 128, torch.bfloat16, 721)
    run_step(dtattn, c, 1234, 128 ** -0.5, torch.bfloat16, f"splits={splits}", flags=dtattn.DT_FLAG_DECODE_SPLITS(splits))


def test_decode_loop_equals_attention_over_final_cache(dtattn):
    """Eight consecutive one-token steps: every step reads the rows the previous steps appended, and the last
    step's output equals plain attention (dt_sdpa_forward) over the final cache with the rotated query."""
    B, Hq, Hkv, D, dtype, start, steps = 2, 16, 4, 256, torch.bfloat16, 120, 8
    cap = start + steps
    k_cache = so.seeded_normal((B, cap, Hkv, D), 731).to(dtype)
    v_cache = so.seeded_normal((B, cap, Hkv, D), 732).to(dtype)
    kc_ref, vc_ref = k_cache.clone(), v_cache.clone()
    kc, vc = k_cache.to(DEV), v_cache.to(DEV)
    for t in range(steps):
        q = so.seeded_normal((B, 1, Hq, D), 740 + 3 * t).to(dtype)
        kn = so.seeded_normal((B, 1, Hkv, D), 741 + 3 * t).to(dtype)
        vn = so.seeded_normal((B, 1, Hkv, D), 742 + 3 * t).to(dtype)
        rot = so.qwen_rotary_table(1, start + t, D, 64).to(dtype)
        ref = so.decode_step_explicit(q, kc_ref, vc_ref, kn, vn, rot, D ** -0.5, start + t, dtype)
        out = dtattn.decode_step(q.to(DEV), kc, vc, kn.to(DEV), vn.to(DEV), rot.to(DEV), D ** -0.5, start + t)
        check(out, ref, dtype, f"step {t}")
    torch.cuda.synchronize()
    assert torch.equal(kc.cpu().view(torch.int16), kc_ref.view(torch.int16))
    assert torch.equal(vc.cpu().view(torch.int16), vc_ref.view(torch.int16))
    q_rot = so.cmul(q.float(), rot.float()[:, :, None, :]).to(dtype)
    plain = dtattn.sdpa_forward(q_rot.to(DEV), kc, vc, D ** -0.5, True)
    torch.cuda.synchronize()
    mx, mean = so.error_stats(out.float().cpu(), plain.float().cpu())
    assert mx <= so.TOL_MAX_ABS and mean <= so.TOL_MEAN_ABS, (mx, mean)
    assert dtattn.device_status() == 0


def test_decode_step_argument_checks(dtattn):
    lib = dtattn.lib()
    q, kc, vc, kn, vn, rot = [t.to(DEV) if t is not None else None
                              for t in make_case(1, 64, 2, 2, 8, 8, 64, torch.float16, 751)]
    o = torch.empty_like(q)
    need = ctypes.c_size_t(0)
    sp = dtattn.make_step_params(q, kc, vc, kn, vn, rot, o, 0.125, 66)
    assert lib.dt_sdpa_decode_step_workspace_size(ctypes.byref(sp), ctypes.byref(need)) == dtattn.DT_OK
    sp.T_new = 1  # fewer new rows than queries
    assert lib.dt_sdpa_decode_step_workspace_size(ctypes.byref(sp), ctypes.byref(need)) == dtattn.DT_BAD_ARG
    sp.T_new = 17  # more than one unit of new rows
    sp.attn.Sk = 100
    assert lib.dt_sdpa_decode_step(ctypes.byref(sp), None, 0, None) == dtattn.DT_UNSUPPORTED
    sp = dtattn.make_step_params(q, kc, vc, kn, vn, rot, o, 0.125, 66)
    sp.rotary = sp.rotary + 2  # misaligned table
    assert lib.dt_sdpa_decode_step(ctypes.byref(sp), None, 0, None) == dtattn.DT_UNSUPPORTED
    sp = dtattn.make_step_params(q, kc, vc, kn, vn, rot, o, 0.125, 66)
    sp.k_new.ptr = None
    assert lib.dt_sdpa_decode_step(ctypes.byref(sp), None, 0, None) == dtattn.DT_BAD_ARG


@pytest.mark.parametrize("case", [
    # B, cached, T_new, Sq, Hq, Hkv, D, dtype, rotary_dim
    (1, 3000, 1, 1, 16, 4, 256, torch.bfloat16, 64),   # Qwen3.5: qNorm, kNorm, partial rotary, append, attention
    (2, 700, 3, 1, 32, 8, 128, torch.float16, None),
    (1, 0, 5, 5, 8, 4, 64, torch.bfloat16, None),
])
def test_decode_step_with_qk_rmsnorm(dtattn, case):
    """qNorm / kNorm (Qwen3_5.swift:164-167) inside the step.  The RMS sum is accumulated in another order than on the
    CPU and uses the hardware reciprocal square root, so an appended key may land on the neighbouring 16-bit value
    (and the rotation carries that into its pair): keys within two units in the last place of their pair on at most
    1 % of the elements, values and every other cache row bit-identical, output within the stated tolerance."""
    B, cached, Tn, Sq, Hq, Hkv, D, dtype, rdim = case
    q, k_cache, v_cache, k_new, v_new, rot = make_case(B, cached, Tn, Sq, Hq, Hkv, D, dtype, 801, rdim)
    wq = (1.0 + 0.2 * so.seeded_normal((D,), 811)).to(dtype)
    wk = (1.0 + 0.2 * so.seeded_normal((D,), 812)).to(dtype)
    kc_ref, vc_ref = k_cache.clone(), v_cache.clone()
    ref = so.decode_step_explicit(q, kc_ref, vc_ref, k_new, v_new, rot, D ** -0.5, cached, dtype, wq, wk, 1e-6)
    kc, vc = k_cache.to(DEV), v_cache.to(DEV)
    out = dtattn.decode_step(q.to(DEV), kc, vc, k_new.to(DEV), v_new.to(DEV), rot.to(DEV), D ** -0.5, cached,
                             q_norm_weight=wq.to(DEV), k_norm_weight=wk.to(DEV), norm_eps=1e-6)
    torch.cuda.synchronize()
    assert dtattn.device_status() == 0
    assert torch.equal(vc.cpu().view(torch.int16), vc_ref.view(torch.int16))
    got, want = kc.cpu(), kc_ref
    keep = torch.ones(got.shape[1], dtype=torch.bool)
    keep[cached:cached + Tn] = False
    assert torch.equal(got[:, keep].view(torch.int16), want[:, keep].view(torch.int16)), "rows outside the append changed"
    g, w = got[:, cached:cached + Tn].float(), want[:, cached:cached + Tn].float()
    ulp = 2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -10
    pair = w.abs().reshape(*w.shape[:-1], -1, 2).amax(dim=-1, keepdim=True).expand(*w.shape[:-1], -1, 2).reshape(w.shape)
    diff = (g - w).abs()
    assert not bool((diff > 2 * ulp * pair + 1e-30).any()), float(diff.max())
    assert float((diff > 0).float().mean()) <= 1e-2
    check(out, ref, dtype, str(case))


@pytest.mark.parametrize("case", [
    # B, cached, T_new, Sq, Hq, Hkv, D, window
    (1, 3000, 1, 1, 32, 8, 128, 128),    # only the last 128 rows are streamed
    (2, 100, 4, 4, 8, 2, 64, 50),        # the window starts inside the cache and ends among the new rows
    (1, 20, 3, 3, 8, 8, 128, 2),         # a window narrower than the new rows: nothing of the cache is visible
])
def test_decode_step_with_sinks_and_sliding_window(dtattn, case):
    """The fused step with the operator variants of DeepSeek4.swift:482-493 (a cache, a window, sinks)."""
    B, cached, Tn, Sq, Hq, Hkv, D, window = case
    dtype = torch.bfloat16
    q, k_cache, v_cache, k_new, v_new, rot = make_case(B, cached, Tn, Sq, Hq, Hkv, D, dtype, 901)
    sinks = (so.seeded_normal((Hq,), 911) * 2.0).to(dtype)
    kc_ref, vc_ref = k_cache.clone(), v_cache.clone()
    ref = so.decode_step_explicit(q, kc_ref, vc_ref, k_new, v_new, rot, D ** -0.5, cached, dtype, sinks=sinks,
                                  sliding_window=window)
    kc, vc = k_cache.to(DEV), v_cache.to(DEV)
    out = dtattn.decode_step(q.to(DEV), kc, vc, k_new.to(DEV), v_new.to(DEV), rot.to(DEV), D ** -0.5, cached,
                             sinks=sinks.to(DEV), sliding_window=window)
    torch.cuda.synchronize()
    assert dtattn.device_status() == 0
    assert torch.equal(kc.cpu().view(torch.int16), kc_ref.view(torch.int16))
    assert torch.equal(vc.cpu().view(torch.int16), vc_ref.view(torch.int16))
    check(out, ref, dtype, str(case))
