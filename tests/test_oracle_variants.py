"""The oracle's restatements of the operator variants and of the steps either side of the operator, checked on the
CPU against closed-form answers that do not depend on the oracle's own code, and against the committed fixtures
(tests/golden/variants_golden.json, written by tests/golden/make_golden.py)."""
import importlib.util
import json
import math
import os

import torch

from oracle import sdpa_oracle as so

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def test_sink_closed_form():
    """q = 0 makes every score 0: the weights are uniform and the sink takes exp(sink) / (n + exp(sink))."""
    n, D = 10, 8
    q = torch.zeros(1, 1, 2, D)
    k = so.seeded_normal((1, n, 2, D), 1)
    v = so.seeded_normal((1, n, 2, D), 2)
    sinks = torch.tensor([0.0, math.log(3.0)])
    o = so.sdpa_explicit(q, k, v, 1.0, False, compute_dtype=torch.float64, sinks=sinks)
    mean_v = v.double().mean(dim=1)  # [1, 2, D]
    assert torch.allclose(o[0, 0, 0], mean_v[0, 0] * n / (n + 1.0), atol=1e-12)
    assert torch.allclose(o[0, 0, 1], mean_v[0, 1] * n / (n + 3.0), atol=1e-12)


def test_sliding_window_closed_form():
    """q = 0, causal, window W: row i is the mean of values max(0, i-W+1) .. i."""
    S, W, D = 9, 3, 4
    q = torch.zeros(1, S, 1, D)
    k = so.seeded_normal((1, S, 1, D), 3)
    v = so.seeded_normal((1, S, 1, D), 4)
    o = so.sdpa_explicit(q, k, v, 1.0, True, compute_dtype=torch.float64, sliding_window=W)
    for i in range(S):
        want = v[0, max(0, i - W + 1):i + 1, 0].double().mean(dim=0)
        assert torch.allclose(o[0, i, 0], want, atol=1e-12), i
    # bottom-right alignment: one new query over a cache of 9 rows sees the last W rows
    o1 = so.sdpa_explicit(q[:, :1], k, v, 1.0, True, compute_dtype=torch.float64, sliding_window=W)
    assert torch.allclose(o1[0, 0, 0], v[0, S - W:, 0].double().mean(dim=0), atol=1e-12)


def test_varlen_is_per_sequence_attention():
    q = so.seeded_normal((1, 12, 2, 8), 5)
    k = so.seeded_normal((1, 15, 2, 8), 6)
    v = so.seeded_normal((1, 15, 2, 8), 7)
    o = so.sdpa_varlen_explicit(q, k, v, 0.3, [0, 4, 4, 12], [0, 5, 9, 15], False, compute_dtype=torch.float64)
    assert torch.allclose(o[:, :4], so.sdpa_explicit(q[:, :4], k[:, :5], v[:, :5], 0.3, compute_dtype=torch.float64))
    assert torch.allclose(o[:, 4:], so.sdpa_explicit(q[:, 4:], k[:, 9:], v[:, 9:], 0.3, compute_dtype=torch.float64))


def test_rotary_table_and_cmul_closed_form():
    """Qwen3_5RotaryEmbedding (Qwen3_5.swift:85-108): pair k of token i holds (cos, sin) of
    (cached + i) / theta^(2k / rotaryDim); pairs beyond rotaryDim hold (1, 0).  cmul rotates (1, 0) onto (cos, sin)."""
    tab = so.qwen_rotary_table(3, 5, 16, 8, theta=100.0)
    assert tab.shape == (1, 3, 16)
    ang = 6.0 / 100.0 ** (2.0 * 1 / 8)
    assert abs(float(tab[0, 1, 2]) - math.cos(ang)) < 1e-6 and abs(float(tab[0, 1, 3]) - math.sin(ang)) < 1e-6
    assert torch.equal(tab[0, :, 8::2], torch.ones(3, 4)) and torch.equal(tab[0, :, 9::2], torch.zeros(3, 4))
    x = torch.zeros(1, 3, 1, 16)
    x[..., 0::2] = 1.0
    y = so.cmul(x, tab[:, :, None, :])
    assert torch.allclose(y, tab[:, :, None, :])
    # a rotation keeps the norm of every pair
    z = so.seeded_normal((1, 3, 2, 16), 8)
    r = so.cmul(z, tab[:, :, None, :])
    assert torch.allclose(r[..., 0::2] ** 2 + r[..., 1::2] ** 2, z[..., 0::2] ** 2 + z[..., 1::2] ** 2, atol=1e-5)


def test_rmsnorm_closed_form():
    x = torch.full((1, 2, 3, 8), 3.0, dtype=torch.bfloat16)
    w = torch.full((8,), 0.5, dtype=torch.bfloat16)
    y = so.qk_prologue_explicit(x, w, None, 0.0, torch.bfloat16)
    assert torch.equal(y.float(), torch.full((1, 2, 3, 8), 0.5))      # x / rms(x) = 1
    w_tok = torch.full((24,), 2.0, dtype=torch.bfloat16)
    y = so.qk_prologue_explicit(x, w_tok, None, 0.0, torch.bfloat16, norm_per_token=True, post_scale=0.25)
    assert torch.equal(y.float(), torch.full((1, 2, 3, 8), 0.5))      # 1 * 2 * 0.25


def test_decode_step_appends_then_attends():
    dt = torch.float16
    q = so.seeded_normal((1, 1, 4, 16), 9).to(dt)
    kn, vn = so.seeded_normal((1, 1, 2, 16), 10).to(dt), so.seeded_normal((1, 1, 2, 16), 11).to(dt)
    kc, vc = so.seeded_normal((1, 12, 2, 16), 12).to(dt), so.seeded_normal((1, 12, 2, 16), 13).to(dt)
    k0, v0 = kc.clone(), vc.clone()
    o = so.decode_step_explicit(q, kc, vc, kn, vn, None, 0.25, 7, dt)
    assert torch.equal(kc[:, :7], k0[:, :7]) and torch.equal(kc[:, 8:], k0[:, 8:]) and torch.equal(kc[:, 7:8], kn)
    assert torch.equal(vc[:, 7:8], vn) and torch.equal(vc[:, 8:], v0[:, 8:])
    assert torch.allclose(o, so.sdpa_explicit(q, kc[:, :8], vc[:, :8], 0.25, True))


def test_variant_fixtures():
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(GOLDEN, "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    with open(os.path.join(GOLDEN, "variants_golden.json")) as f:
        want = json.load(f)
    got = mod.variant_cases()
    assert set(got) == set(want) and len(want) >= 7
    for name, w in want.items():
        g = got[name]
        assert g["index"] == w["index"], name
        assert max(abs(a - b) for a, b in zip(g["values"], w["values"])) < 1e-9, name
        assert abs(g["sum"] - w["sum"]) < 1e-6 * max(1.0, abs(w["sum"])), name


def test_sparse_indexed_attention_closed_forms():
    """SparseIndexedAttention (DeepSeek4.swift:521-545) restated: raw rows under the causal window and selected rows of
    the compressed tensor in one softmax.  Checked against forms that do not use the restatement's own code path."""
    B, Sq, Sr, Sc, Hq, Hkv, D = 2, 6, 10, 7, 4, 1, 16
    q = so.seeded_normal((B, Sq, Hq, D), 61)
    kr, vr = so.seeded_normal((B, Sr, Hkv, D), 62), so.seeded_normal((B, Sr, Hkv, D), 63)
    kc, vc = so.seeded_normal((B, Sc, Hkv, D), 64), so.seeded_normal((B, Sc, Hkv, D), 65)
    sinks = so.seeded_normal((Hq,), 66)
    # (1) every compressed row selected by every query, no window: plain attention over [compressed; raw] keys with
    # the causal rule on the raw part only, which an additive mask expresses
    sel_all = torch.arange(Sc, dtype=torch.int32).view(1, 1, Sc).expand(1, Sq, Sc).contiguous()
    got = so.sparse_indexed_explicit(q, kr, vr, kc, vc, sel_all, 0.3, sinks=sinks, compute_dtype=torch.float64)
    mask = torch.zeros(1, 1, Sq, Sc + Sr, dtype=torch.float64)
    i, j = torch.arange(Sq).view(Sq, 1), torch.arange(Sr).view(1, Sr)
    mask[0, 0, :, Sc:] = torch.where(j > i + (Sr - Sq), float("-inf"), 0.0)
    want = so.sdpa_explicit(q, torch.cat([kc, kr], 1), torch.cat([vc, vr], 1), 0.3, mask=mask, sinks=sinks,
                            compute_dtype=torch.float64)
    assert (got - want).abs().max() < 1e-12
    # (2) no valid selected row: the raw sliding-window operator
    none = torch.full((1, Sq, 3), -1, dtype=torch.int32)
    got = so.sparse_indexed_explicit(q, kr, vr, kc, vc, none, 0.3, sinks=sinks, sliding_window=4, compute_dtype=torch.float64)
    want = so.sdpa_explicit(q, kr, vr, 0.3, True, sinks=sinks, sliding_window=4, compute_dtype=torch.float64)
    assert (got - want).abs().max() < 1e-12
    # (3) a row listed twice counts twice; out-of-range entries name no row
    sel = torch.tensor([[2, 2, 99], [0, 5, -1], [1, 1, 1], [6, -7, 3], [4, 4, 0], [7, 8, 9]], dtype=torch.int32).view(1, Sq, 3)
    got = so.sparse_indexed_explicit(q, kr, vr, kc, vc, sel, 0.3, sliding_window=3, compute_dtype=torch.float64)
    for b in range(B):
        for t in range(Sq):
            rows = [c for c in sel[0, t].tolist() if 0 <= c < Sc]
            raw = [r for r in range(Sr) if r <= t + (Sr - Sq) and r > t + (Sr - Sq) - 3]
            k_list = torch.cat([kr[b, raw], kc[b, rows]], 0) if rows else kr[b, raw]
            v_list = torch.cat([vr[b, raw], vc[b, rows]], 0) if rows else vr[b, raw]
            want_t = so.sdpa_explicit(q[b:b + 1, t:t + 1], k_list.unsqueeze(0), v_list.unsqueeze(0), 0.3,
                                      compute_dtype=torch.float64)
            assert (got[b, t] - want_t[0, 0]).abs().max() < 1e-12
