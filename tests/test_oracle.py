"""CPU checks of the oracle itself: the two restatements agree, the pieces the reference tree does pin
are reproduced, and the committed golden fixtures still match."""
import json
import math
import os

import numpy as np
import pytest
import torch

from oracle import c_oracle
from oracle import sdpa_oracle as so

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")

SHAPES = [
    # B, Sq, Sk, Hq, Hkv, D, causal
    (2, 33, 50, 4, 2, 40, False),
    (1, 5, 70, 8, 2, 64, True),
    (1, 64, 64, 2, 2, 128, True),
    (1, 1, 300, 8, 2, 128, True),     # decode: one query sees every cached row
    (2, 17, 1, 3, 3, 16, False),      # a single key
    (1, 7, 3, 2, 1, 8, True),         # Sq > Sk under a causal mask: the first rows see nothing -> zeros
]


@pytest.mark.parametrize("shape", SHAPES)
def test_python_and_c_oracles_agree(shape):
    B, Sq, Sk, Hq, Hkv, D, causal = shape
    q = so.seeded_normal((B, Sq, Hq, D), 11)
    k = so.seeded_normal((B, Sk, Hkv, D), 12)
    v = so.seeded_normal((B, Sk, Hkv, D), 13)
    ref, lse = so.sdpa_explicit(q, k, v, D ** -0.5, causal, compute_dtype=torch.float64, return_lse=True)
    out, lse_c = c_oracle.sdpa_c(q, k, v, D ** -0.5, causal, return_lse=True)
    mx, mean = so.error_stats(out, ref)
    assert mx < 2e-6 and mean < 2e-7
    fin = torch.isfinite(lse)
    assert torch.allclose(lse_c[fin].double(), lse[fin], atol=2e-6)
    out32 = so.sdpa_explicit(q, k, v, D ** -0.5, causal)
    assert so.error_stats(out32, ref)[0] < 2e-6


def test_masked_equals_causal():
    """The additive-mask form of causality (TextEncoder.swift:151-158) and is_causal give the same result."""
    B, S, H, D = 1, 24, 2, 32
    q, k, v = (so.seeded_normal((B, S, H, D), s) for s in (1, 2, 3))
    mask = torch.zeros(1, 1, S, S)
    mask.masked_fill_(torch.triu(torch.ones(S, S, dtype=torch.bool), 1), so.MASK_FILL)
    a = so.sdpa_explicit(q, k, v, D ** -0.5, mask=mask)
    b = so.sdpa_explicit(q, k, v, D ** -0.5, is_causal=True)
    c = c_oracle.sdpa_c(q, k, v, D ** -0.5, mask=mask)
    assert so.error_stats(a, b)[0] < 1e-6 and so.error_stats(c, b)[0] < 1e-6


def test_scale_conventions_are_one_operator():
    """.scale1 (Q pre-multiplied, scale 1), .scaleMerged (scale 1/sqrt k) and Wan's k^-1/4 on both Q and K
    (Flux1.swift:224-232, Wan.swift:95-103) are the same function."""
    B, S, H, D = 1, 40, 2, 64
    q, k, v = (so.seeded_normal((B, S, H, D), s) for s in (4, 5, 6))
    merged = so.sdpa_explicit(q, k, v, D ** -0.5)
    scale1 = so.sdpa_explicit(q * D ** -0.5, k, v, 1.0)
    wan = so.sdpa_explicit(q * D ** -0.25, k * D ** -0.25, v, 1.0)
    assert so.error_stats(scale1, merged)[0] < 1e-6 and so.error_stats(wan, merged)[0] < 1e-6


def test_gqa_grouping_is_contiguous():
    """Query heads [i*G, (i+1)*G) read KV head i (Llama.swift:74-86)."""
    B, S, Hq, Hkv, D = 1, 12, 6, 2, 16
    q = so.seeded_normal((B, S, Hq, D), 7)
    k = so.seeded_normal((B, S, Hkv, D), 8)
    v = so.seeded_normal((B, S, Hkv, D), 9)
    full = so.sdpa_explicit(q, k, v, 0.25)
    for h in range(Hq):
        one = so.sdpa_explicit(q[:, :, h:h + 1], k[:, :, h // 3:h // 3 + 1], v[:, :, h // 3:h // 3 + 1], 0.25)
        assert so.error_stats(one, full[:, :, h:h + 1])[0] < 1e-6


@pytest.mark.parametrize("seed,count", [(42, 1000), (7, 10), (7, 1003), (0, 16)])
def test_seeded_normal_matches_reference_generator(seed, count):
    """TorchRandomSource (Random/TorchRandomSource.swift) says it reproduces torch's CPU randn: the
    restatement's uniform stream is bit-identical to torch.rand and its normals agree with torch.randn to
    float rounding of the transcendental functions."""
    r = so.TorchRandomSourceRestated(seed)
    u = np.array([r.next_float() for _ in range(64)], dtype=np.float32)
    torch.manual_seed(seed)
    assert np.array_equal(u, torch.rand(64).numpy())
    got = so.TorchRandomSourceRestated(seed).normal_array(count)
    torch.manual_seed(seed)
    want = torch.randn(count).numpy()
    assert np.abs(got - want).max() <= 1e-6


def test_flux_rope_table_properties():
    """Flux1RotaryPositionEmbedding (Flux1.swift:5-72): unit-modulus pairs, identity for text tokens, axis
    split 16/56/56 of a 128-dim head, theta_k = pos / 10000^(2k/dim)."""
    hh, ww, tt, ch = 4, 6, 5, 128
    rot = so.flux_rope_table(hh, ww, tt, ch)
    assert rot.shape == (1, tt + hh * ww, 1, ch)
    c, s = rot[..., 0::2], rot[..., 1::2]
    assert torch.allclose(c * c + s * s, torch.ones_like(c), atol=1e-6)
    assert torch.all(c[:, :tt] == 1) and torch.all(s[:, :tt] == 0)
    y, x = 3, 4
    tok = tt + y * ww + x
    k = 5
    assert math.isclose(float(c[0, tok, 0, 8 + k]), math.cos(y / 10000 ** (2 * k / 56)), abs_tol=1e-6)
    assert math.isclose(float(s[0, tok, 0, 8 + 28 + k]), math.sin(x / 10000 ** (2 * k / 56)), abs_tol=1e-6)
    assert torch.all(c[0, tok, 0, :8] == 1)
    # cmul is a rotation: norms of pairs are preserved
    z = so.seeded_normal((1, tt + hh * ww, 2, ch), 3)
    r = so.cmul(z, rot)
    assert torch.allclose(z[..., 0::2] ** 2 + z[..., 1::2] ** 2, r[..., 0::2] ** 2 + r[..., 1::2] ** 2, atol=1e-5)


def test_instruction_count_formula():
    """B*H*(2D+5)*Sa*Sb (InstructionCount.swift:9-17); the FLOP figure the bench uses is 4*B*H*Sa*Sb*D."""
    assert so.instruction_count(1, 24, 128, 4608, 4608) == 24 * 261 * 4608 * 4608
    assert so.flops(1, 24, 4608, 4608, 128) == 260919263232


def test_config_shapes():
    c = so.CONFIGS
    assert (c["flux_joint"].Sq, c["flux_joint"].Hq, c["flux_joint"].D) == (4608, 24, 128)
    assert c["wan_self"].Sq == 21 * 45 * 80
    q, k, v = so.make_inputs(c["sdxl_cross"].shrink(Sq=64))
    assert q.shape == (2, 64, 20, 64) and k.shape == (2, 77, 20, 64) and q.dtype == torch.float16
    # per-head generation gives every rank the same values as each other rank sees for those heads
    small = c["flux_joint"].shrink(Sq=48, Sk=48, Hq=4, Hkv=4, rope_hw=(4, 8, 16))
    qa, ka, va = so.make_inputs(small, heads=(0, 4))
    qb, kb, vb = so.make_inputs(small, heads=(2, 4))
    assert torch.equal(qa[:, :, 2:], qb) and torch.equal(ka[:, :, 2:], kb) and torch.equal(va[:, :, 2:], vb)


def test_golden_fixtures():
    """Outputs of the oracle on small seeded cases, committed with the script that made them
    (tests/golden/make_golden.py).  The reference holds no attention fixtures of its own, so these pin the
    oracle against drift, not against the reference."""
    with open(os.path.join(GOLDEN, "sdpa_golden.json")) as f:
        cases = json.load(f)
    assert len(cases) >= 6
    for case in cases:
        cfg = case["cfg"]
        q = so.seeded_normal((cfg["B"], cfg["Sq"], cfg["Hq"], cfg["D"]), cfg["seed"])
        k = so.seeded_normal((cfg["B"], cfg["Sk"], cfg["Hkv"], cfg["D"]), cfg["seed"] + 1)
        v = so.seeded_normal((cfg["B"], cfg["Sk"], cfg["Hkv"], cfg["D"]), cfg["seed"] + 2)
        out = c_oracle.sdpa_c(q, k, v, cfg["scale"], cfg["causal"])
        got = out.flatten()[case["index"]].double()
        want = torch.tensor(case["values"], dtype=torch.float64)
        assert (got - want).abs().max() < 2e-6, cfg
        assert abs(float(out.double().sum()) - case["sum"]) < 1e-3 * max(1.0, abs(case["sum"]))
