"""Q/K prologue (dt_qk_prologue): RMSNorm, rotary cmul and pre-scale of queries and keys in one pass, against the
oracle's restatement of the reference's separate nodes (Flux1.swift:164-188, Wan.swift:86-98,
Qwen3_5.swift:164-182).  cmul and the scale are exact on both sides; the RMS sum is accumulated in a different
order than on the CPU, so a normalised value may land on the neighbouring 16-bit value, and the rotation then
carries that unit into both members of its complex pair: the tests allow two units in the last place of the
pair's larger member, on at most 1 % of the elements, and require every other element to be bit-identical.
Without normalisation everything is bit-identical."""
import ctypes

import pytest
import torch

from oracle import sdpa_oracle as so
from test_gpu_parity import DEV, check

pytestmark = pytest.mark.gpu
ULP = {torch.bfloat16: 2.0 ** -7, torch.float16: 2.0 ** -10}


def close_1ulp(got, want, dtype, what, exact=False):
    g, w = got.float().cpu(), want.float()
    assert torch.isfinite(g).all(), what
    diff = (g - w).abs()
    if exact:
        assert torch.equal(got.cpu().view(torch.int16), want.view(torch.int16)), f"{what}: not bit-identical"
        return
    pair = w.abs().reshape(*w.shape[:-1], -1, 2).amax(dim=-1, keepdim=True).expand(*w.shape[:-1], -1, 2).reshape(w.shape)
    bad = diff > 2 * ULP[dtype] * pair + 1e-30
    assert not bool(bad.any()), f"{what}: {int(bad.sum())} elements beyond two ulp of their pair, max diff {float(diff.max())}"
    frac = float((diff > 0).float().mean())
    assert frac <= 1e-2, f"{what}: {frac:.2e} of the elements differ"


def test_flux_joint_prologue_then_attention(dtattn):
    """Text and image tokens are normalised with their own weights and written into one joint buffer (the
    reference's concat), rotated with the Flux table, then attended."""
    dtype, H, D, t, hh, ww = torch.bfloat16, 4, 128, 64, 12, 16
    S = t + hh * ww
    rot = so.flux_rope_table(hh, ww, t, D).to(dtype)               # [1, S, 1, D]
    parts, weights = {}, {}
    for i, name in enumerate(("cq", "ck", "xq", "xk")):
        n = t if name[0] == "c" else hh * ww
        parts[name] = so.seeded_normal((1, n, H, D), 800 + i, 2.0).to(dtype)
        weights[name] = (1.0 + 0.1 * so.seeded_normal((D,), 810 + i)).to(dtype)
    v = so.seeded_normal((1, S, H, D), 820).to(dtype)
    want = {}
    for name in parts:
        r = rot[:, :t] if name[0] == "c" else rot[:, t:]
        want[name] = so.qk_prologue_explicit(parts[name], weights[name], r, 1e-6, dtype)
    q_ref, k_ref = torch.cat([want["cq"], want["xq"]], 1), torch.cat([want["ck"], want["xk"]], 1)
    q_joint = torch.zeros(1, S, H, D, dtype=dtype, device=DEV)
    k_joint = torch.zeros_like(q_joint)
    rot_d = rot.to(DEV)
    dtattn.qk_prologue(parts["cq"].to(DEV), parts["ck"].to(DEV), q_out=q_joint[:, :t], k_out=k_joint[:, :t],
                       q_weight=weights["cq"].to(DEV), k_weight=weights["ck"].to(DEV), rotary=rot_d[:, :t])
    dtattn.qk_prologue(parts["xq"].to(DEV), parts["xk"].to(DEV), q_out=q_joint[:, t:], k_out=k_joint[:, t:],
                       q_weight=weights["xq"].to(DEV), k_weight=weights["xk"].to(DEV), rotary=rot_d[:, t:])
    torch.cuda.synchronize()
    close_1ulp(q_joint, q_ref, dtype, "flux q")
    close_1ulp(k_joint, k_ref, dtype, "flux k")
    out = dtattn.sdpa_forward(q_joint, k_joint, v.to(DEV), D ** -0.5)
    torch.cuda.synchronize()
    ref = so.sdpa_explicit(q_ref, k_ref, v, D ** -0.5, compute_dtype=torch.float64).float()
    check(out, ref, dtype, "flux prologue + attention")


def test_wan_per_token_norm_rotary_and_quarter_power_scale(dtattn):
    dtype, B, S, H, D = torch.float16, 2, 300, 5, 128
    x_q = so.seeded_normal((B, S, H, D), 830).to(dtype)
    x_k = so.seeded_normal((B, S, H, D), 831, 3.0).to(dtype)
    w_q = (1.0 + 0.2 * so.seeded_normal((H * D,), 832)).to(dtype)
    w_k = (1.0 + 0.2 * so.seeded_normal((H * D,), 833)).to(dtype)
    rot = so.qwen_rotary_table(S, 0, D, D, 10000.0).to(dtype)[:, :, None, :]
    scale = float(D) ** -0.25
    q, k = dtattn.qk_prologue(x_q.to(DEV), x_k.to(DEV), q_weight=w_q.to(DEV), k_weight=w_k.to(DEV),
                              rotary=rot.to(DEV), norm_per_token=True, post_scale=scale)
    torch.cuda.synchronize()
    close_1ulp(q, so.qk_prologue_explicit(x_q, w_q, rot, 1e-6, dtype, True, scale), dtype, "wan q")
    close_1ulp(k, so.qk_prologue_explicit(x_k, w_k, rot, 1e-6, dtype, True, scale), dtype, "wan k")


@pytest.mark.parametrize("case", [
    # B, S, H, D, dtype, rotary_dim
    (1, 77, 16, 256, torch.bfloat16, 64),   # Qwen3.5: partial rotary
    (2, 130, 8, 64, torch.float16, None),
    (1, 257, 8, 40, torch.float16, None),   # SD1.5 head dim: 5 of 8 lanes active
    (3, 9, 3, 96, torch.bfloat16, None),
])
def test_per_head_norm_and_rotary(dtattn, case):
    B, S, H, D, dtype, rdim = case
    x = so.seeded_normal((B, S, H, D), 840, 1.5).to(dtype)
    w = (1.0 + 0.3 * so.seeded_normal((D,), 841)).to(dtype)
    rot = so.qwen_rotary_table(S, 11, D, rdim).to(dtype)[:, :, None, :]
    q, _ = dtattn.qk_prologue(x.to(DEV), q_weight=w.to(DEV), rotary=rot.to(DEV))
    torch.cuda.synchronize()
    close_1ulp(q, so.qk_prologue_explicit(x, w, rot, 1e-6, dtype), dtype, str(case))


def test_rotation_only_is_bit_exact_in_place_and_per_head_table(dtattn):
    dtype, B, S, H, D = torch.bfloat16, 2, 100, 6, 128
    x = so.seeded_normal((B, S, H, D), 850).to(dtype)
    ang = so.seeded_normal((B, S, H, D // 2), 851) * 3.0
    rot = torch.stack([ang.cos(), ang.sin()], dim=-1).reshape(B, S, H, D).to(dtype)  # a table per batch and head
    xd = x.to(DEV)
    dtattn.qk_prologue(xd, q_out=xd, rotary=rot.to(DEV))  # in place
    torch.cuda.synchronize()
    close_1ulp(xd, so.qk_prologue_explicit(x, None, rot, 1e-6, dtype), dtype, "rotation only", exact=True)
    # pre-scale only (Wan with the rotation done elsewhere)
    y, _ = dtattn.qk_prologue(x.to(DEV), post_scale=0.3)
    torch.cuda.synchronize()
    close_1ulp(y, so.qk_prologue_explicit(x, None, None, 1e-6, dtype, False, 0.3), dtype, "scale only", exact=True)


def test_prologue_argument_checks(dtattn):
    lib = dtattn.lib()
    x = torch.zeros(1, 4, 2, 64, dtype=torch.float16, device=DEV)
    p = dtattn.make_prologue_params(x, x)
    assert lib.dt_qk_prologue(ctypes.byref(p), None, None) == dtattn.DT_OK
    p.D = 60
    assert lib.dt_qk_prologue(ctypes.byref(p), None, None) == dtattn.DT_UNSUPPORTED
    p = dtattn.make_prologue_params(x, x)
    p.dtype = dtattn.DT_F32
    assert lib.dt_qk_prologue(ctypes.byref(p), None, None) == dtattn.DT_UNSUPPORTED
    p = dtattn.make_prologue_params(x, x)
    p.y.ptr = None
    assert lib.dt_qk_prologue(ctypes.byref(p), None, None) == dtattn.DT_BAD_ARG
    assert lib.dt_qk_prologue(None, None, None) == dtattn.DT_BAD_ARG
    q = dtattn.make_prologue_params(x, x)
    k = dtattn.make_prologue_params(x, x, norm_per_token=True)
    assert lib.dt_qk_prologue(ctypes.byref(q), ctypes.byref(k), None) == dtattn.DT_BAD_ARG
    torch.cuda.synchronize()
