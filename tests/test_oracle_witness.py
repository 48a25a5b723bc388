"""An independent witness for the CPU oracle.

The reference holds no attention kernel, test or golden vector, so the oracle cannot be pinned against the
reference's own arithmetic.  What can be done is to compare both restatements (oracle/sdpa_oracle.py and
oracle/sdpa_oracle.c) with an implementation none of this repository's authors wrote: torch's CPU
``scaled_dot_product_attention`` in float64.  torch knows nothing of the operator's variants, so each one is
handed to it in a form it does understand: grouped heads through ``enable_gqa``, the bottom-right causal rule and
the sliding window as an explicit boolean mask, an additive mask as a float mask, an attention sink as one more
key column whose value row is zero.
"""
import pytest
import torch
import torch.nn.functional as F

from oracle import c_oracle
from oracle import sdpa_oracle as so


def torch_witness(q, k, v, scale, is_causal=False, mask=None, sliding_window=0, sinks=None):
    """torch CPU SDPA in float64 on BSHD inputs; returns BSHD float64."""
    B, Sq, Hq, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    qd, kd, vd = (t.double().permute(0, 2, 1, 3) for t in (q, k, v))
    i = torch.arange(Sq).view(Sq, 1)
    j = torch.arange(Sk).view(1, Sk)
    visible = torch.ones(Sq, Sk, dtype=torch.bool)
    if is_causal:
        visible &= j <= i + (Sk - Sq)
    if sliding_window > 0:
        visible &= j > i + (Sk - Sq) - sliding_window
    bias = torch.zeros(B, Hq, Sq, Sk, dtype=torch.float64)
    if mask is not None:
        bias = bias + mask.double()
    bias = bias.masked_fill(~visible, float("-inf"))
    if sinks is not None:
        # one more key per KV head would be shared by the group's query heads, but a sink is per QUERY head: expand
        # the KV heads instead of using enable_gqa, then append a key column whose score is the sink logit
        G = Hq // Hkv
        kd, vd = kd.repeat_interleave(G, dim=1), vd.repeat_interleave(G, dim=1)
        kd = torch.cat([kd, torch.zeros(B, Hq, 1, D, dtype=torch.float64)], dim=2)
        vd = torch.cat([vd, torch.zeros(B, Hq, 1, D, dtype=torch.float64)], dim=2)
        sink_col = sinks.double().view(1, Hq, 1, 1).expand(B, Hq, Sq, 1)
        bias = torch.cat([bias, sink_col], dim=3)  # q . 0 = 0, so the column's score is exactly the sink
        out = F.scaled_dot_product_attention(qd, kd, vd, attn_mask=bias, scale=scale)
    else:
        out = F.scaled_dot_product_attention(qd, kd, vd, attn_mask=bias, scale=scale, enable_gqa=Hq != Hkv)
    # rows with no visible key: torch yields NaN (softmax over -inf only); the operator defines them as zeros
    dead = ~visible.any(dim=1) if sinks is None else torch.zeros(Sq, dtype=torch.bool)
    out = out.permute(0, 2, 1, 3).contiguous()
    out[:, dead] = 0.0
    return out


# the five benchmark configurations shrunk (same head counts / head dims / ratios), then the ragged, grouped and
# Sq < Sk cases the oracle's own tests use
CASES = [
    # B, Sq, Sk, Hq, Hkv, D, causal, scale, seeds-scale
    ("sd15_self", 2, 96, 96, 8, 8, 40, False),
    ("sdxl_cross", 2, 128, 77, 20, 20, 64, False),
    ("flux_joint", 1, 144, 144, 24, 24, 128, False),
    ("wan_self", 1, 211, 211, 5, 5, 128, False),
    ("decode_gqa", 3, 1, 517, 32, 8, 128, True),
    ("ragged", 2, 33, 50, 4, 2, 40, False),
    ("gqa_causal_sq_lt_sk", 1, 5, 70, 8, 2, 64, True),
    ("square_causal", 1, 64, 64, 2, 2, 128, True),
    ("single_key", 2, 17, 1, 3, 3, 16, False),
    ("sq_gt_sk_causal", 1, 7, 3, 2, 1, 8, True),
    ("verify_4_tokens", 1, 4, 200, 16, 4, 256, True),
]


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_oracles_agree_with_torch_sdpa(case):
    _, B, Sq, Sk, Hq, Hkv, D, causal = case
    q = so.seeded_normal((B, Sq, Hq, D), 101)
    k = so.seeded_normal((B, Sk, Hkv, D), 102)
    v = so.seeded_normal((B, Sk, Hkv, D), 103)
    scale = D ** -0.5
    want = torch_witness(q, k, v, scale, causal)
    py64 = so.sdpa_explicit(q, k, v, scale, causal, compute_dtype=torch.float64)
    py32 = so.sdpa_explicit(q, k, v, scale, causal)
    c32 = c_oracle.sdpa_c(q, k, v, scale, causal)
    assert so.error_stats(py64, want)[0] < 1e-12
    assert so.error_stats(py32, want)[0] < 3e-6
    assert so.error_stats(c32, want)[0] < 3e-6


def test_flux_inputs_with_rope_agree_with_torch_sdpa():
    """The benchmark's Flux inputs are rotated before the call (Flux1.swift:187-188): same check on those."""
    H, D, text, side = 3, 128, 32, 8
    S = text + side * side
    q, k, v = (so.seeded_normal((1, S, H, D), s) for s in (2, 3, 4))
    rot = so.flux_rope_table(side, side, text, D)
    q, k = so.cmul(q, rot), so.cmul(k, rot)
    want = torch_witness(q, k, v, D ** -0.5)
    assert so.error_stats(so.sdpa_explicit(q, k, v, D ** -0.5, compute_dtype=torch.float64), want)[0] < 1e-12
    assert so.error_stats(c_oracle.sdpa_c(q, k, v, D ** -0.5), want)[0] < 3e-6


@pytest.mark.parametrize("bshape", [(1, 1), (2, 1), (1, 4), (2, 4)])
def test_additive_mask_agrees_with_torch_sdpa(bshape):
    """[B or 1, H or 1, Sq, Sk] additive mask with the reference's finite fill (CLIPTextModel.swift:46-51,
    TextEncoder.swift:147-158), alone and on top of the causal rule (Llama.swift:70-73)."""
    B, Sq, Sk, H, D = 2, 19, 31, 4, 32
    q, k, v = so.seeded_normal((B, Sq, H, D), 5), so.seeded_normal((B, Sk, H, D), 6), so.seeded_normal((B, Sk, H, D), 7)
    g = torch.Generator().manual_seed(9)
    mask = torch.randn(bshape[0], bshape[1], Sq, Sk, generator=g)
    mask = mask.masked_fill(torch.rand(bshape[0], bshape[1], Sq, Sk, generator=g) < 0.3, so.MASK_FILL)
    mask[..., 0] = 0.0  # every row keeps one visible key
    for causal in (False, True):
        want = torch_witness(q, k, v, 0.2, causal, mask=mask)
        assert so.error_stats(so.sdpa_explicit(q, k, v, 0.2, causal, mask, compute_dtype=torch.float64), want)[0] < 1e-10
        assert so.error_stats(c_oracle.sdpa_c(q, k, v, 0.2, causal, mask=mask), want)[0] < 3e-6


@pytest.mark.parametrize("Sq,Sk,W", [(1, 300, 128), (6, 40, 5), (32, 32, 7), (9, 64, 100)])
def test_sliding_window_and_sinks_agree_with_torch_sdpa(Sq, Sk, W):
    """hasAttentionSinks / slidingWindow (DeepSeek4.swift:482-493) in the forms torch understands."""
    B, Hq, Hkv, D = 2, 8, 2, 64
    q = so.seeded_normal((B, Sq, Hq, D), 21)
    k = so.seeded_normal((B, Sk, Hkv, D), 22)
    v = so.seeded_normal((B, Sk, Hkv, D), 23)
    sinks = so.seeded_normal((Hq,), 24) * 2.0
    for use_sinks in (False, True):
        s = sinks if use_sinks else None
        want = torch_witness(q, k, v, D ** -0.5, True, sliding_window=W, sinks=s)
        got = so.sdpa_explicit(q, k, v, D ** -0.5, True, sinks=s, sliding_window=W, compute_dtype=torch.float64)
        assert so.error_stats(got, want)[0] < 1e-12


def test_variable_length_agrees_with_torch_sdpa():
    """Packed sequences (Qwen3_5VL.swift:428-437): the witness is torch SDPA on each sequence by itself."""
    Hq, Hkv, D = 4, 2, 32
    offs_q, offs_k = [0, 7, 7, 30, 41], [0, 9, 9, 29, 60]
    q = so.seeded_normal((1, offs_q[-1], Hq, D), 31)
    k = so.seeded_normal((1, offs_k[-1], Hkv, D), 32)
    v = so.seeded_normal((1, offs_k[-1], Hkv, D), 33)
    got = so.sdpa_varlen_explicit(q, k, v, 0.3, offs_q, offs_k, compute_dtype=torch.float64)
    for s in range(len(offs_q) - 1):
        q0, q1, k0, k1 = offs_q[s], offs_q[s + 1], offs_k[s], offs_k[s + 1]
        if q1 > q0:
            want = torch_witness(q[:, q0:q1], k[:, k0:k1], v[:, k0:k1], 0.3)
            assert so.error_stats(got[:, q0:q1], want)[0] < 1e-12


def test_log_sum_exp_agrees_with_torch():
    B, Sq, Sk, H, D = 1, 12, 45, 2, 16
    q, k, v = so.seeded_normal((B, Sq, H, D), 41), so.seeded_normal((B, Sk, H, D), 42), so.seeded_normal((B, Sk, H, D), 43)
    _, lse = so.sdpa_explicit(q, k, v, 0.25, True, compute_dtype=torch.float64, return_lse=True)
    _, lse_c = c_oracle.sdpa_c(q, k, v, 0.25, True, return_lse=True)
    s = torch.einsum("bqhd,bkhd->bhqk", q.double(), k.double()) * 0.25
    i, j = torch.arange(Sq).view(Sq, 1), torch.arange(Sk).view(1, Sk)
    want = torch.logsumexp(s.masked_fill(j > i + (Sk - Sq), float("-inf")), dim=-1)
    assert torch.allclose(lse, want, atol=1e-12) and torch.allclose(lse_c.double(), want, atol=3e-6)
