"""Sparse indexed attention (SparseIndexedAttention, DeepSeek4.swift:521-545) through the C ABI against the CPU oracle:
raw rows under the causal sliding window plus per-query selected rows of a compressed tensor, one softmax, sinks."""
import ctypes

import pytest
import torch

from oracle import sdpa_oracle as so

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ROUND = {torch.float16: 2.0 ** -11, torch.bfloat16: 2.0 ** -9, torch.float32: 0.0}


def make_case(B, Sq, Sr, Sc, n_sel, Hq, Hkv, D, dtype, seed, per_batch_lists=False):
    q = so.seeded_normal((B, Sq, Hq, D), seed).to(dtype)
    kr = so.seeded_normal((B, Sr, Hkv, D), seed + 1).to(dtype)
    vr = so.seeded_normal((B, Sr, Hkv, D), seed + 2).to(dtype)
    kc = so.seeded_normal((B, max(Sc, 1), Hkv, D), seed + 3).to(dtype)[:, :Sc]
    vc = so.seeded_normal((B, max(Sc, 1), Hkv, D), seed + 4).to(dtype)[:, :Sc]
    g = torch.Generator().manual_seed(seed)
    # lists with duplicates, "no row" entries (-1 and beyond the end) and, for some queries, nothing valid at all
    sel = torch.randint(-2, Sc + 2, (B if per_batch_lists else 1, Sq, n_sel), generator=g, dtype=torch.int32)
    sel[:, ::5] = -1
    sinks = (so.seeded_normal((Hq,), seed + 5) * 2).to(dtype)
    return q, kr, vr, kc, vc, sel, sinks


CASES = [
    # B, Sq, Sr, Sc, n_sel, Hq, Hkv, D, dtype, window
    (1, 1, 600, 150, 64, 64, 1, 512, torch.float16, 128),     # the reference's decode step: 64 heads over one KV head, dim 512
    (1, 40, 40, 10, 10, 16, 1, 512, torch.bfloat16, 16),      # a short prefill: every query lists all compressed rows
    (2, 33, 70, 21, 9, 8, 2, 128, torch.float16, 20),         # grouped heads, Sq < Sr, batch
    (1, 17, 17, 0, 0, 4, 4, 64, torch.float32, 5),            # no compressed rows at all
    (2, 9, 30, 12, 40, 6, 3, 96, torch.float32, 0),           # no window: causal over all raw rows; more entries than rows
    (1, 5, 12, 8, 3, 24, 1, 40, torch.bfloat16, 100),         # 24 heads per KV head (two CTAs of 12), window wider than the rows
    # the tensor-core kernel (16-bit, head dim a multiple of 64):
    (1, 1, 9000, 2048, 512, 64, 1, 512, torch.bfloat16, 128),  # the decode step at length: 20 tiles over a cluster of 8 CTAs
    (1, 2, 700, 300, 130, 64, 1, 512, torch.float16, 128),    # two new tokens: cluster of 4, a last tile of 2 keys
    (1, 70, 70, 20, 20, 64, 1, 512, torch.bfloat16, 128),     # a prefill: one CTA per token and head group, no cluster
    (2, 33, 40, 16, 7, 24, 1, 128, torch.float16, 9),         # 24 heads per KV head: a group of 16 and a group of 8; batch
    (1, 50, 90, 30, 33, 12, 3, 64, torch.bfloat16, 0),        # three KV heads of 4 query heads, no window, head dim 64
    (1, 3, 300, 0, 0, 32, 2, 256, torch.float16, 40),         # no compressed rows, head dim 256
]


@pytest.mark.parametrize("forced", [False, True])
@pytest.mark.parametrize("case", CASES)
def test_sparse_indexed_attention(dtattn, case, forced):
    """Every case on the kernel the library picks and on the CUDA-core kernel (DT_FLAG_FORCE_GENERIC)."""
    B, Sq, Sr, Sc, n_sel, Hq, Hkv, D, dtype, window = case
    q, kr, vr, kc, vc, sel, sinks = make_case(B, Sq, Sr, Sc, n_sel, Hq, Hkv, D, dtype, 801, per_batch_lists=B > 1)
    dev = lambda t: t.to(DEV)
    lse = torch.full((B, Hq, Sq), float("nan"), dtype=torch.float32, device=DEV)
    out = dtattn.sparse_indexed_attention(dev(q), dev(kr), dev(vr), dev(kc) if Sc else None, dev(vc) if Sc else None,
                                          dev(sel) if n_sel else None, D ** -0.5, dev(sinks), window, lse=lse,
                                          flags=dtattn.DT_FLAG_FORCE_GENERIC if forced else 0)
    torch.cuda.synchronize()
    ref, ref_lse = so.sparse_indexed_explicit(q, kr, vr, kc if Sc else None, vc if Sc else None, sel if n_sel else None,
                                              D ** -0.5, sinks, window, compute_dtype=torch.float64, return_lse=True)
    got = out.float().cpu()
    assert torch.isfinite(got).all()
    mx, mean = so.error_stats(got, ref.float())
    assert mx <= so.TOL_MAX_ABS + 2 * ROUND[dtype] * float(ref.abs().max()), (case, mx)
    assert mean <= so.TOL_MEAN_ABS + ROUND[dtype] * float(ref.abs().mean()), (case, mean)
    assert (lse.cpu().double() - ref_lse).abs().max() < 2e-3


def test_operator_mirror_and_equivalence_with_the_window_operator(dtattn):
    """With no valid selected row the operator is ScaledDotProductAttention(isCausal, hasAttentionSinks, slidingWindow)
    (DeepSeek4.swift:482-493), which the other kernels serve: same inputs, same result."""
    B, Sq, Sr, Hq, D, dtype = 1, 64, 300, 8, 128, torch.float16
    q, kr, vr, kc, vc, sel, sinks = make_case(B, Sq, Sr, 16, 4, Hq, 1, D, dtype, 811)
    sel.fill_(-1)
    op = dtattn.SparseIndexedAttention(scale=D ** -0.5, is_causal=True, has_attention_sinks=True, sliding_window=128)
    a = op(q.to(DEV), kr.to(DEV), vr.to(DEV), kc.to(DEV), vc.to(DEV), sel[0].to(DEV), sinks.view(1, 1, Hq, 1).to(DEV))
    b = dtattn.sdpa_forward(q.to(DEV), kr.to(DEV), vr.to(DEV), D ** -0.5, True, sinks=sinks.to(DEV), sliding_window=128)
    torch.cuda.synchronize()
    assert (a.float() - b.float()).abs().max() <= 2e-3


@pytest.mark.parametrize("shape", [(9, 200, 64, 40), (70, 400, 200, 150), (130, 130, 33, 200)])
def test_keys_that_are_also_the_values(dtattn, shape):
    """The reference's layout (DeepSeek4.swift:489-491): one tensor serves as keys and values; the tensor-core kernel
    then gathers each row once, and with enough tokens and keys works on 64 keys per step instead of 32 (the second
    and third shape; the third has a last tile of 6 keys and lists longer than the compressed tensor).  Also without
    sinks, and with a strided (row-padded) view."""
    Sq, Sr, Sc, n_sel = shape
    B, Hq, D, dtype = 1, 64, 512, torch.bfloat16
    q, kr, _, kc, _, sel, sinks = make_case(B, Sq, Sr, Sc, n_sel, Hq, 1, D, dtype, 821)
    big_r = torch.zeros(B, Sr, 1, D + 64, dtype=dtype)
    big_r[..., :D] = kr
    kr_view = big_r[..., :D]  # rows 576 elements apart
    ref = so.sparse_indexed_explicit(q, kr_view, kr_view, kc, kc, sel, D ** -0.5, None, 128, compute_dtype=torch.float64)
    kd, cd = big_r.to(DEV)[..., :D], kc.to(DEV)
    for flags in (0, dtattn.DT_FLAG_FORCE_GENERIC):
        out = dtattn.sparse_indexed_attention(q.to(DEV), kd, kd, cd, cd, sel.to(DEV), D ** -0.5, None, 128, flags=flags)
        torch.cuda.synchronize()
        mx, mean = so.error_stats(out.float().cpu(), ref.float())
        assert mx <= so.TOL_MAX_ABS + 2 * ROUND[dtype] * float(ref.abs().max()) and mean <= 2 * so.TOL_MEAN_ABS, (flags, mx, mean)


def test_sparse_indexed_bad_arguments(dtattn):
    lib = dtattn.lib()
    p = dtattn.SparseIndexedParams()
    assert lib.dt_sparse_indexed_attention(None, None) == dtattn.DT_BAD_ARG
    assert lib.dt_sparse_indexed_attention(ctypes.byref(p), None) == dtattn.DT_BAD_ARG  # all zero
    p.B, p.Sq, p.Hq, p.Hkv, p.D, p.Sr, p.dtype, p.scale = 1, 1, 4, 3, 64, 8, 0, 1.0
    assert lib.dt_sparse_indexed_attention(ctypes.byref(p), None) == dtattn.DT_BAD_ARG  # heads do not divide
    p.Hkv, p.D = 1, 1024
    t = torch.zeros(64, dtype=torch.float16, device=DEV)
    for name in ("q", "o", "k_raw", "v_raw"):
        setattr(p, name, dtattn.Tensor4(t.data_ptr(), 0, 0, 0))
    assert lib.dt_sparse_indexed_attention(ctypes.byref(p), None) == dtattn.DT_UNSUPPORTED  # head dim beyond 512
