"""GPU parity tests: every call goes through the C ABI (dtattn -> libdtattn.so) and is compared with the CPU
oracle on the same seeded inputs.

Tolerance (stated by the task for fp16/bf16 against the fp32 oracle): max-abs <= 2e-3 and mean-abs <= 2e-4.
Where a small test shape makes |O| approach 1, the output's own rounding (2^-9 relative for bf16, 2^-11 for
fp16) is added to the max-abs bound; the benchmark shapes are held to the plain figures.
"""
import ctypes
import math

import pytest
import torch

from oracle import c_oracle
from oracle import sdpa_oracle as so

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
ROUND = {torch.float16: 2.0 ** -11, torch.bfloat16: 2.0 ** -9, torch.float32: 0.0}


def oracle(q, k, v, scale, causal=False, mask=None):
    """fp32 C oracle for anything sizeable, float64 explicit form for tiny cases."""
    B, Sq, Hq, D = q.shape
    if B * Hq * Sq * k.shape[1] * D <= 1 << 22:
        return so.sdpa_explicit(q, k, v, scale, causal, mask, compute_dtype=torch.float64).float()
    return c_oracle.sdpa_c(q, k, v, scale, causal, mask)


def check(out, ref, dtype, what="", strict=False):
    """strict: the plain figures (benchmark shapes).  Otherwise the rounding of a 16-bit result is added:
    P is rounded to the I/O type before P*V (as the reference's explicit graph does, UNet.swift:257-259) and
    O is rounded once more on output, so a result of magnitude |O| carries up to ~2 ulp of it."""
    out = out.float().cpu()
    assert torch.isfinite(out).all(), f"{what}: non-finite output"
    mx, mean = so.error_stats(out, ref)
    bound_max = so.TOL_MAX_ABS + (0.0 if strict else 2 * ROUND[dtype] * float(ref.abs().max()))
    bound_mean = so.TOL_MEAN_ABS + (0.0 if strict else ROUND[dtype] * float(ref.abs().mean()))
    assert mx <= bound_max and mean <= bound_mean, \
        f"{what}: max-abs {mx:.3e} (bound {bound_max:.3e}) mean-abs {mean:.3e} (bound {bound_mean:.3e})"
    return mx, mean


def run(dtattn, q, k, v, scale, causal=False, mask=None, flags=0, lse=None):
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    md = mask.to(DEV) if mask is not None else None
    out = dtattn.sdpa_forward(qd, kd, vd, scale, causal, md, flags=flags, lse=lse)
    torch.cuda.synchronize()
    assert dtattn.device_status() == 0, "a device-side wait ran out"
    return out


def inputs(B, Sq, Sk, Hq, Hkv, D, dtype, seed, scale=1.0):
    q = so.seeded_normal((B, Sq, Hq, D), seed, scale).to(dtype)
    k = so.seeded_normal((B, Sk, Hkv, D), seed + 1, scale).to(dtype)
    v = so.seeded_normal((B, Sk, Hkv, D), seed + 2, scale).to(dtype)
    return q, k, v


# --------------------------------------------------------------------------------------------------
# generic (CUDA-core) kernel: any head dim, fp32, masks
# --------------------------------------------------------------------------------------------------

GENERIC = [
    # B, Sq, Sk, Hq, Hkv, D, dtype, causal
    (2, 48, 48, 8, 8, 40, torch.float32, False),      # SD1.5 head dim, upcast (fp32) attention
    (1, 33, 70, 4, 2, 80, torch.float16, False),
    (1, 20, 20, 2, 2, 160, torch.float16, True),
    (2, 9, 300, 4, 1, 256, torch.bfloat16, True),
    (1, 7, 3, 2, 1, 8, torch.float32, True),          # Sq > Sk causal: first rows see no key -> zeros
    (1, 1, 1, 1, 1, 16, torch.float32, False),
]


@pytest.mark.parametrize("case", GENERIC)
def test_generic_kernel(dtattn, case):
    B, Sq, Sk, Hq, Hkv, D, dtype, causal = case
    q, k, v = inputs(B, Sq, Sk, Hq, Hkv, D, dtype, 21)
    out = run(dtattn, q, k, v, D ** -0.5, causal)
    check(out, oracle(q, k, v, D ** -0.5, causal), dtype, str(case))


def test_generic_mask_and_lse(dtattn):
    """CLIP-style additive causal mask (CLIPTextModel.swift:46-51) with -greatestFiniteMagnitude fill, plus LSE."""
    B, S, H, D = 2, 77, 4, 64
    for dtype in (torch.float32, torch.float16):
        q, k, v = inputs(B, S, S, H, H, D, dtype, 31)
        mask = torch.zeros(1, 1, S, S, dtype=dtype)
        mask.masked_fill_(torch.triu(torch.ones(S, S, dtype=torch.bool), 1), -torch.finfo(dtype).max)
        lse = torch.empty(B, H, S, dtype=torch.float32, device=DEV)
        out = run(dtattn, q, k, v, D ** -0.5, False, mask, lse=lse)
        ref, ref_lse = so.sdpa_explicit(q, k, v, D ** -0.5, True, compute_dtype=torch.float64, return_lse=True)
        check(out, ref.float(), dtype, "masked")
        assert (lse.cpu().double() - ref_lse).abs().max() < 2e-3


def test_sd15_self_attention_full_size(dtattn):
    """configs[0] shape on the GPU: [2,4096,8,40] fp32, against the C oracle on a sample of query rows."""
    cfg = so.CONFIGS["sd15_self"]
    q, k, v = so.make_inputs(cfg)
    out = run(dtattn, q, k, v, cfg.scale)
    rows = torch.arange(0, cfg.Sq, 37)
    ref = c_oracle.sdpa_c(q[:, rows].contiguous(), k, v, cfg.scale)
    check(out[:, rows.to(DEV)], ref, torch.float32, "sd15", strict=True)


# --------------------------------------------------------------------------------------------------
# decode (split-KV) kernel
# --------------------------------------------------------------------------------------------------

DECODE = [
    # B, Sq, Sk, Hq, Hkv, D, dtype
    (1, 1, 256, 8, 2, 128, torch.float16),
    (2, 1, 1000, 32, 8, 128, torch.float16),      # ragged: 1000 = 62*16 + 8
    (3, 1, 515, 8, 8, 64, torch.bfloat16),        # MHA decode, head dim 64
    (1, 4, 777, 8, 2, 128, torch.bfloat16),       # multi-token verify: 4 new tokens x 4 heads = 16 rows
    (1, 2, 4096, 16, 2, 128, torch.float16),      # group of 8
    (2, 1, 8192, 16, 4, 64, torch.float16),
    (1, 1, 4096, 16, 4, 256, torch.bfloat16),     # the reference's Qwen3.5 attention: head dim 256, 4 KV heads (Qwen3_5.swift:59-82)
    (2, 2, 1000, 24, 4, 256, torch.float16),      # 24 query heads: groups of 6, two new tokens -> 12 rows
    (1, 1, 300, 4, 4, 256, torch.float16),
]


@pytest.mark.parametrize("case", DECODE)
def test_decode_kernel(dtattn, case):
    B, Sq, Sk, Hq, Hkv, D, dtype = case
    q, k, v = inputs(B, Sq, Sk, Hq, Hkv, D, dtype, 41)
    p = dtattn.make_params(q, k, v, q, D ** -0.5, True)
    assert dtattn.kernel_name(p) == "decode_splitkv"
    out = run(dtattn, q, k, v, D ** -0.5, True)
    check(out, oracle(q, k, v, D ** -0.5, True), dtype, str(case))


@pytest.mark.parametrize("B", [1, 16])
def test_decode_config_full_size(dtattn, B):
    """configs[4]: 32 query heads, 8 KV heads, d128, 8192 cached rows, fp16; also through a cache VIEW
    ([B, capacity, Hkv, D] with only the first T rows visible, Qwen3_5TextGeneration.swift:1661-1684)."""
    cfg = so.CONFIGS["decode_b16" if B == 16 else "decode_b1"]
    q, k, v = so.make_inputs(cfg)
    ref = c_oracle.sdpa_c(q, k, v, cfg.scale, True)
    lse = torch.empty(B, cfg.Hq, 1, dtype=torch.float32, device=DEV)
    out = run(dtattn, q, k, v, cfg.scale, True, lse=lse)
    check(out, ref, torch.float16, "decode", strict=True)
    ref_lse = so.sdpa_explicit(q[:1], k[:1], v[:1], cfg.scale, True, return_lse=True)[1]
    assert (lse[:1].cpu() - ref_lse).abs().max() < 2e-3
    # cache view: capacity 8192 + 64, prefix of 8192 rows, rest holds NaN that must never be read
    cap = cfg.Sk + 64
    kc = torch.full((B, cap, cfg.Hkv, cfg.D), float("nan"), dtype=torch.float16, device=DEV)
    vc = torch.full_like(kc, float("nan"))
    kc[:, :cfg.Sk] = k.to(DEV)
    vc[:, :cfg.Sk] = v.to(DEV)
    out2 = dtattn.sdpa_forward(q.to(DEV), kc[:, :cfg.Sk], vc[:, :cfg.Sk], cfg.scale, True)
    torch.cuda.synchronize()
    assert torch.equal(out2, out), "a strided cache view must give bitwise the same result"
    # determinism: the ticketed combine reads partials in a fixed order
    out3 = run(dtattn, q, k, v, cfg.scale, True)
    assert torch.equal(out3, out)


def test_decode_workspace_contract(dtattn):
    """Too small a workspace is refused; the workspace is left clean for the next call."""
    cfg = so.CONFIGS["decode_b1"]
    q, k, v = (t.to(DEV) for t in so.make_inputs(cfg))
    o = torch.empty_like(q)
    p = dtattn.make_params(q, k, v, o, cfg.scale, True)
    need = dtattn.workspace_size(p)
    assert need > 0
    lib = dtattn.lib()
    s = torch.cuda.current_stream().cuda_stream
    assert lib.dt_sdpa_forward(ctypes.byref(p), None, 0, ctypes.c_void_p(s)) == dtattn.DT_WORKSPACE
    ws = torch.empty(need, dtype=torch.uint8, device=DEV)
    assert lib.dt_sdpa_forward(ctypes.byref(p), ctypes.c_void_p(ws.data_ptr()), need - 1, ctypes.c_void_p(s)) == dtattn.DT_WORKSPACE
    assert lib.dt_sdpa_workspace_init(ctypes.c_void_p(ws.data_ptr()), need, ctypes.c_void_p(s)) == 0
    outs = []
    for _ in range(3):
        assert lib.dt_sdpa_forward(ctypes.byref(p), ctypes.c_void_p(ws.data_ptr()), need, ctypes.c_void_p(s)) == 0
        torch.cuda.synchronize()
        outs.append(o.clone())
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[1], outs[2])
    assert int(ws[:4096].view(torch.int32)[: cfg.B * cfg.Hkv].abs().sum()) == 0, "ticket counters must return to zero"


def test_decode_shapes_share_one_workspace(dtattn):
    """Calls of different shapes through the same workspace: the ticket counters of one call must never
    land where another call left partial results."""
    ws = dtattn.Workspace(torch.device(DEV))
    shapes = [(1, 1, 8192, 32, 8, 128), (16, 1, 4096, 32, 8, 128), (2, 4, 2000, 16, 4, 128), (16, 1, 4096, 32, 8, 128),
              (1, 1, 8192, 32, 8, 128)]
    for i, (B, Sq, Sk, Hq, Hkv, D) in enumerate(shapes):
        q, k, v = inputs(B, Sq, Sk, Hq, Hkv, D, torch.float16, 200 + i)
        out = dtattn.sdpa_forward(q.to(DEV), k.to(DEV), v.to(DEV), D ** -0.5, True, workspace=ws)
        torch.cuda.synchronize()
        check(out, oracle(q, k, v, D ** -0.5, True), torch.float16, f"shared workspace {i}")


# --------------------------------------------------------------------------------------------------
# tcgen05 prefill kernel
# --------------------------------------------------------------------------------------------------

PREFILL = [
    # B, Sq, Sk, Hq, Hkv, D, dtype, causal
    (1, 128, 128, 1, 1, 128, torch.bfloat16, False),   # one tile, one block
    (1, 256, 128, 1, 1, 128, torch.bfloat16, False),   # both tiles
    (1, 256, 512, 2, 2, 128, torch.bfloat16, False),   # several blocks: online softmax + rescale
    (1, 256, 1536, 2, 2, 128, torch.float16, False),   # ring wraps (12 K/V blocks through 5 slots)
    (2, 300, 333, 3, 3, 128, torch.bfloat16, False),   # ragged rows and keys, batch
    (1, 128, 77, 2, 2, 64, torch.float16, False),      # SDXL cross-attention shape, head dim 64
    (2, 500, 77, 4, 4, 64, torch.float16, False),      # (larger short-key shapes take the dedicated kernel: test_gpu_short_kv.py)
    (1, 512, 512, 4, 2, 64, torch.bfloat16, False),    # grouped KV heads
    (1, 384, 384, 2, 2, 128, torch.bfloat16, True),    # causal
    (1, 200, 456, 2, 1, 128, torch.float16, True),     # causal, bottom-right aligned, ragged
    (1, 100, 100, 1, 1, 64, torch.bfloat16, True),
    (2, 320, 320, 8, 8, 40, torch.float16, False),     # SD1.5 head dims in half precision: zero-padded to 64 / 128 by TMA
    (1, 200, 300, 4, 4, 80, torch.float16, False),
    (1, 130, 77, 2, 2, 96, torch.bfloat16, False),
    (1, 256, 256, 2, 1, 8, torch.float16, True),
    # head dim 256 (AuraFlow.swift:358, Gemma3.swift:148, the shipped Qwen3.5 configs): one 128-row tile per work item
    (1, 128, 128, 1, 1, 256, torch.bfloat16, False),   # one tile, one block
    (1, 300, 700, 3, 3, 256, torch.bfloat16, False),   # ragged rows and keys, six blocks through the two-slot ring
    (2, 640, 640, 4, 2, 256, torch.float16, True),     # causal, grouped KV heads, batch
    (1, 200, 456, 2, 1, 256, torch.float16, True),     # causal, bottom-right aligned, ragged
    (1, 260, 300, 2, 2, 160, torch.float16, False),    # SD1.5's deepest blocks: D = 160 zero-padded to 256
    (1, 256, 256, 2, 2, 192, torch.bfloat16, True),
]


@pytest.mark.parametrize("case", PREFILL)
def test_prefill_kernel(dtattn, case):
    B, Sq, Sk, Hq, Hkv, D, dtype, causal = case
    scale_in = 0.5 if D == 64 else 1.0
    q, k, v = inputs(B, Sq, Sk, Hq, Hkv, D, dtype, 51, scale_in)
    p = dtattn.make_params(q, k, v, q, D ** -0.5, causal)
    assert dtattn.kernel_name(p) == "prefill_tcgen05"
    lse = torch.empty(B, Hq, Sq, dtype=torch.float32, device=DEV)
    out = run(dtattn, q, k, v, D ** -0.5, causal, lse=lse)
    check(out, oracle(q, k, v, D ** -0.5, causal), dtype, str(case))
    ref_lse = so.sdpa_explicit(q, k, v, D ** -0.5, causal, return_lse=True)[1]
    assert (lse.cpu() - ref_lse).abs().max() < 5e-3


def test_prefill_large_magnitude_scores(dtattn):
    """Scores that grow block after block force the O rescale path (the row max rises by far more than 2^8)."""
    B, S, H, D = 1, 640, 1, 128
    q, k, v = inputs(B, S, S, H, H, D, torch.bfloat16, 61)
    ramp = torch.linspace(0.2, 3.0, S).view(1, S, 1, 1)
    k = (k.float() * ramp).to(torch.bfloat16)
    out = run(dtattn, q, k, v, 1.0)     # scale 1: scores of magnitude ~ 30..100
    check(out, oracle(q, k, v, 1.0), torch.bfloat16, "large scores")


def test_prefill_large_magnitude_scores_head_dim_256(dtattn):
    """The same at head dim 256, where S is double-buffered and a block's scores arrive before the previous block's
    P*V has run: the O rescale has to wait for that P*V.  Many rows, several heads and a causal variant, so that the
    rescale happens in most blocks of most tiles."""
    B, S, H, D = 1, 1280, 4, 256
    q, k, v = inputs(B, S, S, H, H, D, torch.bfloat16, 63)
    ramp = torch.linspace(0.1, 2.0, S).view(1, S, 1, 1)
    k = (k.float() * ramp).to(torch.bfloat16)
    for causal in (False, True):
        out = run(dtattn, q, k, v, 0.5, causal)     # scores of magnitude up to ~ 250: the row max rises block after block
        check(out, oracle(q, k, v, 0.5, causal), torch.bfloat16, f"large scores d256 causal={causal}")


def test_prefill_strided_views(dtattn):
    """Row-offset and batch-strided views are honoured without a copy (Flux1.swift:236-243, UNet.swift:334-344)."""
    B, S, H, D, dtype = 2, 300, 2, 128, torch.bfloat16
    big = so.seeded_normal((B, S + 40, 3 * H, D), 71).to(dtype).to(DEV)   # fused qkv-like buffer
    q = big[:, 40:, 0:H]
    k = big[:, :S, H:2 * H]
    v = big[:, 20:S + 20, 2 * H:3 * H]
    obuf = torch.zeros((B, S + 8, H, D), dtype=dtype, device=DEV)
    out = obuf[:, 8:]
    dtattn.sdpa_forward(q, k, v, D ** -0.5, out=out)
    torch.cuda.synchronize()
    assert dtattn.device_status() == 0
    ref = oracle(q.cpu().contiguous(), k.cpu().contiguous(), v.cpu().contiguous(), D ** -0.5)
    check(out, ref, dtype, "strided")
    assert float(obuf[:, :8].abs().sum()) == 0.0, "rows outside the output view were written"


def test_prefill_matches_generic_kernel(dtattn):
    """Two independent GPU implementations agree on a shape too big for the CPU oracle to cover fully."""
    B, S, H, D, dtype = 1, 2048, 6, 128, torch.bfloat16
    q, k, v = (t.to(DEV) for t in inputs(B, S, S, H, H, D, dtype, 81))
    a = dtattn.sdpa_forward(q, k, v, D ** -0.5)
    b = dtattn.sdpa_forward(q, k, v, D ** -0.5, flags=dtattn.DT_FLAG_FORCE_GENERIC)
    torch.cuda.synchronize()
    mx, mean = so.error_stats(a.float().cpu(), b.float().cpu())
    assert mx <= 2e-3 and mean <= 2e-4, (mx, mean)


def test_sdxl_cross_attention_full_size(dtattn):
    """configs[1]: Q [2,4096,20,64], K/V [2,77,20,64] fp16, N(0,1)*0.5."""
    cfg = so.CONFIGS["sdxl_cross"]
    q, k, v = so.make_inputs(cfg)
    out = run(dtattn, q, k, v, cfg.scale)
    check(out, c_oracle.sdpa_c(q, k, v, cfg.scale), torch.float16, "sdxl", strict=True)


def test_flux_joint_attention_full_size(dtattn):
    """configs[2]: [1,4608,24,128] bf16 with Flux RoPE pre-applied; C oracle on every 9th query row, plus
    size-independent properties on the full tensor."""
    cfg = so.CONFIGS["flux_joint"]
    q, k, v = so.make_inputs(cfg)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    out = dtattn.sdpa_forward(qd, kd, vd, cfg.scale)
    torch.cuda.synchronize()
    assert dtattn.device_status() == 0
    rows = torch.arange(0, cfg.Sq, 9)
    ref = c_oracle.sdpa_c(q[:, rows].contiguous(), k, v, cfg.scale)
    check(out[:, rows.to(DEV)], ref, torch.bfloat16, "flux", strict=True)
    # determinism
    assert torch.equal(dtattn.sdpa_forward(qd, kd, vd, cfg.scale), out)
    # rows of P sum to one: with V = 1 the output is exactly 1 up to bf16 rounding of P
    ones = torch.ones_like(vd)
    o1 = dtattn.sdpa_forward(qd, kd, ones, cfg.scale).float()
    assert float((o1 - 1).abs().max()) <= 2 ** -7
    # permuting the keys (K and V rows together) leaves the result unchanged
    perm = torch.randperm(cfg.Sk, generator=torch.Generator().manual_seed(5)).to(DEV)
    op = dtattn.sdpa_forward(qd, kd[:, perm].contiguous(), vd[:, perm].contiguous(), cfg.scale)
    mx, mean = so.error_stats(op.float().cpu(), out.float().cpu())
    assert mx <= 2e-3 and mean <= 2e-4, (mx, mean)
    # linear in V
    v2 = so.seeded_normal(tuple(v.shape), 99).to(torch.bfloat16).to(DEV)
    o2 = dtattn.sdpa_forward(qd, kd, v2, cfg.scale).float()
    o12 = dtattn.sdpa_forward(qd, kd, (vd.float() * 0.5 + v2.float() * 0.25).to(torch.bfloat16), cfg.scale).float()
    mx, mean = so.error_stats((0.5 * out.float() + 0.25 * o2).cpu(), o12.cpu())
    assert mx <= 4e-3 and mean <= 4e-4, (mx, mean)
    torch.cuda.synchronize()
    assert dtattn.device_status() == 0


def test_wan_one_rank_slice_full_length(dtattn):
    """configs[3] at its full 75,600-token length for the 5 heads one of 8 ranks owns; the C oracle checks a
    sample of query rows of each head against all 75,600 keys (75,600 = 590*128 + 80: ragged last tile)."""
    cfg = so.CONFIGS["wan_self"]
    q, k, v = so.make_inputs(cfg, heads=(0, 5))
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    out = dtattn.sdpa_forward(qd, kd, vd, cfg.scale)
    torch.cuda.synchronize()
    assert dtattn.device_status() == 0
    rows = torch.cat([torch.arange(0, cfg.Sq, 2500), torch.arange(cfg.Sq - 90, cfg.Sq, 7)])
    ref = c_oracle.sdpa_c(q[:, rows].contiguous(), k, v, cfg.scale)
    check(out[:, rows.to(DEV)], ref, torch.bfloat16, "wan", strict=True)
    assert torch.isfinite(out.float()).all()


# --------------------------------------------------------------------------------------------------
# operator surface and host path
# --------------------------------------------------------------------------------------------------

def test_operator_mirror_on_device(dtattn):
    """The Python mirror of ScaledDotProductAttention(scale:isCausal:flags:) (Qwen3_5.swift:193-196)."""
    q, k, v = inputs(1, 1, 640, 16, 4, 128, torch.float16, 91)
    op = dtattn.ScaledDotProductAttention(scale=128 ** -0.5, is_causal=True, flags=[dtattn.GEMMFlag.Float16])
    out = op(q.to(DEV), k.to(DEV), v.to(DEV))
    torch.cuda.synchronize()
    check(out, oracle(q, k, v, 128 ** -0.5, True), torch.float16, "operator")


def test_host_entry_point(dtattn):
    """dt_sdpa_forward_host: host tensors in, host tensor out (the end-to-end path the benchmark times)."""
    for (B, Sq, Sk, Hq, Hkv, D, dtype, causal) in [(1, 300, 300, 2, 2, 128, torch.bfloat16, False),
                                                    (2, 1, 2000, 8, 2, 128, torch.float16, True),
                                                    (1, 40, 40, 2, 2, 40, torch.float32, False)]:
        q, k, v = inputs(B, Sq, Sk, Hq, Hkv, D, dtype, 95)
        out = dtattn.sdpa_forward(q, k, v, D ** -0.5, causal)
        assert not out.is_cuda
        check(out, oracle(q, k, v, D ** -0.5, causal), dtype, "host path")
    # a large tensor-core shape takes a pipelined path: one image without a causal rule sends K and V whole and the
    # queries in runs of rows (2300 rows: the last run is ragged); a batch of two goes by head groups (copies of one
    # group overlap the attention of another); sinks travel with both
    for (B, S, causal, with_sinks) in [(1, 2300, False, False), (1, 2304, False, True), (2, 1152, False, True),
                                       (1, 2304, True, False)]:
        q, k, v = inputs(B, S, S, 16, 8, 128, torch.bfloat16, 97 + S + B)
        sinks = (so.seeded_normal((16,), 99) * 2.0).to(torch.bfloat16) if with_sinks else None
        out = dtattn.sdpa_forward(q, k, v, 128 ** -0.5, causal, sinks=sinks)
        if not with_sinks:
            rows = torch.arange(0, S, 11)
            want = oracle(q, k, v, 128 ** -0.5, causal)[:, rows] if causal else \
                oracle(q[:, rows].contiguous(), k, v, 128 ** -0.5)
            check(out[:, rows], want, torch.bfloat16, "host path, pipelined")
        out2 = dtattn.sdpa_forward(q.cuda(), k.cuda(), v.cuda(), 128 ** -0.5, causal,
                                   sinks=None if sinks is None else sinks.cuda()).cpu()
        assert torch.equal(out, out2), "host path and device path must agree bitwise"
    # the UNet cross-attention shape from host tensors: the short key/value kernel behind the host entry point
    q, k, v = inputs(2, 4096, 77, 20, 20, 64, torch.float16, 96, 0.5)
    out = dtattn.sdpa_forward(q, k, v, 0.125)
    check(out, c_oracle.sdpa_c(q, k, v, 0.125), torch.float16, "host path, cross-attention", strict=True)
    # sinks on the plain (single-stream) host path
    q, k, v = inputs(1, 300, 300, 4, 2, 64, torch.float16, 93)
    sinks = (so.seeded_normal((4,), 94) * 2.0).to(torch.float16)
    out = dtattn.sdpa_forward(q, k, v, 0.125, True, sinks=sinks)
    ref = so.sdpa_explicit(q, k, v, 0.125, True, compute_dtype=torch.float64, sinks=sinks).float()
    check(out, ref, torch.float16, "host path, sinks")
    assert dtattn.lib().dt_host_release() == 0


def test_permute_gathered(dtattn):
    world, B, S, Hl, D = 4, 2, 37, 3, 128
    src = torch.randn(world, B, S, Hl, D, device=DEV).to(torch.bfloat16)
    dst = torch.zeros(B, S, world * Hl, D, dtype=torch.bfloat16, device=DEV)
    st = dtattn.lib().dt_permute_gathered(ctypes.c_void_p(src.data_ptr()), dtattn._view4(dst), world, B, S, Hl, D,
                                          dtattn.DT_BF16, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert st == 0
    torch.cuda.synchronize()
    want = src.permute(1, 2, 0, 3, 4).reshape(B, S, world * Hl, D)
    assert torch.equal(dst, want)


def test_decode_with_programmatic_dependent_launch(dtattn):
    """DT_FLAG_KV_PREFIX_STABLE: back-to-back decode calls that share one workspace and one stream may overlap (the
    next call streams its cache while the previous one combines); every call must still be right.  The caches are
    not written by anything in the stream, which is what the flag promises."""
    dtype = torch.float16
    sets = []
    for i, (B, Sk, Hq, Hkv, D) in enumerate([(1, 8192, 32, 8, 128), (2, 3000, 16, 4, 256), (1, 5000, 8, 8, 64)]):
        q, k, v = inputs(B, 1, Sk, Hq, Hkv, D, dtype, 1001 + 10 * i)
        ref = oracle(q, k, v, D ** -0.5, True)
        sets.append((q.to(DEV), k.to(DEV), v.to(DEV), ref, D))
    outs = []
    for rep in range(20):
        for q, k, v, ref, D in sets:
            outs.append((dtattn.sdpa_forward(q, k, v, D ** -0.5, True, flags=dtattn.DT_FLAG_KV_PREFIX_STABLE), ref))
    torch.cuda.synchronize()
    assert dtattn.device_status() == 0
    for out, ref in outs:
        check(out, ref, dtype, "decode, dependent launch")
    # the fused step with the flag: other kernels (here: plain decode calls on another cache) sit between two steps
    # of one cache, as a model's other layers do
    B, Hq, Hkv, D, start = 1, 16, 4, 128, 700
    k_cache = so.seeded_normal((B, start + 6, Hkv, D), 1051).to(dtype)
    v_cache = so.seeded_normal((B, start + 6, Hkv, D), 1052).to(dtype)
    kc_ref, vc_ref = k_cache.clone(), v_cache.clone()
    kc, vc = k_cache.to(DEV), v_cache.to(DEV)
    pend = []
    for t in range(6):
        qn = so.seeded_normal((B, 1, Hq, D), 1060 + 3 * t).to(dtype)
        kn = so.seeded_normal((B, 1, Hkv, D), 1061 + 3 * t).to(dtype)
        vn = so.seeded_normal((B, 1, Hkv, D), 1062 + 3 * t).to(dtype)
        ref = so.decode_step_explicit(qn, kc_ref, vc_ref, kn, vn, None, D ** -0.5, start + t, dtype)
        pend.append((dtattn.decode_step(qn.to(DEV), kc, vc, kn.to(DEV), vn.to(DEV), None, D ** -0.5, start + t,
                                        flags=dtattn.DT_FLAG_KV_PREFIX_STABLE), ref))
        q0, k0, v0, _, D0 = sets[0]
        dtattn.sdpa_forward(q0, k0, v0, D0 ** -0.5, True, flags=dtattn.DT_FLAG_KV_PREFIX_STABLE)
    torch.cuda.synchronize()
    for out, ref in pend:
        check(out, ref, dtype, "decode step, dependent launch")
    assert torch.equal(kc.cpu().view(torch.int16), kc_ref.view(torch.int16))
