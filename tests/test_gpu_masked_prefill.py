"""Additive-mask attention on the tensor-core kernel, through the C ABI, against the CPU oracle.

The reference passes a mask as the operator's 4th input: alone for the 77-token CLIP encoder
(CLIPTextModel.swift:46-51) and together with ``isCausal: true`` for its LLM text encoders (Llama.swift:70-73,
Qwen3.swift:57-59, Gemma3.swift:51).  Masks are [B or 1, H or 1, Sq, Sk] in the tensors' type, filled with
-greatestFiniteMagnitude where a key is hidden (TextEncoder.swift:147-158).
"""
import pytest
import torch

from oracle import c_oracle
from oracle import sdpa_oracle as so

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ROUND = {torch.float16: 2.0 ** -11, torch.bfloat16: 2.0 ** -9}


def make_mask(bm, hm, Sq, Sk, dtype, seed, hidden=0.3, causal_fill=False, row_stride=None):
    """Random additive biases with a share of hidden entries; every row keeps key 0 visible.  row_stride > Sk gives
    a row-padded view (what a 16-byte aligned mask of an odd length looks like)."""
    g = torch.Generator().manual_seed(seed)
    stride = row_stride or Sk
    store = torch.zeros(bm, hm, Sq, stride, dtype=torch.float32)
    m = store[..., :Sk]
    m.copy_(0.5 * torch.randn(bm, hm, Sq, Sk, generator=g))
    m.masked_fill_(torch.rand(bm, hm, Sq, Sk, generator=g) < hidden, -torch.finfo(dtype).max)
    if causal_fill:
        i, j = torch.arange(Sq).view(Sq, 1), torch.arange(Sk).view(1, Sk)
        m.masked_fill_(j > i + (Sk - Sq), -torch.finfo(dtype).max)
    m[..., 0] = 0.0
    return store.to(dtype)[..., :Sk]


def run_and_check(dtattn, q, k, v, mask, scale, causal, what, want_lse=True, strict=False):
    B, Sq, Hq, D = q.shape
    qd, kd, vd, md = q.to(DEV), k.to(DEV), v.to(DEV), mask.to(DEV)
    if mask.stride(2) != mask.shape[3]:  # keep the padded row stride on the device
        store = torch.full((mask.shape[0], mask.shape[1], mask.shape[2], mask.stride(2)), float("nan"), dtype=mask.dtype,
                           device=DEV)  # the padding holds NaN: it must never be used as a mask value
        store[..., :mask.shape[3]] = md
        md = store[..., :mask.shape[3]]
    out = torch.empty_like(qd)
    lse = torch.empty(B, Hq, Sq, dtype=torch.float32, device=DEV) if want_lse else None
    p = dtattn.make_params(qd, kd, vd, out, scale, causal, md, lse)
    assert dtattn.kernel_name(p) == "prefill_tcgen05", what
    dtattn.sdpa_forward(qd, kd, vd, scale, causal, md, out=out, lse=lse)
    torch.cuda.synchronize()
    assert dtattn.device_status() == 0, "a device-side wait ran out"
    small = B * Hq * Sq * k.shape[1] * D <= 1 << 24
    if small:
        ref, ref_lse = so.sdpa_explicit(q, k, v, scale, causal, mask, compute_dtype=torch.float64, return_lse=True)
        ref = ref.float()
    else:
        ref, ref_lse = c_oracle.sdpa_c(q, k, v, scale, causal, mask, return_lse=True)
    got = out.float().cpu()
    assert torch.isfinite(got).all(), what
    mx, mean = so.error_stats(got, ref)
    rnd = ROUND[q.dtype]
    bound_max = so.TOL_MAX_ABS + (0.0 if strict else 2 * rnd * float(ref.abs().max()))
    bound_mean = so.TOL_MEAN_ABS + (0.0 if strict else rnd * float(ref.abs().mean()))
    assert mx <= bound_max and mean <= bound_mean, f"{what}: max-abs {mx:.3e} ({bound_max:.3e}) mean-abs {mean:.3e} ({bound_mean:.3e})"
    if want_lse:
        assert (lse.cpu().double() - ref_lse.double()).abs().max() < 3e-3, what
    return mx, mean


CASES = [
    # B, Sq, Sk, Hq, Hkv, D, dtype, causal, mask batch, mask heads
    (2, 200, 200, 4, 4, 64, torch.float16, False, 1, 1),     # one mask for everything
    (2, 300, 520, 8, 2, 128, torch.bfloat16, False, 2, 1),   # per-batch padding mask, grouped heads, ragged tiles
    (1, 256, 256, 4, 4, 128, torch.bfloat16, True, 1, 4),    # per-head bias on top of the causal rule
    (2, 130, 384, 6, 3, 64, torch.bfloat16, True, 2, 6),     # Sq < Sk causal (bottom-right) + full mask
    (1, 77, 80, 2, 2, 64, torch.float16, False, 1, 1),       # one key block
    (1, 512, 1032, 2, 1, 128, torch.float16, True, 1, 1),    # nine key blocks, the last one of 8 keys
    (1, 40, 200, 2, 2, 40, torch.float16, False, 1, 2),      # SD1.5 head dim (zero-padded to 64)
    (2, 300, 520, 8, 4, 256, torch.bfloat16, True, 2, 1),    # Gemma3 text encoder (Gemma3.swift:51,148): D = 256, causal + padding mask
    (1, 200, 200, 2, 2, 256, torch.float16, False, 1, 2),    # D = 256, per-head bias
]


@pytest.mark.parametrize("case", CASES)
def test_masked_attention_on_the_tensor_core_kernel(dtattn, case):
    B, Sq, Sk, Hq, Hkv, D, dtype, causal, bm, hm = case
    q = so.seeded_normal((B, Sq, Hq, D), 501).to(dtype)
    k = so.seeded_normal((B, Sk, Hkv, D), 502).to(dtype)
    v = so.seeded_normal((B, Sk, Hkv, D), 503).to(dtype)
    mask = make_mask(bm, hm, Sq, Sk, dtype, 504)
    run_and_check(dtattn, q, k, v, mask, D ** -0.5, causal, str(case))


def test_clip_length_mask_with_padded_rows(dtattn):
    """77 keys (CLIPTextModel.swift:46-51): a [1,1,77,77] mask whose rows are padded to 80 entries is 16-byte
    aligned and runs on the tensor-core kernel; the three entries past each row's end are never read as mask values
    (they hold NaN here).  The unpadded mask (row stride 77) goes to the CUDA-core kernel."""
    B, S, H, D, dtype = 2, 77, 4, 64, torch.float16
    q, k, v = (so.seeded_normal((B, S, H, D), s).to(dtype) for s in (511, 512, 513))
    mask = make_mask(1, 1, S, S, dtype, 514, hidden=0.0, causal_fill=True, row_stride=80)
    run_and_check(dtattn, q, k, v, mask, D ** -0.5, False, "clip padded")
    dense = mask.contiguous()
    p = dtattn.make_params(q.to(DEV), k.to(DEV), v.to(DEV), q.to(DEV), D ** -0.5, False, dense.to(DEV))
    assert dtattn.kernel_name(p) == "generic"


def test_mask_storage_that_ends_with_the_last_row(dtattn):
    """Sk = 100 with rows 104 entries apart, in a buffer that ends right after the last row's 100th entry: the
    vector that straddles Sk is fetched element by element, so nothing past the buffer is touched."""
    B, Sq, Sk, H, D, dtype = 1, 150, 100, 2, 64, torch.bfloat16
    q = so.seeded_normal((B, Sq, H, D), 521).to(dtype)
    k = so.seeded_normal((B, Sk, H, D), 522).to(dtype)
    v = so.seeded_normal((B, Sk, H, D), 523).to(dtype)
    full = make_mask(1, 1, Sq, Sk, dtype, 524, row_stride=104)
    flat = torch.zeros((Sq - 1) * 104 + Sk, dtype=dtype)
    mask = flat.as_strided((1, 1, Sq, Sk), (0, 0, 104, 1))
    mask.copy_(full)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    md = flat.to(DEV).as_strided((1, 1, Sq, Sk), (0, 0, 104, 1))
    p = dtattn.make_params(qd, kd, vd, qd, D ** -0.5, False, md)
    assert dtattn.kernel_name(p) == "prefill_tcgen05"
    out = dtattn.sdpa_forward(qd, kd, vd, D ** -0.5, False, md)
    torch.cuda.synchronize()
    ref = so.sdpa_explicit(q, k, v, D ** -0.5, False, mask, compute_dtype=torch.float64).float()
    mx, mean = so.error_stats(out.float().cpu(), ref)
    assert mx <= so.TOL_MAX_ABS + 2 * ROUND[dtype] * float(ref.abs().max()) and mean <= 2 * so.TOL_MEAN_ABS, (mx, mean)


def test_llm_text_encoder_shape(dtattn):
    """Llama-style text encoder (Llama.swift:57-96): 32 query heads over 8 KV heads, d128, isCausal plus a padding
    mask shared by the heads, at a prompt length where the mask tile traffic matters."""
    B, S, Hq, Hkv, D, dtype = 2, 1024, 32, 8, 128, torch.bfloat16
    q = so.seeded_normal((B, S, Hq, D), 531).to(dtype)
    k = so.seeded_normal((B, S, Hkv, D), 532).to(dtype)
    v = so.seeded_normal((B, S, Hkv, D), 533).to(dtype)
    mask = torch.zeros(B, 1, S, S, dtype=dtype)
    mask[0, :, :, 700:] = -torch.finfo(dtype).max  # prompt 0 has 700 real tokens, the rest is padding
    mask[1, :, :, 1000:] = -torch.finfo(dtype).max
    run_and_check(dtattn, q, k, v, mask, D ** -0.5, True, "llama text encoder", want_lse=False)


def test_masked_and_causal_flag_agree(dtattn):
    """The additive form of the causal rule (TextEncoder.swift:151-158) and isCausal give the same result."""
    B, S, H, D, dtype = 1, 384, 4, 128, torch.bfloat16
    q, k, v = (so.seeded_normal((B, S, H, D), s).to(dtype).to(DEV) for s in (541, 542, 543))
    mask = make_mask(1, 1, S, S, dtype, 544, hidden=0.0, causal_fill=True)
    mask[mask > -1e30] = 0.0
    a = dtattn.sdpa_forward(q, k, v, D ** -0.5, False, mask.to(DEV))
    b = dtattn.sdpa_forward(q, k, v, D ** -0.5, True)
    torch.cuda.synchronize()
    assert (a.float() - b.float()).abs().max() <= 2 ** -8 * float(b.float().abs().max())
