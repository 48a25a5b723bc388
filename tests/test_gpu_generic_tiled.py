"""The register-tiled CUDA-core kernel (64 query rows x 64 keys per step), through the C ABI, against the oracle.

It serves what the tensor-core kernels do not take: fp32 tensors (the reference's upcastAttention,
UNet.swift:217-265) of any head dim, and masks whose rows are not 16-byte aligned.  fp32 results must agree with the
float64 oracle to fp32 rounding of a few hundred accumulated terms; the 16-bit cases carry the tolerance of the other
parity tests.
"""
import pytest
import torch

from oracle import sdpa_oracle as so
from test_gpu_parity import DEV, check, inputs

pytestmark = pytest.mark.gpu

FP32_MAX_ABS = 2e-5  # |O| <= max|V| ~ 4.5 with unit-normal inputs; a few hundred fp32 terms per output
FP32_MEAN_ABS = 2e-6


def run(dtattn, q, k, v, scale, causal, expect="generic", **kw):
    dev = {key: (val.to(DEV) if torch.is_tensor(val) else val) for key, val in kw.items()}
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    lse = torch.full((q.shape[0], q.shape[2], q.shape[1]), float("nan"), dtype=torch.float32, device=DEV)
    out = torch.full(q.shape, float("nan"), dtype=q.dtype, device=DEV)
    p = dtattn.make_params(qd, kd, vd, out, scale, causal, dev.get("mask"), lse,
                           **{k_: v_ for k_, v_ in dev.items() if k_ != "mask"})
    assert dtattn.kernel_name(p) == expect
    dtattn.sdpa_forward(qd, kd, vd, scale, causal, dev.get("mask"), out=out, lse=lse,
                        **{k_: v_ for k_, v_ in dev.items() if k_ != "mask"})
    torch.cuda.synchronize()
    assert dtattn.device_status() == 0
    return out, lse


def check_fp32(out, ref, what):
    got = out.float().cpu()
    assert torch.isfinite(got).all(), what
    mx, mean = so.error_stats(got, ref.float())
    assert mx <= FP32_MAX_ABS and mean <= FP32_MEAN_ABS, f"{what}: max-abs {mx:.3e} mean-abs {mean:.3e}"


SHAPES = [
    # B, Sq, Sk, Hq, Hkv, D, causal
    (2, 256, 256, 8, 8, 40, False),    # SD1.5 upcast attention, 16x16 latent
    (1, 100, 130, 4, 2, 36, False),    # D = 4 (mod 8): the padded pitch; ragged rows and keys; grouped heads
    (1, 65, 64, 2, 2, 44, True),       # Sq > Sk causal: row 0 sees no key
    (2, 64, 300, 4, 1, 64, True),      # Sq < Sk causal (bottom-right aligned)
    (1, 200, 200, 3, 3, 80, True),
    (1, 130, 77, 2, 2, 160, False),    # SD1.5 deepest blocks' head dim: three column groups per thread, the last partial
    (1, 96, 200, 2, 2, 256, False),    # largest head dim: 216 KB of shared memory
    (1, 33, 5, 1, 1, 4, False),        # smallest D the tiled kernel takes
]


@pytest.mark.parametrize("case", SHAPES)
def test_fp32_against_the_oracle(dtattn, case):
    B, Sq, Sk, Hq, Hkv, D, causal = case
    q, k, v = inputs(B, Sq, Sk, Hq, Hkv, D, torch.float32, 1201)
    ref, lse_ref = so.sdpa_explicit(q, k, v, D ** -0.5, causal, compute_dtype=torch.float64, return_lse=True)
    out, lse = run(dtattn, q, k, v, D ** -0.5, causal)
    check_fp32(out, ref, str(case))
    finite = torch.isfinite(lse_ref)
    assert torch.allclose(lse.cpu()[finite], lse_ref.float()[finite], atol=1e-4, rtol=1e-5)
    assert bool((lse.cpu()[~finite] == float("-inf")).all())


def test_fp32_mask_sinks_and_window(dtattn):
    B, Sq, Sk, Hq, Hkv, D = 2, 150, 190, 4, 2, 40
    q, k, v = inputs(B, Sq, Sk, Hq, Hkv, D, torch.float32, 1211)
    g = torch.Generator().manual_seed(1212)
    mask = 0.5 * torch.randn(B, 1, Sq, Sk, generator=g)
    mask.masked_fill_(torch.rand(B, 1, Sq, Sk, generator=g) < 0.3, -torch.finfo(torch.float32).max)
    mask[..., 0] = 0.0
    sinks = so.seeded_normal((Hq,), 1213) * 2.0
    for causal, window, with_mask, with_sinks in ((False, 0, True, False), (True, 0, True, True), (True, 37, False, True),
                                                  (False, 64, False, False)):
        ref, lse_ref = so.sdpa_explicit(q, k, v, D ** -0.5, causal, mask if with_mask else None, compute_dtype=torch.float64,
                                        return_lse=True, sinks=sinks if with_sinks else None, sliding_window=window)
        kw = {}
        if with_mask:
            kw["mask"] = mask
        if with_sinks:
            kw["sinks"] = sinks
        if window:
            kw["sliding_window"] = window
        out, lse = run(dtattn, q, k, v, D ** -0.5, causal, **kw)
        what = f"causal={causal} window={window} mask={with_mask} sinks={with_sinks}"
        check_fp32(out, ref, what)
        assert torch.allclose(lse.cpu(), lse_ref.float(), atol=1e-4, rtol=1e-5), what


def test_fp32_variable_length_batch(dtattn):
    Hq, Hkv, D = 4, 2, 40
    len_q = [5, 0, 130, 64, 1, 70]
    len_k = [7, 3, 130, 100, 300, 0]
    off_q, off_k = [0], [0]
    for a, b in zip(len_q, len_k):
        off_q.append(off_q[-1] + a)
        off_k.append(off_k[-1] + b)
    q = so.seeded_normal((1, off_q[-1], Hq, D), 1221)
    k = so.seeded_normal((1, off_k[-1], Hkv, D), 1222)
    v = so.seeded_normal((1, off_k[-1], Hkv, D), 1223)
    for causal in (False, True):
        ref = so.sdpa_varlen_explicit(q, k, v, D ** -0.5, off_q, off_k, causal, compute_dtype=torch.float64).float()
        out = torch.zeros(q.shape, dtype=torch.float32, device=DEV)
        oq = torch.tensor(off_q, dtype=torch.int32, device=DEV)
        ok = torch.tensor(off_k, dtype=torch.int32, device=DEV)
        dtattn.sdpa_forward(q.to(DEV), k.to(DEV), v.to(DEV), D ** -0.5, causal, out=out, seq_offsets_q=oq, seq_offsets_k=ok,
                            max_seq_q=max(len_q), max_seq_k=max(len_k))
        torch.cuda.synchronize()
        assert dtattn.device_status() == 0
        check_fp32(out, ref, f"varlen causal={causal}")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_half_precision_head_dim_160_and_strided_views(dtattn, dtype):
    """D = 160 in half precision (SD1.5's deepest blocks), read through the reference's fused-projection layout (q, k,
    v are slices of one [B, S, 3, H, D] tensor: token stride 3 H D), on the CUDA-core kernel and on the kernel the
    library picks by itself (the tensor-core one, zero-padded to 256)."""
    B, S, H, D = 2, 256, 8, 160
    qkv = so.seeded_normal((B, S, 3, H, D), 1231).to(dtype)
    q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
    ref = so.sdpa_explicit(q, k, v, D ** -0.5, False, compute_dtype=torch.float64).float()
    dev = qkv.to(DEV)
    for flags in (dtattn.DT_FLAG_FORCE_GENERIC, 0):
        out = dtattn.sdpa_forward(dev[:, :, 0], dev[:, :, 1], dev[:, :, 2], D ** -0.5, False, flags=flags)
        torch.cuda.synchronize()
        assert dtattn.device_status() == 0
        check(out, ref, dtype, f"d160 {dtype} flags={flags}")


def test_unaligned_mask_rows_in_half_precision(dtattn):
    """A dense [1,1,77,77] fp16 mask (row stride 77 elements: not 16-byte aligned) keeps the call off the tensor-core
    kernel; 77 query rows are enough for the tiled kernel."""
    B, S, H, D, dtype = 2, 77, 4, 64, torch.float16
    q, k, v = inputs(B, S, S, H, H, D, dtype, 1241)
    i, j = torch.arange(S).view(S, 1), torch.arange(S).view(1, S)
    mask = torch.zeros(1, 1, S, S, dtype=dtype).masked_fill_(j > i, -torch.finfo(dtype).max)
    ref = so.sdpa_explicit(q, k, v, D ** -0.5, False, mask, compute_dtype=torch.float64).float()
    out, _ = run(dtattn, q, k, v, D ** -0.5, False, mask=mask)
    check(out, ref, dtype, "clip mask, dense rows")
