"""The short key/value cross-attention kernel (text conditioning of the UNet models, UNetXL.swift:57-185,
UNet.swift:269-504: image queries against the 77 tokens of a prompt), through the C ABI, against the CPU oracle
and against the general tensor-core kernel on the same inputs."""
import pytest
import torch

from oracle import c_oracle
from oracle import sdpa_oracle as so

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ROUND = {torch.float16: 2.0 ** -11, torch.bfloat16: 2.0 ** -9}

CASES = [
    # B, Sq, Sk, Hq, Hkv, D, dtype
    (2, 4096, 77, 20, 20, 64, torch.float16),     # the SDXL shape: 1280 tiles over 444 warpgroup runs
    (2, 1024, 77, 8, 8, 40, torch.float16),       # SD1.5 cross-attention: head dim 40, zero-padded by TMA
    (1, 1000, 77, 5, 5, 64, torch.bfloat16),      # ragged last tile (1000 = 7 * 128 + 104)
    (3, 130, 80, 12, 4, 64, torch.bfloat16),      # grouped KV heads, two tiles per head: runs cross heads and batches
    (1, 4100, 81, 2, 2, 64, torch.float16),       # 81 keys: the 96-key variant, 15 padded keys hidden
    (1, 4096, 96, 2, 1, 64, torch.bfloat16),      # exactly 96 keys
    (1, 4096, 1, 2, 2, 64, torch.float16),        # one key: every row's output is that key's value
    (2, 2048, 16, 3, 3, 32, torch.bfloat16),      # one 16-key unit, head dim 32
    (1, 33000, 77, 1, 1, 64, torch.float16),      # 258 tiles of one head: every run longer than the Q double buffer
]


def oracle(q, k, v, scale):
    B, Sq, Hq, D = q.shape
    if B * Hq * Sq * k.shape[1] * D <= 1 << 24:
        return so.sdpa_explicit(q, k, v, scale, compute_dtype=torch.float64, return_lse=True)
    return c_oracle.sdpa_c(q, k, v, scale, return_lse=True)


@pytest.mark.parametrize("case", CASES)
def test_short_kv_kernel(dtattn, case):
    B, Sq, Sk, Hq, Hkv, D, dtype = case
    q = so.seeded_normal((B, Sq, Hq, D), 601, 0.5).to(dtype)
    k = so.seeded_normal((B, Sk, Hkv, D), 602, 0.5).to(dtype)
    v = so.seeded_normal((B, Sk, Hkv, D), 603, 0.5).to(dtype)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    out = torch.full(q.shape, float("nan"), dtype=dtype, device=DEV)
    lse = torch.full((B, Hq, Sq), float("nan"), dtype=torch.float32, device=DEV)
    p = dtattn.make_params(qd, kd, vd, out, D ** -0.5, False, None, lse)
    assert dtattn.kernel_name(p) == "crossattn_short"
    dtattn.sdpa_forward(qd, kd, vd, D ** -0.5, out=out, lse=lse)
    torch.cuda.synchronize()
    assert dtattn.device_status() == 0, "a device-side wait ran out"
    ref, ref_lse = oracle(q, k, v, D ** -0.5)
    got = out.float().cpu()
    assert torch.isfinite(got).all()
    mx, mean = so.error_stats(got, ref.float())
    assert mx <= so.TOL_MAX_ABS + 2 * ROUND[dtype] * float(ref.abs().max()), (case, mx)
    assert mean <= so.TOL_MEAN_ABS + ROUND[dtype] * float(ref.abs().mean()), (case, mean)
    assert (lse.cpu().double() - ref_lse.double()).abs().max() < 3e-3
    # the general tensor-core kernel on the same inputs (a causal rule that hides nothing would change nothing, so
    # the other kernel is reached through a view with fewer rows per call)
    rows = 4096 // (B * Hq) // 8 * 8
    if 0 < rows < Sq:
        other = dtattn.sdpa_forward(qd[:, :rows].contiguous()[:, :max(1, rows // 2)], kd, vd, D ** -0.5)
        torch.cuda.synchronize()
        n = other.shape[1]
        assert (other.float() - out[:, :n].float()).abs().max() <= 4 * ROUND[dtype] * float(ref.abs().max()) + 1e-3


def test_short_kv_strided_views(dtattn):
    """Batch halves of a larger buffer and a row-offset view, as the reference passes them when the conditional and
    unconditional prompts have different lengths (UNetXL.swift:98-172): no copy is made."""
    B, Sq, Sk, H, D, dtype = 2, 2304, 77, 10, 64, torch.float16
    big_q = so.seeded_normal((B, Sq + 64, H, D), 611, 0.5).to(dtype).to(DEV)
    big_kv = so.seeded_normal((B, 128, 2 * H, D), 612, 0.5).to(dtype).to(DEV)
    q = big_q[:, 64:]                       # row-offset view: batch stride larger than Sq * H * D
    k = big_kv[:, :Sk, :H]                  # keys and values interleaved by head group in one buffer
    v = big_kv[:, :Sk, H:]
    out_store = torch.full((B, Sq, H, D + 64), float("nan"), dtype=dtype, device=DEV)
    out = out_store.as_strided((B, Sq, H, D), (Sq * H * (D + 64), H * (D + 64), D + 64, 1))
    p = dtattn.make_params(q, k, v, out, 0.125)
    assert dtattn.kernel_name(p) == "crossattn_short"
    dtattn.sdpa_forward(q, k, v, 0.125, out=out)
    torch.cuda.synchronize()
    assert dtattn.device_status() == 0
    ref = c_oracle.sdpa_c(q.cpu(), k.cpu(), v.cpu(), 0.125)
    mx, mean = so.error_stats(out.float().cpu(), ref)
    assert mx <= so.TOL_MAX_ABS and mean <= so.TOL_MEAN_ABS, (mx, mean)
    assert torch.isnan(out_store[..., D:]).all(), "bytes outside the output view were written"


def test_short_kv_is_deterministic(dtattn):
    B, Sq, Sk, H, D, dtype = 2, 4096, 77, 20, 64, torch.float16
    q = so.seeded_normal((B, Sq, H, D), 621, 0.5).to(dtype).to(DEV)
    k = so.seeded_normal((B, Sk, H, D), 622, 0.5).to(dtype).to(DEV)
    v = so.seeded_normal((B, Sk, H, D), 623, 0.5).to(dtype).to(DEV)
    a = dtattn.sdpa_forward(q, k, v, 0.125)
    b = dtattn.sdpa_forward(q, k, v, 0.125)
    c = dtattn.sdpa_forward(q, k, v, 0.125)
    torch.cuda.synchronize()
    assert torch.equal(a, b) and torch.equal(a, c)
