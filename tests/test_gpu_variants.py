"""Operator variants used elsewhere in the reference tree: attention sinks and sliding window
(DeepSeek4.swift:482-493), variable-length batches (Qwen3_5VL.swift:428-437) and Wan's causal chunking, which the
reference builds from plain calls on row-offset views (Wan.swift:104-127).  Each case goes through the C ABI and is
compared with the oracle's explicit form."""
import pytest
import torch

from oracle import sdpa_oracle as so
from test_gpu_parity import DEV, check, inputs

pytestmark = pytest.mark.gpu


def run(dtattn, q, k, v, scale, causal, **kw):
    dev = {key: (val.to(DEV) if torch.is_tensor(val) else val) for key, val in kw.items()}
    out = dtattn.sdpa_forward(q.to(DEV), k.to(DEV), v.to(DEV), scale, causal, **dev)
    torch.cuda.synchronize()
    assert dtattn.device_status() == 0
    return out


SINK_WINDOW = [
    # B, Sq, Sk, Hq, Hkv, D, dtype, causal, window, sinks, forced generic
    (2, 33, 70, 4, 2, 64, torch.float16, True, 0, True, False),
    (1, 40, 40, 8, 1, 128, torch.bfloat16, True, 16, True, False),     # DeepSeek raw attention: one shared KV head
    (1, 300, 300, 4, 4, 128, torch.bfloat16, True, 128, False, False),  # window across 128-key blocks
    (1, 300, 300, 4, 4, 64, torch.float16, True, 1, False, False),      # every query sees only itself
    (2, 257, 300, 2, 2, 128, torch.float16, True, 1000, True, False),   # window wider than the sequence
    (1, 64, 200, 2, 1, 80, torch.float16, False, 50, True, False),      # window without the causal rule
    (1, 1, 4096, 32, 8, 128, torch.float16, True, 128, True, False),    # decode over a cache, last 128 rows
    (2, 1, 1000, 16, 4, 256, torch.bfloat16, True, 77, True, False),
    (1, 4, 777, 8, 2, 64, torch.bfloat16, True, 300, True, False),      # 4 new tokens x group of 4
    (1, 300, 300, 4, 4, 128, torch.bfloat16, True, 128, True, True),    # same through the CUDA-core kernel
    (1, 20, 20, 2, 2, 40, torch.float32, True, 7, True, False),
    (1, 1500, 1500, 4, 2, 128, torch.bfloat16, True, 512, True, False),  # leading K/V blocks skipped per query tile
    (2, 700, 900, 4, 4, 64, torch.float16, True, 200, True, False),
    (1, 700, 900, 4, 2, 256, torch.bfloat16, True, 200, True, False),   # D = 256 on the tensor-core kernel
]


@pytest.mark.parametrize("case", SINK_WINDOW)
def test_sinks_and_sliding_window(dtattn, case):
    B, Sq, Sk, Hq, Hkv, D, dtype, causal, window, with_sinks, generic = case
    q, k, v = inputs(B, Sq, Sk, Hq, Hkv, D, dtype, 901)
    sinks = (so.seeded_normal((Hq,), 904) * 2.0).to(dtype) if with_sinks else None
    ref, lse_ref = so.sdpa_explicit(q, k, v, D ** -0.5, causal, compute_dtype=torch.float64, return_lse=True,
                                    sinks=sinks, sliding_window=window)
    lse = torch.zeros(B, Hq, Sq, dtype=torch.float32, device=DEV)
    out = run(dtattn, q, k, v, D ** -0.5, causal, sinks=sinks, sliding_window=window, lse=lse,
              flags=dtattn.DT_FLAG_FORCE_GENERIC if generic else 0)
    check(out, ref.float(), dtype, str(case))
    assert torch.allclose(lse.cpu(), lse_ref.float(), atol=2e-3, rtol=1e-3), "log-sum-exp"


def test_variants_stay_on_the_fast_kernels(dtattn):
    """Sinks and sliding window are handled inside the tensor-core and split-KV kernels, not by falling back."""
    for shape, want in (((1, 1500, 1500, 4, 2, 128), "prefill_tcgen05"), ((1, 1, 4096, 32, 8, 128), "decode_splitkv")):
        B, Sq, Sk, Hq, Hkv, D = shape
        q, k, v = [t.to(DEV) for t in inputs(B, Sq, Sk, Hq, Hkv, D, torch.float16, 951)]
        sinks = torch.zeros(Hq, dtype=torch.float16, device=DEV)
        p = dtattn.make_params(q, k, v, torch.empty_like(q), D ** -0.5, True, sinks=sinks, sliding_window=100)
        assert dtattn.kernel_name(p) == want


def test_sink_dominates_row(dtattn):
    """A sink far above every score takes nearly all the weight: the output goes to zero, not to NaN."""
    q, k, v = inputs(1, 5, 9, 2, 2, 64, torch.float16, 911)
    sinks = torch.tensor([60.0, -60.0], dtype=torch.float16)
    out = run(dtattn, q, k, v, 0.125, True, sinks=sinks)
    ref = so.sdpa_explicit(q, k, v, 0.125, True, compute_dtype=torch.float64, sinks=sinks).float()
    check(out, ref, torch.float16, "dominant sink")
    assert float(out[:, :, 0].abs().max()) < 1e-6


@pytest.mark.parametrize("causal", [False, True])
def test_variable_length_batch(dtattn, causal):
    dtype, Hq, Hkv, D = torch.bfloat16, 8, 4, 128
    len_q = [5, 0, 130, 64, 1]
    len_k = [7, 3, 130, 100, 300]
    off_q = [0]
    off_k = [0]
    for a, b in zip(len_q, len_k):
        off_q.append(off_q[-1] + a)
        off_k.append(off_k[-1] + b)
    q = so.seeded_normal((1, off_q[-1], Hq, D), 921).to(dtype)
    k = so.seeded_normal((1, off_k[-1], Hkv, D), 922).to(dtype)
    v = so.seeded_normal((1, off_k[-1], Hkv, D), 923).to(dtype)
    ref = so.sdpa_varlen_explicit(q, k, v, D ** -0.5, off_q, off_k, causal, compute_dtype=torch.float64).float()
    op = dtattn.ScaledDotProductAttention(scale=D ** -0.5, is_causal=causal, is_variable_length=True,
                                          max_sequence_length=(max(len_q), max(len_k)))
    oq = torch.tensor(off_q, dtype=torch.int32, device=DEV)
    ok = torch.tensor(off_k, dtype=torch.int32, device=DEV)
    out = torch.zeros(q.shape, dtype=dtype, device=DEV)
    op(q.to(DEV), k.to(DEV), v.to(DEV), oq, ok, out=out)
    torch.cuda.synchronize()
    check(out, ref, dtype, f"varlen causal={causal}")


@pytest.mark.parametrize("D,dtype", [(128, torch.bfloat16), (64, torch.float16), (80, torch.float16), (256, torch.bfloat16)])
def test_variable_length_batch_on_the_tensor_core_kernel(dtattn, D, dtype):
    """Packed vision-encoder style batch (Qwen3_5VL.swift:428-437, non-causal): sequences that end inside a 32-row
    store group, exactly on a tile edge, one row past it, an empty one, and one with queries but no keys."""
    Hq, Hkv = 4, 2
    len_q = [5, 0, 130, 64, 1, 300, 256, 257, 33, 7]
    len_k = [7, 3, 130, 100, 300, 300, 256, 513, 0, 129]
    off_q, off_k = [0], [0]
    for a, b in zip(len_q, len_k):
        off_q.append(off_q[-1] + a)
        off_k.append(off_k[-1] + b)
    q = so.seeded_normal((1, off_q[-1], Hq, D), 925).to(dtype)
    k = so.seeded_normal((1, off_k[-1], Hkv, D), 926).to(dtype)
    v = so.seeded_normal((1, off_k[-1], Hkv, D), 927).to(dtype)
    ref, lse_ref = torch.zeros(q.shape), torch.full((1, Hq, off_q[-1]), float("-inf"))
    for s_ in range(len(len_q)):
        q0, q1, k0, k1 = off_q[s_], off_q[s_ + 1], off_k[s_], off_k[s_ + 1]
        if q1 > q0 and k1 > k0:
            o_, l_ = so.sdpa_explicit(q[:, q0:q1], k[:, k0:k1], v[:, k0:k1], D ** -0.5, compute_dtype=torch.float64,
                                      return_lse=True)
            ref[:, q0:q1], lse_ref[:, :, q0:q1] = o_.float(), l_.float()
    oq = torch.tensor(off_q, dtype=torch.int32, device=DEV)
    ok = torch.tensor(off_k, dtype=torch.int32, device=DEV)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    out = torch.full(q.shape, float("nan"), dtype=dtype, device=DEV)
    lse = torch.zeros(1, Hq, off_q[-1], dtype=torch.float32, device=DEV)
    p = dtattn.make_params(qd, kd, vd, out, D ** -0.5, False, seq_offsets_q=oq, seq_offsets_k=ok,
                           max_seq_q=max(len_q), max_seq_k=max(len_k))
    assert dtattn.kernel_name(p) == "prefill_tcgen05"
    dtattn.sdpa_forward(qd, kd, vd, D ** -0.5, False, out=out, lse=lse, seq_offsets_q=oq, seq_offsets_k=ok,
                        max_seq_q=max(len_q), max_seq_k=max(len_k))
    torch.cuda.synchronize()
    assert dtattn.device_status() == 0
    check(out, ref, dtype, f"varlen tensor-core D={D}")
    finite = torch.isfinite(lse_ref)
    assert torch.allclose(lse.cpu()[finite], lse_ref[finite], atol=2e-3, rtol=1e-3)
    assert bool((lse.cpu()[~finite] == float("-inf")).all())


def test_operator_mirror_takes_sinks_input(dtattn):
    q, k, v = inputs(1, 12, 12, 4, 1, 64, torch.float16, 931)
    sinks = so.seeded_normal((1, 1, 4, 1), 934).to(torch.float16)
    op = dtattn.ScaledDotProductAttention(scale=0.125, is_causal=True, has_attention_sinks=True, sliding_window=5)
    out = op(q.to(DEV), k.to(DEV), v.to(DEV), sinks.to(DEV))
    torch.cuda.synchronize()
    ref = so.sdpa_explicit(q, k, v, 0.125, True, compute_dtype=torch.float64, sinks=sinks.reshape(-1),
                           sliding_window=5).float()
    check(out, ref, torch.float16, "operator mirror")
    with pytest.raises(ValueError):
        op(q.to(DEV), k.to(DEV), v.to(DEV))


def test_wan_causal_chunking_from_plain_calls_on_views(dtattn):
    """Wan.swift:104-127: queries of frame group i attend keys of groups 0..i (+ pad frames), each group one plain
    call on row-offset views of the same tensors."""
    dtype, H, D = torch.bfloat16, 4, 128
    time, per_frame, group, pad = 6, 50, 2, 1
    hw = time * per_frame
    frames, pad_frames = per_frame * group, per_frame * pad
    q, k, v = inputs(1, hw, hw, H, H, D, dtype, 941)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    out = torch.empty_like(qd)
    ref = torch.empty(q.shape, dtype=torch.float32)
    for i in range((time + group - 1) // group):
        r0, r1 = i * frames, min(hw, (i + 1) * frames)
        kk = min(hw, (i + 1) * frames + pad_frames)
        dtattn.sdpa_forward(qd[:, r0:r1], kd[:, :kk], vd[:, :kk], D ** -0.5, out=out[:, r0:r1])
        ref[:, r0:r1] = so.sdpa_explicit(q[:, r0:r1], k[:, :kk], v[:, :kk], D ** -0.5, compute_dtype=torch.float64).float()
    torch.cuda.synchronize()
    check(out, ref, dtype, "causal chunking")
