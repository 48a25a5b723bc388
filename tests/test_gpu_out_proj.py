"""Attention with the output projection folded in (dt_sdpa_forward_projected; the reference's
multiHeadOutputProjectionFused: true, UNet.swift:122-130): the attention kernel followed by the TMA + tcgen05 GEMM,
against the oracle's explicit attention, rounded to the 16-bit type like the unfused graph's tensor, times the Dense
weight in float64."""
import ctypes

import pytest
import torch

from oracle import sdpa_oracle as so
from test_gpu_parity import DEV, check, inputs

pytestmark = pytest.mark.gpu


def reference(q, k, v, scale, w, bias, causal, dtype):
    attn = so.sdpa_explicit(q, k, v, scale, causal, compute_dtype=torch.float64).to(dtype)  # [B,S,H,D]
    B, S, H, D = attn.shape
    out = attn.reshape(B, S, H * D).double() @ w.double().t()
    if bias is not None:
        out = out + bias.double()
    return out.float()


CASES = [
    # B, Sq, Sk, H, D, C, dtype, bias, causal
    (2, 1024, 1024, 8, 40, 320, torch.float16, True, False),    # SD1.5 self-attention at 32x32, unify heads 320 -> 320
    (2, 1024, 77, 10, 64, 640, torch.float16, True, False),     # SDXL cross-attention, 640 channels
    (1, 300, 300, 4, 64, 200, torch.bfloat16, False, False),    # ragged M and N tiles, no bias
    (1, 130, 130, 20, 64, 1280, torch.bfloat16, True, True),    # K = 1280: twenty 64-wide K steps, ring wraps 5 times
    (3, 17, 50, 2, 128, 64, torch.float16, True, False),        # less than one tile in every dimension
    (1, 1, 2000, 32, 128, 4096, torch.float16, True, True),     # decode step followed by o_proj (Qwen3_5.swift:198-202)
    (1, 2560, 77, 20, 64, 2048, torch.float16, True, False),    # 160 tiles on 148 SMs: one round + 12 tiles in quarter slices
    (1, 1408, 77, 4, 64, 4608, torch.bfloat16, True, False),    # 198 tiles: one round + 50 tiles in half slices
    (1, 1300, 77, 4, 64, 4504, torch.float16, False, False),    # the same with ragged last row and column tiles
]


@pytest.mark.parametrize("case", CASES)
def test_projected_attention(dtattn, case):
    B, Sq, Sk, H, D, C, dtype, with_bias, causal = case
    q, k, v = inputs(B, Sq, Sk, H, H, D, dtype, 961)
    K = H * D
    w = (so.seeded_normal((C, K), 964) * K ** -0.5 * 2.0).to(dtype)
    bias = so.seeded_normal((C,), 965).to(dtype) if with_bias else None
    ref = reference(q, k, v, D ** -0.5, w, bias, causal, dtype)
    out = dtattn.sdpa_forward_projected(q.to(DEV), k.to(DEV), v.to(DEV), D ** -0.5, w.to(DEV),
                                        None if bias is None else bias.to(DEV), causal)
    torch.cuda.synchronize()
    assert dtattn.device_status() == 0
    check(out, ref, dtype, str(case))


def test_operator_mirror_with_fused_projection_and_strided_output(dtattn):
    dtype, B, S, H, D, C = torch.float16, 2, 200, 8, 40, 320
    q, k, v = inputs(B, S, S, H, H, D, dtype, 971)
    w = (so.seeded_normal((C, H * D), 974) * (H * D) ** -0.5).to(dtype)
    bias = so.seeded_normal((C,), 975).to(dtype)
    op = dtattn.ScaledDotProductAttention(scale=D ** -0.5, flags=[dtattn.GEMMFlag.Float16],
                                          multi_head_output_projection_fused=True)
    op.set_output_projection(w.to(DEV), bias.to(DEV))
    big = torch.full((B, S + 8, C + 64), 7.0, dtype=dtype, device=DEV)
    view = big[:, 8:, :C]  # rows and columns around the view must stay untouched
    op(q.to(DEV), k.to(DEV), v.to(DEV), out=view)
    torch.cuda.synchronize()
    check(view, reference(q, k, v, D ** -0.5, w, bias, False, dtype), dtype, "strided out")
    assert bool((big[:, :8] == 7.0).all()) and bool((big[:, :, C:] == 7.0).all())


def test_projected_argument_checks(dtattn):
    lib = dtattn.lib()
    q, k, v = [t.to(DEV) for t in inputs(1, 16, 16, 4, 4, 64, torch.float16, 981)]
    w = torch.zeros(128, 256, dtype=torch.float16, device=DEV)
    out = torch.zeros(1, 16, 128, dtype=torch.float16, device=DEV)
    p = dtattn.make_params(q, k, v, q, 0.125)
    pr = dtattn.OutProj()
    pr.weight, pr.C = w.data_ptr(), 128
    pr.out = dtattn.Tensor4(out.data_ptr(), out.stride(0), out.stride(1), 128)
    need = ctypes.c_size_t(0)
    assert lib.dt_sdpa_projected_workspace_size(ctypes.byref(p), ctypes.byref(pr), ctypes.byref(need)) == dtattn.DT_OK
    assert need.value >= 16 * 256 * 2
    assert lib.dt_sdpa_forward_projected(ctypes.byref(p), ctypes.byref(pr), None, 0, None) == dtattn.DT_WORKSPACE
    pr.C = 100  # not a multiple of 8
    assert lib.dt_sdpa_projected_workspace_size(ctypes.byref(p), ctypes.byref(pr), ctypes.byref(need)) == dtattn.DT_UNSUPPORTED
    pr.C, pr.weight = 128, None
    assert lib.dt_sdpa_projected_workspace_size(ctypes.byref(p), ctypes.byref(pr), ctypes.byref(need)) == dtattn.DT_BAD_ARG


def test_row_parallel_form_on_one_rank(dtattn):
    """The head-sharded projected call with a world of one: the GEMM epilogue writes fp32 slabs, the reduction adds
    the bias and rounds.  (Two ranks are covered by tests/test_gpu_headsharded.py on a 2-GPU box.)"""
    dtype, B, S, H, D, C = torch.bfloat16, 2, 333, 4, 64, 200
    q, k, v = inputs(B, S, S, H, H, D, dtype, 991)
    w = (so.seeded_normal((C, H * D), 994) * (H * D) ** -0.5 * 2.0).to(dtype)
    bias = so.seeded_normal((C,), 995).to(dtype)
    comm = dtattn.HeadShardedComm(0, 1, lambda b: b)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    _, recv_bytes, rpr = comm.projected_sizes(qd, kd, vd, D ** -0.5, C)
    assert rpr % 128 == 0 and rpr >= B * S
    recv = torch.zeros(recv_bytes // 4, dtype=torch.float32, device=DEV)
    comm.register_output(recv)
    rows = torch.full((rpr, C), float("nan"), dtype=dtype, device=DEV)
    for _ in range(2):
        comm.forward_projected(qd, kd, vd, D ** -0.5, w.to(DEV), bias.to(DEV), recv, rows)
    torch.cuda.synchronize()
    assert dtattn.device_status() == 0
    ref = reference(q, k, v, D ** -0.5, w, bias, False, dtype).reshape(B * S, C)
    check(rows[:B * S], ref, dtype, "row-parallel, one rank")
    comm.close()
