"""CPU checks of the C-ABI boundary: the library loads, exports every symbol the header declares, and
rejects bad requests with the documented status codes (no kernel runs here)."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "dtattn.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dt_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(dtattn):
    names = declared_functions()
    assert len(names) >= 15
    lib = dtattn.lib()
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/dtattn.h but not exported"
    assert set(names) == {s[0] for s in dtattn.SYMBOLS}, "binding table and header disagree"


def test_struct_layout_matches_header(dtattn):
    # 10 x 4-byte scalars, 4 x (ptr + 3 int64), mask ptr + 3 int64, lse ptr, sinks ptr, 4 x int32, 2 x ptr
    assert ctypes.sizeof(dtattn.Tensor4) == 32
    assert ctypes.sizeof(dtattn.SdpaParams) == 40 + 4 * 32 + 8 + 24 + 8 + 8 + 16 + 16
    assert dtattn.SdpaParams.sinks.offset == 208 and dtattn.SdpaParams.seq_offsets_q.offset == 232
    assert dtattn.lib().dt_abi_version() == 2


def test_status_strings(dtattn):
    assert dtattn.status_string(0) == "ok"
    for code in range(-7, 0):
        assert dtattn.status_string(code) not in ("ok", "unknown status")
    assert dtattn.status_string(-99) == "unknown status"


def _params(dtattn, **over):
    B, Sq, Sk, Hq, Hkv, D = 1, 8, 8, 4, 2, 64
    q = torch.zeros(B, Sq, Hq, D, dtype=torch.float16)
    k = torch.zeros(B, Sk, Hkv, D, dtype=torch.float16)
    v = torch.zeros(B, Sk, Hkv, D, dtype=torch.float16)
    o = torch.zeros(B, Sq, Hq, D, dtype=torch.float16)
    p = dtattn.make_params(q, k, v, o, 0.125)
    for key, val in over.items():
        setattr(p, key, val)
    return p, (q, k, v, o)


def test_bad_arguments_are_rejected(dtattn):
    lib = dtattn.lib()
    n = ctypes.c_size_t()
    assert lib.dt_sdpa_workspace_size(None, ctypes.byref(n)) == dtattn.DT_BAD_ARG
    for over in (dict(Hkv=3), dict(B=0), dict(Sq=-1), dict(D=0), dict(dtype=7), dict(scale=float("nan")),
                 dict(sliding_window=-1), dict(seq_offsets_q=8), dict(seq_offsets_q=8, seq_offsets_k=8, n_seq=0)):
        p, keep = _params(dtattn, **over)
        assert lib.dt_sdpa_workspace_size(ctypes.byref(p), ctypes.byref(n)) == dtattn.DT_BAD_ARG, over
        assert lib.dt_sdpa_forward(ctypes.byref(p), None, 0, None) == dtattn.DT_BAD_ARG, over
    p, keep = _params(dtattn, D=512)
    assert lib.dt_sdpa_workspace_size(ctypes.byref(p), ctypes.byref(n)) == dtattn.DT_UNSUPPORTED
    p, keep = _params(dtattn)
    p.q.ptr = None
    assert lib.dt_sdpa_forward(ctypes.byref(p), None, 0, None) == dtattn.DT_BAD_ARG
    assert lib.dt_device_status(None, None) == dtattn.DT_BAD_ARG
    assert lib.dt_comm_init(None, 0, 1, None, 10) == dtattn.DT_BAD_ARG
    assert lib.dt_comm_unique_id(None) == dtattn.DT_BAD_ARG


def test_noalloc_entry_point_validates_before_anything_runs(dtattn):
    """dt_sdpa_decode_noalloc applies the argument rules of dt_sdpa_forward: misaligned output / sink / log-sum-exp
    pointers, a NaN scale and a negative window come back as DT_BAD_ARG on a machine without any GPU."""
    lib = dtattn.lib()
    for over in (dict(scale=float("nan")), dict(sliding_window=-1), dict(sinks=0x10001), dict(lse=0x10002), dict(B=0)):
        p, keep = _params(dtattn, Sq=1, Sk=512, D=128, **over)
        assert lib.dt_sdpa_decode_noalloc(ctypes.byref(p), None) == dtattn.DT_BAD_ARG, over
    p, keep = _params(dtattn, Sq=1, Sk=512, D=128)
    p.o.ptr = keep[3].data_ptr() + 1
    assert lib.dt_sdpa_decode_noalloc(ctypes.byref(p), None) == dtattn.DT_BAD_ARG
    p, keep = _params(dtattn, Sq=64, Sk=512, D=128)  # 64 rows x 2 heads per KV head: not a decode shape
    assert lib.dt_sdpa_decode_noalloc(ctypes.byref(p), None) == dtattn.DT_UNSUPPORTED
    assert lib.dt_sdpa_decode_noalloc_status(None, None) == dtattn.DT_BAD_ARG


def test_decode_split_flag_changes_the_workspace_only_within_bounds(dtattn):
    """DT_FLAG_DECODE_SPLITS fixes the split count; it is clamped to 256 and to the number of 16-key units, so the
    combining CTA's shared-memory tables cannot be overrun by a caller's value."""
    sizes = {}
    for n in (0, 1, 2, 64, 256, 4095):
        p, keep = _params(dtattn, B=2, Sq=1, Sk=16384, Hq=8, Hkv=2, D=128, flags=dtattn.DT_FLAG_DECODE_SPLITS(n))
        assert dtattn.kernel_name(p) == "decode_splitkv"
        sizes[n] = dtattn.workspace_size(p)
    assert sizes[1] == 0 and sizes[2] < sizes[64] < sizes[256] == sizes[4095]
    p, keep = _params(dtattn, B=1, Sq=1, Sk=48, Hq=8, Hkv=2, D=128, flags=dtattn.DT_FLAG_DECODE_SPLITS(200))
    per_part = 4 * 128 * 4 + 4 * 2 * 4  # one partial of one KV head: 4 rows x (128 floats + m, l)
    assert dtattn.workspace_size(p) <= 4096 + 2 * 256 + 2 * 3 * per_part  # 48 keys = 3 units = at most 3 splits


def test_kernel_selection(dtattn):
    """Which kernel serves which reference call site (decided on the host, no GPU needed)."""
    def pick(B, Sq, Sk, Hq, Hkv, D, dtype, causal=False, flags=0):
        q = torch.zeros(1, dtype=dtype).expand(B, Sq, Hq, D)  # shapes only; never dereferenced
        q = torch.empty_strided((B, Sq, Hq, D), (Sq * Hq * D, Hq * D, D, 1), dtype=dtype, device="meta")
        k = torch.empty_strided((B, Sk, Hkv, D), (Sk * Hkv * D, Hkv * D, D, 1), dtype=dtype, device="meta")
        p = dtattn.SdpaParams()
        p.B, p.Sq, p.Sk, p.Hq, p.Hkv, p.D = B, Sq, Sk, Hq, Hkv, D
        p.dtype = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}[dtype]
        p.scale, p.is_causal, p.flags = D ** -0.5, int(causal), flags
        for name, t in (("q", q), ("k", k), ("v", k), ("o", q)):
            setattr(p, name, dtattn.Tensor4(0x10000, t.stride(0), t.stride(1), t.stride(2)))
        return dtattn.kernel_name(p)

    assert pick(2, 4096, 4096, 8, 8, 40, torch.float32) == "generic"              # SD1.5 self-attention, fp32 (upcast)
    assert pick(2, 4096, 4096, 8, 8, 40, torch.float16) == "prefill_tcgen05"       # SD1.5 in half precision: D padded to 64
    assert pick(2, 4096, 77, 20, 20, 64, torch.float16) == "crossattn_short"       # SDXL cross-attention: 77 text tokens
    assert pick(2, 4096, 77, 8, 8, 40, torch.float16) == "crossattn_short"         # SD1.5 cross-attention
    assert pick(1, 128, 77, 2, 2, 64, torch.float16) == "prefill_tcgen05"          # a handful of rows: the general kernel
    assert pick(2, 64, 77, 20, 20, 64, torch.float16, True) == "prefill_tcgen05"   # causal: the general kernel
    assert pick(2, 4096, 128, 20, 20, 64, torch.float16) == "prefill_tcgen05"      # more than 96 keys
    assert pick(1, 4608, 4608, 24, 24, 128, torch.bfloat16) == "prefill_tcgen05"   # Flux joint attention
    assert pick(1, 4352, 4352, 12, 12, 256, torch.bfloat16) == "prefill_tcgen05"   # AuraFlow joint attention: D = 256
    assert pick(1, 2048, 2048, 16, 4, 256, torch.bfloat16, True) == "prefill_tcgen05"  # Qwen3.5 prompt prefill, D = 256
    assert pick(1, 1, 2048, 16, 4, 256, torch.bfloat16, True) == "decode_splitkv"  # ... and its decode step
    assert pick(2, 256, 256, 8, 8, 160, torch.float16) == "prefill_tcgen05"        # SD1.5 deepest blocks: D = 160 padded to 256
    assert pick(1, 75600, 75600, 5, 5, 128, torch.bfloat16) == "prefill_tcgen05"   # Wan, one rank's heads
    assert pick(16, 1, 8192, 32, 8, 128, torch.float16, True) == "decode_splitkv"  # GQA decode
    assert pick(1, 4608, 4608, 24, 24, 128, torch.bfloat16, flags=2) == "generic"


def test_operator_mirror_validates_like_the_reference(dtattn):
    op = dtattn.ScaledDotProductAttention(scale=0.125, is_causal=True, flags=[dtattn.GEMMFlag.Float16])
    assert op.scale == 0.125 and op.is_causal
    fused = dtattn.ScaledDotProductAttention(scale=1.0, multi_head_output_projection_fused=True)
    with pytest.raises(ValueError):  # the operator owns the unify-heads Dense: its parameters must be set first
        fused(torch.zeros(1, 4, 2, 64, dtype=torch.float16), None, None)
    with pytest.raises(NotImplementedError):
        dtattn.ScaledDotProductAttention(scale=1.0, flags=[dtattn.GEMMFlag.Int8, dtattn.GEMMFlag.Float16])
    q = torch.zeros(1, 4, 2, 64, dtype=torch.float16)
    with pytest.raises(ValueError):
        dtattn.ScaledDotProductAttention(scale=1.0, has_attention_mask=True)(q, q, q)


def test_no_cpu_fallback(dtattn):
    """Host tensors go through the device; without a GPU the call must fail loudly, not compute on the CPU."""
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    q = torch.zeros(1, 4, 2, 64, dtype=torch.float16)
    with pytest.raises(dtattn.DtError) as e:
        dtattn.ScaledDotProductAttention(scale=1.0)(q, q, q)
    assert e.value.status in (dtattn.DT_CUDA, dtattn.DT_NO_DEVICE, dtattn.DT_UNSUPPORTED)


def test_new_entry_points_validate_without_a_gpu(dtattn):
    """Host-side checks of the decode-step, prologue and projected calls: sizes and refusals are decided before
    anything touches a device."""
    lib = dtattn.lib()
    f16 = torch.float16
    q = torch.zeros(1, 1, 8, 128, dtype=f16)
    cache = torch.zeros(1, 4096, 2, 128, dtype=f16)
    new = torch.zeros(1, 1, 2, 128, dtype=f16)
    rot = torch.zeros(1, 1, 128, dtype=f16)
    sp = dtattn.make_step_params(q, cache, cache, new, new, rot, q, 0.1, 3000)
    need = ctypes.c_size_t(0)
    assert lib.dt_sdpa_decode_step_workspace_size(ctypes.byref(sp), ctypes.byref(need)) == dtattn.DT_OK
    assert need.value > 4096                       # split over the cached rows: ticket area plus partials
    sp.T_new = 0
    assert lib.dt_sdpa_decode_step_workspace_size(ctypes.byref(sp), ctypes.byref(need)) == dtattn.DT_BAD_ARG
    sp = dtattn.make_step_params(q, cache, cache, new, new, rot, q, 0.1, 1)   # empty cache: nothing to split
    assert lib.dt_sdpa_decode_step_workspace_size(ctypes.byref(sp), ctypes.byref(need)) == dtattn.DT_OK
    assert need.value == 0

    x = torch.zeros(1, 16, 4, 64, dtype=f16)
    pp = dtattn.make_prologue_params(x, x)
    pp.D = 260
    assert lib.dt_qk_prologue(ctypes.byref(pp), None, None) == dtattn.DT_UNSUPPORTED
    pp = dtattn.make_prologue_params(x, x)
    pp.x.stride_s = 250                             # rows that are not 16-byte aligned
    assert lib.dt_qk_prologue(ctypes.byref(pp), None, None) == dtattn.DT_UNSUPPORTED

    p = dtattn.make_params(x, x, x, x, 0.125)
    pr = dtattn.OutProj()
    w = torch.zeros(512, 256, dtype=f16)
    out = torch.zeros(1, 16, 512, dtype=f16)
    pr.weight, pr.C = w.data_ptr(), 512
    pr.out = dtattn.Tensor4(out.data_ptr(), out.stride(0), out.stride(1), 512)
    assert lib.dt_sdpa_projected_workspace_size(ctypes.byref(p), ctypes.byref(pr), ctypes.byref(need)) == dtattn.DT_OK
    assert need.value == 4096 + 16 * 256 * 2        # ticket area kept clear, then the attention output
    p.dtype = dtattn.DT_F32
    assert lib.dt_sdpa_projected_workspace_size(ctypes.byref(p), ctypes.byref(pr), ctypes.byref(need)) == dtattn.DT_UNSUPPORTED

    # sinks / window / variable length on the plain call: kernel choice is made on the host
    qd = torch.zeros(1, 300, 4, 128, dtype=f16)
    offs = torch.zeros(3, dtype=torch.int32)
    p = dtattn.make_params(qd, qd, qd, qd, 0.1, False, seq_offsets_q=offs, seq_offsets_k=offs, max_seq_q=200, max_seq_k=200)
    assert dtattn.kernel_name(p) == "prefill_tcgen05"
    p = dtattn.make_params(qd, qd, qd, qd, 0.1, True, seq_offsets_q=offs, seq_offsets_k=offs, max_seq_q=200, max_seq_k=200)
    assert dtattn.kernel_name(p) == "generic"
    p = dtattn.make_params(qd, qd, qd, qd, 0.1, True, sliding_window=64, sinks=torch.zeros(4, dtype=f16))
    assert dtattn.kernel_name(p) == "prefill_tcgen05"


def test_projected_headsharded_sizes(dtattn):
    lib = dtattn.lib()
    q = torch.zeros(1, 4608, 3, 128, dtype=torch.bfloat16)
    p = dtattn.make_params(q, q, q, q, 0.1)
    ws, rb, rpr = ctypes.c_size_t(0), ctypes.c_size_t(0), ctypes.c_int(0)
    assert lib.dt_sdpa_projected_headsharded_sizes(ctypes.byref(p), 8, 3072, ctypes.byref(ws), ctypes.byref(rb),
                                                   ctypes.byref(rpr)) == dtattn.DT_OK
    assert rpr.value == 640                                 # ceil(4608 / 8) = 576 rows, rounded up to whole 128-row tiles
    assert rb.value == 2 * 8 * 640 * 3072 * 4               # two sets of fp32 slabs, one per sending rank
    assert ws.value >= 4096 + 4608 * 384 * 2
    assert lib.dt_sdpa_projected_headsharded_sizes(ctypes.byref(p), 9, 3072, None, None, None) == dtattn.DT_BAD_ARG
    assert lib.dt_sdpa_projected_headsharded_sizes(ctypes.byref(p), 8, 3070, None, None, None) == dtattn.DT_UNSUPPORTED
    from dtattn import sharding
    assert sharding.projection_rows(4608, 8)[0] == 640
