"""ctypes binding of libdtattn.so and a Python mirror of the reference's operator surface.

The reference builds attention as a graph node::

    ScaledDotProductAttention(scale: 1.0 / Float(k).squareRoot(), isCausal: true, flags: [.Float16])(
        queries, keys, values)                       # Libraries/SwiftLLM/Sources/Models/Qwen3_5.swift:193-196

and this module offers the same call shape on torch tensors (used as plain device/host buffers)::

    ScaledDotProductAttention(scale=k ** -0.5, is_causal=True, flags=[GEMMFlag.Float16])(queries, keys, values)

Everything goes through the C ABI in include/dtattn.h.  There is no fallback: if the shared library is
missing, or the tensors are CUDA tensors and the kernels cannot run, the call raises.
"""
from __future__ import annotations

import ctypes
import enum
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("DTATTN_LIB") or os.path.join(_HERE, "..", "lib", "libdtattn.so")

DT_OK, DT_BAD_ARG, DT_UNSUPPORTED, DT_WORKSPACE, DT_CUDA, DT_NCCL, DT_TIMEOUT, DT_NO_DEVICE = 0, -1, -2, -3, -4, -5, -6, -7
DT_SCRATCH_LIMIT = -8
NOALLOC_SCRATCH_BYTES = 8 << 20
DT_F16, DT_BF16, DT_F32 = 0, 1, 2
DT_FLAG_FP16_ACCUM_HINT, DT_FLAG_FORCE_GENERIC, DT_FLAG_KV_PREFIX_STABLE = 1, 2, 4


def DT_FLAG_DECODE_SPLITS(n):
    """Fix the split count of the split-KV decode kernel (1..256; 0 = automatic)."""
    return (int(n) & 0xFFF) << 16


_DTYPES = {torch.float16: DT_F16, torch.bfloat16: DT_BF16, torch.float32: DT_F32}


class Tensor4(ctypes.Structure):
    _fields_ = [("ptr", ctypes.c_void_p), ("stride_b", ctypes.c_int64), ("stride_s", ctypes.c_int64),
                ("stride_h", ctypes.c_int64)]


class SdpaParams(ctypes.Structure):
    _fields_ = [("B", ctypes.c_int32), ("Sq", ctypes.c_int32), ("Sk", ctypes.c_int32), ("Hq", ctypes.c_int32),
                ("Hkv", ctypes.c_int32), ("D", ctypes.c_int32), ("dtype", ctypes.c_int32), ("scale", ctypes.c_float),
                ("is_causal", ctypes.c_int32), ("flags", ctypes.c_uint32),
                ("q", Tensor4), ("k", Tensor4), ("v", Tensor4), ("o", Tensor4),
                ("mask", ctypes.c_void_p), ("mask_stride_b", ctypes.c_int64), ("mask_stride_h", ctypes.c_int64),
                ("mask_stride_q", ctypes.c_int64), ("lse", ctypes.c_void_p),
                ("sinks", ctypes.c_void_p), ("sliding_window", ctypes.c_int32), ("n_seq", ctypes.c_int32),
                ("max_seq_q", ctypes.c_int32), ("max_seq_k", ctypes.c_int32),
                ("seq_offsets_q", ctypes.c_void_p), ("seq_offsets_k", ctypes.c_void_p)]


class DecodeStepParams(ctypes.Structure):
    _fields_ = [("attn", SdpaParams), ("k_new", Tensor4), ("v_new", Tensor4), ("T_new", ctypes.c_int32),
                ("rotary", ctypes.c_void_p), ("rotary_stride_b", ctypes.c_int64), ("rotary_stride_s", ctypes.c_int64),
                ("q_norm_weight", ctypes.c_void_p), ("k_norm_weight", ctypes.c_void_p), ("norm_eps", ctypes.c_float)]


class QkPrologueParams(ctypes.Structure):
    _fields_ = [("B", ctypes.c_int32), ("S", ctypes.c_int32), ("H", ctypes.c_int32), ("D", ctypes.c_int32),
                ("dtype", ctypes.c_int32), ("x", Tensor4), ("y", Tensor4), ("norm_weight", ctypes.c_void_p),
                ("norm_per_token", ctypes.c_int32), ("eps", ctypes.c_float), ("rotary", ctypes.c_void_p),
                ("rotary_stride_b", ctypes.c_int64), ("rotary_stride_s", ctypes.c_int64),
                ("rotary_stride_h", ctypes.c_int64), ("post_scale", ctypes.c_float)]


class OutProj(ctypes.Structure):
    _fields_ = [("weight", ctypes.c_void_p), ("bias", ctypes.c_void_p), ("C", ctypes.c_int32), ("out", Tensor4)]


class SparseIndexedParams(ctypes.Structure):
    _fields_ = [("B", ctypes.c_int32), ("Sq", ctypes.c_int32), ("Hq", ctypes.c_int32), ("Hkv", ctypes.c_int32),
                ("D", ctypes.c_int32), ("Sr", ctypes.c_int32), ("Sc", ctypes.c_int32), ("n_selected", ctypes.c_int32),
                ("dtype", ctypes.c_int32), ("scale", ctypes.c_float), ("is_causal", ctypes.c_int32),
                ("sliding_window", ctypes.c_int32),
                ("q", Tensor4), ("o", Tensor4), ("k_raw", Tensor4), ("v_raw", Tensor4), ("k_comp", Tensor4), ("v_comp", Tensor4),
                ("selected", ctypes.c_void_p), ("selected_stride_b", ctypes.c_int64), ("selected_stride_q", ctypes.c_int64),
                ("sinks", ctypes.c_void_p), ("lse", ctypes.c_void_p), ("flags", ctypes.c_uint32)]


class DtError(RuntimeError):
    def __init__(self, status, what):
        self.status = status
        super().__init__(f"{what}: {status_string(status)} ({status})")


_lib = None

# every symbol include/dtattn.h declares: (name, restype, argtypes)
_P = ctypes.POINTER
SYMBOLS = [
    ("dt_status_string", ctypes.c_char_p, [ctypes.c_int]),
    ("dt_last_cuda_error", ctypes.c_int, []),
    ("dt_abi_version", ctypes.c_int, []),
    ("dt_sdpa_workspace_size", ctypes.c_int, [_P(SdpaParams), _P(ctypes.c_size_t)]),
    ("dt_sdpa_workspace_init", ctypes.c_int, [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]),
    ("dt_sdpa_forward", ctypes.c_int, [_P(SdpaParams), ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]),
    ("dt_sdpa_kernel_name", ctypes.c_int, [_P(SdpaParams), _P(ctypes.c_char_p)]),
    ("dt_sdpa_forward_host", ctypes.c_int, [_P(SdpaParams)]),
    ("dt_host_release", ctypes.c_int, []),
    ("dt_device_status", ctypes.c_int, [ctypes.c_void_p, _P(ctypes.c_int)]),
    ("dt_sdpa_decode_step_workspace_size", ctypes.c_int, [_P(DecodeStepParams), _P(ctypes.c_size_t)]),
    ("dt_sdpa_decode_step", ctypes.c_int, [_P(DecodeStepParams), ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]),
    ("dt_sdpa_decode_noalloc", ctypes.c_int, [_P(SdpaParams), ctypes.c_void_p]),
    ("dt_sdpa_decode_noalloc_status", ctypes.c_int, [ctypes.c_void_p, _P(ctypes.c_int)]),
    ("dt_sdpa_projected_workspace_size", ctypes.c_int, [_P(SdpaParams), _P(OutProj), _P(ctypes.c_size_t)]),
    ("dt_sdpa_forward_projected", ctypes.c_int,
     [_P(SdpaParams), _P(OutProj), ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]),
    ("dt_qk_prologue", ctypes.c_int, [_P(QkPrologueParams), _P(QkPrologueParams), ctypes.c_void_p]),
    ("dt_sparse_indexed_attention", ctypes.c_int, [_P(SparseIndexedParams), ctypes.c_void_p]),
    ("dt_comm_unique_id", ctypes.c_int, [ctypes.c_void_p]),
    ("dt_comm_init", ctypes.c_int, [_P(ctypes.c_void_p), ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_int]),
    ("dt_comm_destroy", ctypes.c_int, [ctypes.c_void_p]),
    ("dt_comm_register_output", ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t]),
    ("dt_sdpa_headsharded_workspace_size", ctypes.c_int, [_P(SdpaParams), ctypes.c_int, ctypes.c_int, _P(ctypes.c_size_t)]),
    ("dt_sdpa_forward_headsharded", ctypes.c_int,
     [ctypes.c_void_p, _P(SdpaParams), Tensor4, ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]),
    ("dt_sdpa_projected_headsharded_sizes", ctypes.c_int,
     [_P(SdpaParams), ctypes.c_int, ctypes.c_int, _P(ctypes.c_size_t), _P(ctypes.c_size_t), _P(ctypes.c_int)]),
    ("dt_sdpa_forward_projected_headsharded", ctypes.c_int,
     [ctypes.c_void_p, _P(SdpaParams), ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, Tensor4,
      ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]),
    ("dt_permute_gathered", ctypes.c_int,
     [ctypes.c_void_p, Tensor4, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
      ctypes.c_void_p]),
]


def lib():
    """The loaded library.  Raises (never falls back) when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} not found: build it with `python draw-things-community_b200/build.py`")
        _lib = ctypes.CDLL(os.path.abspath(LIB_PATH))
        for name, res, args in SYMBOLS:
            fn = getattr(_lib, name)
            fn.restype = res
            fn.argtypes = args
    return _lib


def status_string(status):
    return lib().dt_status_string(int(status)).decode()


def _check(status, what):
    if status != DT_OK:
        raise DtError(status, what)


def _view4(t: torch.Tensor) -> Tensor4:
    assert t.dim() == 4 and (t.stride(3) == 1 or t.shape[3] == 1), "expect a [B,S,H,D] view with contiguous D"
    return Tensor4(t.data_ptr(), t.stride(0), t.stride(1), t.stride(2))


def make_params(q, k, v, o, scale, is_causal=False, mask=None, lse=None, flags=0, sinks=None, sliding_window=0,
                seq_offsets_q=None, seq_offsets_k=None, max_seq_q=0, max_seq_k=0) -> SdpaParams:
    B, Sq, Hq, D = q.shape
    _, Sk, Hkv, _ = k.shape
    p = SdpaParams()
    p.B, p.Sq, p.Sk, p.Hq, p.Hkv, p.D = B, Sq, Sk, Hq, Hkv, D
    p.dtype = _DTYPES[q.dtype]
    p.scale = float(scale)
    p.is_causal = int(bool(is_causal))
    p.flags = int(flags)
    p.q, p.k, p.v, p.o = _view4(q), _view4(k), _view4(v), _view4(o)
    if mask is not None:
        assert mask.dtype == q.dtype and mask.dim() == 4 and mask.shape[2] == Sq and mask.shape[3] == Sk
        assert mask.stride(3) == 1 or Sk == 1
        p.mask = mask.data_ptr()
        p.mask_stride_b = mask.stride(0) if mask.shape[0] > 1 else 0
        p.mask_stride_h = mask.stride(1) if mask.shape[1] > 1 else 0
        p.mask_stride_q = mask.stride(2)
    if lse is not None:
        assert lse.dtype == torch.float32 and lse.is_contiguous() and tuple(lse.shape) == (B, Hq, Sq)
        p.lse = lse.data_ptr()
    if sinks is not None:
        assert sinks.dtype == q.dtype and sinks.is_contiguous() and sinks.numel() == Hq
        p.sinks = sinks.data_ptr()
    p.sliding_window = int(sliding_window)
    if seq_offsets_q is not None:
        for t in (seq_offsets_q, seq_offsets_k):
            assert t.dtype == torch.int32 and t.is_contiguous() and t.device == q.device
        assert seq_offsets_q.numel() == seq_offsets_k.numel() >= 2
        p.n_seq = seq_offsets_q.numel() - 1
        p.seq_offsets_q, p.seq_offsets_k = seq_offsets_q.data_ptr(), seq_offsets_k.data_ptr()
        p.max_seq_q, p.max_seq_k = int(max_seq_q or Sq), int(max_seq_k or Sk)
    return p


def kernel_name(p: SdpaParams) -> str:
    name = ctypes.c_char_p()
    _check(lib().dt_sdpa_kernel_name(ctypes.byref(p), ctypes.byref(name)), "dt_sdpa_kernel_name")
    return name.value.decode()


def workspace_size(p: SdpaParams) -> int:
    n = ctypes.c_size_t(0)
    _check(lib().dt_sdpa_workspace_size(ctypes.byref(p), ctypes.byref(n)), "dt_sdpa_workspace_size")
    return n.value


def device_status(stream=None) -> int:
    """Read and clear the device status word (0 = healthy)."""
    code = ctypes.c_int(0)
    s = stream if stream is not None else torch.cuda.current_stream().cuda_stream
    st = lib().dt_device_status(ctypes.c_void_p(s), ctypes.byref(code))
    if st not in (DT_OK, DT_TIMEOUT):
        raise DtError(st, "dt_device_status")
    return code.value


class Workspace:
    """Caller-owned scratch for dt_sdpa_forward, grown on demand and zero-initialised when (re)allocated."""

    def __init__(self, device):
        self.device = device
        self.buf = None

    def ensure(self, nbytes, stream):
        if nbytes == 0:
            return None, 0
        if self.buf is None or self.buf.numel() < nbytes:
            self.buf = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
            _check(lib().dt_sdpa_workspace_init(ctypes.c_void_p(self.buf.data_ptr()), self.buf.numel(),
                                                ctypes.c_void_p(stream)), "dt_sdpa_workspace_init")
        return self.buf.data_ptr(), self.buf.numel()


def sdpa_forward(q, k, v, scale, is_causal=False, mask=None, out=None, lse=None, flags=0, workspace=None,
                 stream=None, sinks=None, sliding_window=0, seq_offsets_q=None, seq_offsets_k=None, max_seq_q=0,
                 max_seq_k=0):
    """O = softmax(scale * Q K^T [+mask] [causal]) V through the C ABI.

    CUDA tensors -> dt_sdpa_forward on the current (or given) stream; CPU tensors -> dt_sdpa_forward_host,
    which stages through device memory (the end-to-end path).
    """
    B, Sq, Hq, D = q.shape
    if out is None:
        out = torch.empty((B, Sq, Hq, D), dtype=q.dtype, device=q.device)
    p = make_params(q, k, v, out, scale, is_causal, mask, lse, flags, sinks, sliding_window, seq_offsets_q,
                    seq_offsets_k, max_seq_q, max_seq_k)
    if q.is_cuda:
        s = stream if stream is not None else torch.cuda.current_stream(q.device).cuda_stream
        ws = workspace if workspace is not None else _default_workspace(q.device)
        ptr, nbytes = ws.ensure(workspace_size(p), s)
        _check(lib().dt_sdpa_forward(ctypes.byref(p), ctypes.c_void_p(ptr) if ptr else None, nbytes,
                                     ctypes.c_void_p(s)), "dt_sdpa_forward")
    else:
        _check(lib().dt_sdpa_forward_host(ctypes.byref(p)), "dt_sdpa_forward_host")
    return out


def make_step_params(q, k_cache, v_cache, k_new, v_new, rotary, o, scale, total_len, is_causal=True,
                     lse=None, flags=0, q_norm_weight=None, k_norm_weight=None, norm_eps=1e-6, sinks=None,
                     sliding_window=0) -> DecodeStepParams:
    """k_cache / v_cache: [B, capacity, Hkv, D]; the step attends over their first `total_len` rows, of which
    the last k_new.shape[1] are written by the call."""
    sp = DecodeStepParams()
    sp.attn = make_params(q, k_cache[:, :total_len], v_cache[:, :total_len], o, scale, is_causal, None, lse, flags, sinks,
                          sliding_window)
    sp.k_new, sp.v_new = _view4(k_new), _view4(v_new)
    sp.T_new = k_new.shape[1]
    if rotary is not None:
        assert rotary.dim() == 3 and rotary.dtype == q.dtype and rotary.shape[1] == k_new.shape[1]
        assert rotary.stride(2) == 1
        sp.rotary = rotary.data_ptr()
        sp.rotary_stride_b = rotary.stride(0) if rotary.shape[0] > 1 else 0
        sp.rotary_stride_s = rotary.stride(1)
    for name, wt in (("q_norm_weight", q_norm_weight), ("k_norm_weight", k_norm_weight)):
        if wt is not None:
            assert wt.dtype == q.dtype and wt.is_contiguous() and wt.numel() == q.shape[3]
            setattr(sp, name, wt.data_ptr())
    sp.norm_eps = float(norm_eps)
    return sp


def decode_step(q, k_cache, v_cache, k_new, v_new, rotary, scale, cached_len, out=None, lse=None, workspace=None,
                stream=None, flags=0, q_norm_weight=None, k_norm_weight=None, norm_eps=1e-6, sinks=None, sliding_window=0):
    """One KV-cache step in one launch (Qwen3_5.swift:167-196): rotate q and k_new with `rotary`
    ([B or 1, T_new, D], interleaved cos/sin), write rotated k_new and v_new into cache rows
    [cached_len, cached_len + T_new) and return causal attention of the rotated queries over rows
    [0, cached_len + T_new).  q holds the last Sq <= T_new tokens' queries."""
    assert q.is_cuda, "the fused decode step takes device tensors"
    B, Sq, Hq, D = q.shape
    if out is None:
        out = torch.empty((B, Sq, Hq, D), dtype=q.dtype, device=q.device)
    sp = make_step_params(q, k_cache, v_cache, k_new, v_new, rotary, out, scale, cached_len + k_new.shape[1], True, lse,
                          flags, q_norm_weight, k_norm_weight, norm_eps, sinks, sliding_window)
    need = ctypes.c_size_t(0)
    _check(lib().dt_sdpa_decode_step_workspace_size(ctypes.byref(sp), ctypes.byref(need)),
           "dt_sdpa_decode_step_workspace_size")
    s = stream if stream is not None else torch.cuda.current_stream(q.device).cuda_stream
    ws = workspace if workspace is not None else _default_workspace(q.device)
    ptr, nbytes = ws.ensure(need.value, s)
    _check(lib().dt_sdpa_decode_step(ctypes.byref(sp), ctypes.c_void_p(ptr) if ptr else None, nbytes,
                                     ctypes.c_void_p(s)), "dt_sdpa_decode_step")
    return out


def make_prologue_params(x, y, norm_weight=None, rotary=None, eps=1e-6, norm_per_token=False,
                         post_scale=1.0) -> QkPrologueParams:
    p = QkPrologueParams()
    p.B, p.S, p.H, p.D = x.shape
    p.dtype = _DTYPES[x.dtype]
    p.x, p.y = _view4(x), _view4(y)
    if norm_weight is not None:
        assert norm_weight.dtype == x.dtype and norm_weight.is_contiguous()
        assert norm_weight.numel() == (p.H * p.D if norm_per_token else p.D)
        p.norm_weight = norm_weight.data_ptr()
    p.norm_per_token = int(bool(norm_per_token))
    p.eps = float(eps)
    if rotary is not None:
        assert rotary.dim() == 4 and rotary.dtype == x.dtype and rotary.stride(3) == 1
        assert rotary.shape[1] == p.S and rotary.shape[3] == p.D
        p.rotary = rotary.data_ptr()
        p.rotary_stride_b = rotary.stride(0) if rotary.shape[0] > 1 else 0
        p.rotary_stride_s = rotary.stride(1)
        p.rotary_stride_h = rotary.stride(2) if rotary.shape[2] > 1 else 0
    p.post_scale = float(post_scale)
    return p


def qk_prologue(q, k=None, *, q_out=None, k_out=None, q_weight=None, k_weight=None, rotary=None, rotary_k=None,
                eps=1e-6, norm_per_token=False, post_scale=1.0, stream=None):
    """RMSNorm, rotary cmul and pre-scale of queries and keys in one launch (the nodes before the attention
    node at Flux1.swift:164-188, Wan.swift:86-98, Qwen3_5.swift:164-182).  Outputs default to new tensors; pass
    q_out / k_out views (e.g. row-offset views of a joint buffer) to write in place or to fuse a concat."""
    assert q.is_cuda
    q_out = torch.empty_like(q) if q_out is None else q_out
    pq = make_prologue_params(q, q_out, q_weight, rotary, eps, norm_per_token, post_scale)
    pk = None
    if k is not None:
        k_out = torch.empty_like(k) if k_out is None else k_out
        pk = make_prologue_params(k, k_out, k_weight, rotary if rotary_k is None else rotary_k, eps, norm_per_token,
                                  post_scale)
    s = stream if stream is not None else torch.cuda.current_stream(q.device).cuda_stream
    _check(lib().dt_qk_prologue(ctypes.byref(pq), ctypes.byref(pk) if pk is not None else None, ctypes.c_void_p(s)),
           "dt_qk_prologue")
    return q_out, k_out


def sdpa_forward_projected(q, k, v, scale, weight, bias=None, is_causal=False, out=None, workspace=None, stream=None):
    """Attention followed by the "unify heads" Dense in one call (multiHeadOutputProjectionFused,
    UNet.swift:122-130): returns [B, Sq, C] = concat_heads(attention) @ weight.T + bias, weight [C, Hq*D]."""
    assert q.is_cuda, "the projected call takes device tensors"
    B, Sq, Hq, D = q.shape
    C = weight.shape[0]
    assert weight.dtype == q.dtype and weight.is_contiguous() and weight.shape[1] == Hq * D
    if out is None:
        out = torch.empty((B, Sq, C), dtype=q.dtype, device=q.device)
    assert out.stride(2) == 1
    p = make_params(q, k, v, q, scale, is_causal)  # o is a placeholder: the attention output stays in the workspace
    pr = OutProj()
    pr.weight = weight.data_ptr()
    if bias is not None:
        assert bias.dtype == q.dtype and bias.is_contiguous() and bias.numel() == C
        pr.bias = bias.data_ptr()
    pr.C = C
    pr.out = Tensor4(out.data_ptr(), out.stride(0), out.stride(1), C)
    need = ctypes.c_size_t(0)
    _check(lib().dt_sdpa_projected_workspace_size(ctypes.byref(p), ctypes.byref(pr), ctypes.byref(need)),
           "dt_sdpa_projected_workspace_size")
    s = stream if stream is not None else torch.cuda.current_stream(q.device).cuda_stream
    ws = workspace if workspace is not None else _default_workspace(q.device)
    ptr, nbytes = ws.ensure(need.value, s)
    _check(lib().dt_sdpa_forward_projected(ctypes.byref(p), ctypes.byref(pr), ctypes.c_void_p(ptr), nbytes,
                                           ctypes.c_void_p(s)), "dt_sdpa_forward_projected")
    return out


def sparse_indexed_attention(q, k_raw, v_raw, k_comp, v_comp, selected, scale, sinks=None, sliding_window=0,
                             is_causal=True, out=None, lse=None, stream=None, flags=0):
    """SparseIndexedAttention (DeepSeek4.swift:521-545): q [B,Sq,Hq,D] over its sliding causal window of the raw rows
    k_raw / v_raw [B,Sr,Hkv,D] and over the rows of k_comp / v_comp [B,Sc,Hkv,D] (None when there are none) that
    `selected` (int32 [B or 1, Sq, n_selected]; entries outside [0, Sc) mean "no row") names, in one softmax with the
    sinks [Hq].  Device tensors."""
    assert q.is_cuda
    B, Sq, Hq, D = q.shape
    if out is None:
        out = torch.empty_like(q)
    p = SparseIndexedParams()
    p.B, p.Sq, p.Hq, p.Hkv, p.D = B, Sq, Hq, k_raw.shape[2], D
    p.Sr = k_raw.shape[1]
    p.Sc = 0 if k_comp is None else k_comp.shape[1]
    p.dtype = _DTYPES[q.dtype]
    p.scale = float(scale)
    p.is_causal = int(bool(is_causal))
    p.sliding_window = int(sliding_window)
    p.flags = int(flags)
    p.q, p.o, p.k_raw, p.v_raw = _view4(q), _view4(out), _view4(k_raw), _view4(v_raw)
    if k_comp is not None and p.Sc > 0:
        p.k_comp, p.v_comp = _view4(k_comp), _view4(v_comp)
    if selected is not None:
        assert selected.dtype == torch.int32 and selected.dim() == 3 and selected.shape[1] == Sq and selected.stride(2) == 1
        p.n_selected = selected.shape[2]
        p.selected = selected.data_ptr()
        p.selected_stride_b = selected.stride(0) if selected.shape[0] > 1 else 0
        p.selected_stride_q = selected.stride(1)
    if sinks is not None:
        assert sinks.dtype == q.dtype and sinks.is_contiguous() and sinks.numel() == Hq
        p.sinks = sinks.data_ptr()
    if lse is not None:
        assert lse.dtype == torch.float32 and lse.is_contiguous() and tuple(lse.shape) == (B, Hq, Sq)
        p.lse = lse.data_ptr()
    s = stream if stream is not None else torch.cuda.current_stream(q.device).cuda_stream
    _check(lib().dt_sparse_indexed_attention(ctypes.byref(p), ctypes.c_void_p(s)), "dt_sparse_indexed_attention")
    return out


class SparseIndexedAttention:
    """NNC.SparseIndexedAttention(scale:isCausal:hasAttentionSinks:slidingWindow:) with the reference's input order
    (DeepSeek4.swift:536-545): op(queries, rawKeys, rawValues, compressedKeys, compressedValues, selectedRows, sinks)."""

    def __init__(self, scale, is_causal=True, has_attention_sinks=True, sliding_window=0, name=""):
        self.scale, self.is_causal = float(scale), bool(is_causal)
        self.has_attention_sinks, self.sliding_window, self.name = bool(has_attention_sinks), int(sliding_window), name

    def __call__(self, queries, raw_keys, raw_values, compressed_keys, compressed_values, selected_rows, sinks=None, out=None):
        if self.has_attention_sinks != (sinks is not None):
            raise ValueError("hasAttentionSinks and the number of inputs disagree")
        if selected_rows is not None and selected_rows.dim() == 2:  # the reference passes [queryLength, selectedRowCount]
            selected_rows = selected_rows.unsqueeze(0)
        return sparse_indexed_attention(queries, raw_keys, raw_values, compressed_keys, compressed_values, selected_rows,
                                        self.scale, None if sinks is None else sinks.reshape(-1).contiguous(),
                                        self.sliding_window, self.is_causal, out=out)


_workspaces = {}


def _default_workspace(device):
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    if key not in _workspaces:
        _workspaces[key] = Workspace(device)
    return _workspaces[key]


# --------------------------------------------------------------------------------------------------
# Mirror of the reference operator
# --------------------------------------------------------------------------------------------------

class GEMMFlag(enum.Flag):
    """Functional.GEMMFlag as passed by the reference's call sites (UNet.swift:124, Flux1.swift:229-231)."""
    NONE = 0
    Float16 = 1   # half-precision accumulation allowed; this library always accumulates in fp32
    Float32 = 2
    Int8 = 4      # quantised-attention hint; only selected on Metal in the reference (DeviceCapability.swift:132-146)


class ScaledDotProductAttention:
    """NNC.ScaledDotProductAttention(scale:isCausal:hasAttentionMask:flags:multiHeadOutputProjectionFused:name:).

    Argument meaning follows the reference call sites:
      scale                 multiplies Q.K^T (1 for FlashAttentionLevel.scale1, 1/sqrt(k) for .scaleMerged)
      is_causal             bottom-right aligned causal mask (Qwen3_5.swift:193-196)
      has_attention_mask    a 4th input [B|1, H|1, Sq, Sk] is added to the scores (CLIPTextModel.swift:46-51)
      flags                 GEMMFlag set; accepted for signature parity
      has_attention_sinks   a 4th input [1,1,H,1]: one extra unscaled score per head in the softmax denominator
      sliding_window        only the last W keys up to the query's own position are visible
      is_variable_length    packed rows; two more inputs hold the int32 sequence offsets (n_seq + 1 entries each);
                            max_sequence_length = (query, keyValue) bounds of one sequence
      multi_head_output_projection_fused
                            the output Dense is part of the op (UNet.swift:122-130): the result is
                            [B, Sq, C] = concat_heads(attention) @ weight.T + bias
    Like the reference, misuse is a hard error (the reference traps with precondition/fatalError).
    """

    def __init__(self, scale, is_causal=False, has_attention_mask=False, flags=(), multi_head_output_projection_fused=False,
                 name="", has_attention_sinks=False, sliding_window=0, is_variable_length=False,
                 max_sequence_length=None):
        # hasAttentionSinks / slidingWindow: DeepSeek4.swift:482-493; isVariableLength / maxSequenceLength
        # (query:, keyValue:): Qwen3_5VL.swift:428-437
        self.has_attention_sinks = bool(has_attention_sinks)
        self.sliding_window = int(sliding_window or 0)
        self.is_variable_length = bool(is_variable_length)
        self.max_sequence_length = max_sequence_length
        # multiHeadOutputProjectionFused: the operator owns the unify-heads Dense; its parameters are set with
        # set_output_projection (the reference copies them into the model's .weight / .bias, UNet.swift:865-874)
        self.multi_head_output_projection_fused = bool(multi_head_output_projection_fused)
        self.weight = self.bias = None
        self.scale = float(scale)
        self.is_causal = bool(is_causal)
        self.has_attention_mask = bool(has_attention_mask)
        self.name = name
        f = GEMMFlag.NONE
        for x in (flags if isinstance(flags, (list, tuple, set)) else [flags]):
            f |= x
        self.flags = f
        if GEMMFlag.Int8 in f:
            raise NotImplementedError("quantised attention ([.Int8, .Float16]) is never selected off Metal")

    def set_output_projection(self, weight, bias=None):
        self.weight, self.bias = weight, bias

    def __call__(self, queries, keys, values, *extra, mask=None, out=None, lse=None):
        """Extra positional inputs follow the reference's order: the mask (hasAttentionMask), or the sinks tensor
        (hasAttentionSinks, DeepSeek4.swift:489-493), or the two sequence-offset tensors (isVariableLength,
        Qwen3_5VL.swift:434)."""
        extra = list(extra)
        sinks = offs_q = offs_k = None
        if self.has_attention_mask and mask is None and extra:
            mask = extra.pop(0)
        if self.has_attention_sinks:
            if not extra:
                raise ValueError("hasAttentionSinks needs the sinks input")
            sinks = extra.pop(0).reshape(-1).contiguous()
        if self.is_variable_length:
            if len(extra) < 2:
                raise ValueError("isVariableLength needs the query and key/value sequence offsets")
            offs_q, offs_k = extra.pop(0), extra.pop(0)
        if extra:
            raise ValueError("more inputs than the operator was built for")
        if self.has_attention_mask != (mask is not None):
            raise ValueError("hasAttentionMask and the number of inputs disagree")
        abi_flags = DT_FLAG_FP16_ACCUM_HINT if GEMMFlag.Float16 in self.flags else 0
        if self.multi_head_output_projection_fused:
            if self.weight is None:
                raise ValueError("multiHeadOutputProjectionFused: set_output_projection(weight, bias) first")
            if mask is not None or sinks is not None or offs_q is not None or self.sliding_window or lse is not None:
                raise NotImplementedError("the fused output projection takes the plain operator only")
            return sdpa_forward_projected(queries, keys, values, self.scale, self.weight, self.bias, self.is_causal, out=out)
        mq, mk = self.max_sequence_length if self.max_sequence_length else (0, 0)
        return sdpa_forward(queries, keys, values, self.scale, self.is_causal, mask, out=out, lse=lse, flags=abi_flags,
                            sinks=sinks, sliding_window=self.sliding_window, seq_offsets_q=offs_q, seq_offsets_k=offs_k,
                            max_seq_q=mq, max_seq_k=mk)


# --------------------------------------------------------------------------------------------------
# Head-sharded multi-GPU
# --------------------------------------------------------------------------------------------------

class HeadShardedComm:
    """One communicator per process (one process per GPU).  `store_bcast(bytes|None) -> bytes` ships rank 0's
    128-byte id to every rank (torch.distributed's broadcast_object_list does)."""

    def __init__(self, rank, world, store_bcast, timeout_ms=60000):
        self.rank, self.world = rank, world
        ident = None
        if rank == 0:
            buf = ctypes.create_string_buffer(128)
            _check(lib().dt_comm_unique_id(buf), "dt_comm_unique_id")
            ident = buf.raw
        ident = store_bcast(ident)
        self.handle = ctypes.c_void_p()
        _check(lib().dt_comm_init(ctypes.byref(self.handle), rank, world, ident, timeout_ms), "dt_comm_init")
        self.ws = None

    def register_output(self, o_full):
        """Collective.  After this, forward(..., o_full) stores output tiles straight into every rank's o_full
        from the attention epilogue (fused mode) instead of all-gather + permute."""
        assert o_full.is_contiguous()
        _check(lib().dt_comm_register_output(self.handle, ctypes.c_void_p(o_full.data_ptr()),
                                             o_full.numel() * o_full.element_size()), "dt_comm_register_output")

    def forward(self, q_local, k_local, v_local, scale, o_full, chunks=1, is_causal=False, stream=None):
        """q_local [B,Sq,H/world,D] etc. -> o_full [B,Sq,H,D] on every rank."""
        dummy_o = q_local  # `o` of the local params is ignored by the head-sharded entry point
        p = make_params(q_local, k_local, v_local, dummy_o, scale, is_causal)
        n = ctypes.c_size_t(0)
        _check(lib().dt_sdpa_headsharded_workspace_size(ctypes.byref(p), self.world, chunks, ctypes.byref(n)),
               "dt_sdpa_headsharded_workspace_size")
        s = stream if stream is not None else torch.cuda.current_stream(q_local.device).cuda_stream
        if self.ws is None or self.ws.numel() < n.value:
            self.ws = torch.zeros(n.value, dtype=torch.uint8, device=q_local.device)
        _check(lib().dt_sdpa_forward_headsharded(self.handle, ctypes.byref(p), _view4(o_full), chunks,
                                                 ctypes.c_void_p(self.ws.data_ptr()), self.ws.numel(),
                                                 ctypes.c_void_p(s)), "dt_sdpa_forward_headsharded")
        return o_full

    def projected_sizes(self, q_local, k_local, v_local, scale, C, is_causal=False):
        """(workspace bytes, receive-buffer bytes, rows per rank) of forward_projected for these shapes."""
        p = make_params(q_local, k_local, v_local, q_local, scale, is_causal)
        ws, rb, rpr = ctypes.c_size_t(0), ctypes.c_size_t(0), ctypes.c_int(0)
        _check(lib().dt_sdpa_projected_headsharded_sizes(ctypes.byref(p), self.world, C, ctypes.byref(ws), ctypes.byref(rb),
                                                         ctypes.byref(rpr)), "dt_sdpa_projected_headsharded_sizes")
        return ws.value, rb.value, rpr.value

    def forward_projected(self, q_local, k_local, v_local, scale, weight_local, bias, recv, out_rows, is_causal=False,
                          stream=None):
        """Local head slice, row-parallel output projection and reduce-scatter in one call: this rank's rows
        [rank * rows_per_rank, ...) of the flattened [B*Sq, C] output land in out_rows ([rows_per_rank, C]).  recv is
        the fp32 receive buffer registered on every rank with register_output."""
        C = weight_local.shape[0]
        p = make_params(q_local, k_local, v_local, q_local, scale, is_causal)
        need, _, _ = self.projected_sizes(q_local, k_local, v_local, scale, C, is_causal)
        s = stream if stream is not None else torch.cuda.current_stream(q_local.device).cuda_stream
        if getattr(self, "proj_ws", None) is None:
            self.proj_ws = Workspace(q_local.device)
        ptr, nbytes = self.proj_ws.ensure(need, s)
        rows = Tensor4(out_rows.data_ptr(), 0, out_rows.stride(0), C)
        _check(lib().dt_sdpa_forward_projected_headsharded(
            self.handle, ctypes.byref(p), ctypes.c_void_p(weight_local.data_ptr()),
            ctypes.c_void_p(bias.data_ptr()) if bias is not None else None, C, ctypes.c_void_p(recv.data_ptr()), rows,
            ctypes.c_void_p(ptr), nbytes, ctypes.c_void_p(s)), "dt_sdpa_forward_projected_headsharded")
        return out_rows

    def close(self):
        if self.handle:
            lib().dt_comm_destroy(self.handle)
            self.handle = ctypes.c_void_p()
