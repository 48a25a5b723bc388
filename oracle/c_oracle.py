"""ctypes wrapper around oracle/_build/libsdpa_oracle.so (test infrastructure, never shipped)."""
import ctypes
import os

import torch

from . import build_oracle

_lib = None


def lib():
    global _lib
    if _lib is None:
        path = build_oracle.OUT
        if not os.path.exists(path):
            path = build_oracle.build()
        _lib = ctypes.CDLL(path)
        _lib.sdpa_oracle_f32.restype = ctypes.c_int
        _lib.sdpa_oracle_host_cores.restype = ctypes.c_int
    return _lib


def host_cores():
    return lib().sdpa_oracle_host_cores()


def sdpa_c(q, k, v, scale, is_causal=False, mask=None, nthreads=0, return_lse=False):
    """fp32 C oracle on BSHD torch CPU tensors of any float dtype (values are widened to fp32)."""
    qf, kf, vf = (t.float() if t.dtype != torch.float32 else t for t in (q, k, v))
    B, Sq, Hq, D = qf.shape
    _, Sk, Hkv, _ = kf.shape
    assert qf.stride(3) == 1 and kf.stride(3) == 1 and vf.stride(3) == 1
    o = torch.empty((B, Sq, Hq, D), dtype=torch.float32)
    lse = torch.empty((B, Hq, Sq), dtype=torch.float32) if return_lse else None
    mf = None
    ms = (0, 0, 0)
    if mask is not None:
        mf = mask.float().expand(B, Hq, Sq, Sk)
        assert mf.stride(3) == 1 or Sk == 1
        ms = (mf.stride(0), mf.stride(1), mf.stride(2))
    strides = (ctypes.c_int64 * 15)(
        qf.stride(0), qf.stride(1), qf.stride(2), kf.stride(0), kf.stride(1), kf.stride(2),
        vf.stride(0), vf.stride(1), vf.stride(2), o.stride(0), o.stride(1), o.stride(2), *ms)
    p = ctypes.c_void_p
    n = lib().sdpa_oracle_f32(
        p(qf.data_ptr()), p(kf.data_ptr()), p(vf.data_ptr()), p(o.data_ptr()),
        p(lse.data_ptr()) if lse is not None else None, p(mf.data_ptr()) if mf is not None else None,
        strides, B, Sq, Sk, Hq, Hkv, D, ctypes.c_float(scale), int(is_causal), int(nthreads))
    if n < 0:
        raise ValueError("sdpa_oracle_f32: bad argument")
    return (o, lse) if return_lse else o
