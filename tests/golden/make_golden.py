"""Writes tests/golden/sdpa_golden.json and tests/golden/variants_golden.json: sampled outputs of the float64
explicit oracle on small seeded cases.

    python tests/golden/make_golden.py

The reference (drawthingsai/draw-things-community) has no attention fixtures and cannot be run here, so
these vectors come from this repository's own oracle (oracle/sdpa_oracle.py, float64 path).
"""
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import sdpa_oracle as so  # noqa: E402

CASES = [
    dict(B=2, Sq=48, Sk=48, Hq=8, Hkv=8, D=40, causal=False, seed=100),     # SD1.5 self-attention, shrunk
    dict(B=2, Sq=64, Sk=77, Hq=4, Hkv=4, D=64, causal=False, seed=110),     # SDXL cross-attention, shrunk
    dict(B=1, Sq=160, Sk=160, Hq=3, Hkv=3, D=128, causal=False, seed=120),  # Flux / Wan head dim
    dict(B=2, Sq=1, Sk=515, Hq=8, Hkv=2, D=128, causal=True, seed=130),     # GQA decode
    dict(B=1, Sq=4, Sk=130, Hq=8, Hkv=2, D=128, causal=True, seed=140),     # multi-token verify over a cache
    dict(B=1, Sq=96, Sk=96, Hq=2, Hkv=1, D=64, causal=True, seed=150),      # causal prefill
    dict(B=1, Sq=200, Sk=200, Hq=3, Hkv=3, D=256, causal=False, seed=160),  # AuraFlow joint attention head dim, shrunk
    dict(B=1, Sq=150, Sk=280, Hq=4, Hkv=1, D=256, causal=True, seed=170),   # Qwen3.5 prompt continuation: D = 256, grouped heads
    dict(B=2, Sq=70, Sk=70, Hq=2, Hkv=2, D=160, causal=False, seed=180),    # SD1.5 deepest blocks' head dim
]


def sample(t, n=32):
    flat = t.double().flatten()
    idx = [(i * 7919) % flat.numel() for i in range(n)]
    return {"index": idx, "values": [float(x) for x in flat[idx]], "sum": float(flat.sum())}


def variant_cases():
    """Second fixture file: the operator variants and the steps either side of the operator (float64 oracle,
    inputs in bf16/fp16 where the op rounds between stages)."""
    out = {}
    q, k, v = (so.seeded_normal(s, 200 + i) for i, s in enumerate([(1, 40, 8, 64), (1, 40, 2, 64), (1, 40, 2, 64)]))
    sinks = so.seeded_normal((8,), 203) * 2.0
    o = so.sdpa_explicit(q, k, v, 0.125, True, compute_dtype=torch.float64, sinks=sinks, sliding_window=16)
    out["sinks_window"] = sample(o)
    off_q, off_k = [0, 5, 5, 30, 40], [0, 7, 10, 35, 40]
    o = so.sdpa_varlen_explicit(q, k, v, 0.125, off_q, off_k, False, compute_dtype=torch.float64)
    out["varlen"] = sample(o)
    dt = torch.bfloat16
    x = so.seeded_normal((2, 9, 3, 64), 210).to(dt)
    w = (1.0 + 0.3 * so.seeded_normal((64,), 211)).to(dt)
    rot = so.qwen_rotary_table(9, 4, 64, 32).to(dt)[:, :, None, :]
    out["prologue_per_head"] = sample(so.qk_prologue_explicit(x, w, rot, 1e-6, dt))
    w2 = (1.0 + 0.3 * so.seeded_normal((192,), 212)).to(dt)
    out["prologue_per_token"] = sample(so.qk_prologue_explicit(x, w2, rot, 1e-6, dt, True, 64 ** -0.25))
    qd = so.seeded_normal((1, 2, 8, 64), 220).to(dt)
    kn, vn = so.seeded_normal((1, 3, 2, 64), 221).to(dt), so.seeded_normal((1, 3, 2, 64), 222).to(dt)
    kc, vc = so.seeded_normal((1, 50, 2, 64), 223).to(dt), so.seeded_normal((1, 50, 2, 64), 224).to(dt)
    o = so.decode_step_explicit(qd, kc, vc, kn, vn, so.qwen_rotary_table(3, 40, 64).to(dt), 0.125, 40, dt)
    out["decode_step_out"] = sample(o)
    out["decode_step_kcache"] = sample(kc)
    out["decode_step_vcache"] = sample(vc)
    return out


def main():
    vpath = os.path.join(os.path.dirname(os.path.abspath(__file__)), "variants_golden.json")
    with open(vpath, "w") as f:
        json.dump(variant_cases(), f, indent=1)
    print(vpath)
    out = []
    for c in CASES:
        scale = c["D"] ** -0.5
        q = so.seeded_normal((c["B"], c["Sq"], c["Hq"], c["D"]), c["seed"])
        k = so.seeded_normal((c["B"], c["Sk"], c["Hkv"], c["D"]), c["seed"] + 1)
        v = so.seeded_normal((c["B"], c["Sk"], c["Hkv"], c["D"]), c["seed"] + 2)
        o = so.sdpa_explicit(q, k, v, scale, c["causal"], compute_dtype=torch.float64)
        n = o.numel()
        idx = [(i * 7919) % n for i in range(48)]
        out.append({"cfg": dict(c, scale=scale), "index": idx, "values": [float(x) for x in o.flatten()[idx]],
                    "sum": float(o.sum())})
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "sdpa_golden.json")
    with open(path, "w") as f:
        json.dump(out, f, indent=1)
    print(path, len(out))


if __name__ == "__main__":
    main()
