"""Writes tests/golden/sdpa_golden.json: sampled outputs of the float64 explicit oracle on small seeded cases.

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
]


def main():
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
