"""The reference arm of bench.py runs on the CPU alone (it times the C restatement of the path on the host cores), so
its JSON line can be checked here: the keys the bench contract names, one line on stdout, and the same metric, unit
and workload as the GPU arm reports."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_contract_line():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                       capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1, lines
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "sdpa_fwd_tflops" and d["unit"] == "TFLOP/s"
    assert d["higher_is_better"] is True and d["vs_baseline"] is None and d["n_gpus"] == 1 and d["steps"] == 1
    assert d["config"]["workload"] == "flux_joint" and "model" not in d["config"]
    assert d["value"] > 0 and d["ms_per_step"] > 0
    cb = d["cpu_baseline"]
    assert cb["kind"] in ("port", "reference") and cb["cores"] >= 1 and cb["sample"] and cb["value"] == d["value"]
    e2e = d["e2e"]
    assert e2e["value"] == d["value"] and e2e["h2d_bytes_per_step"] == 0 and e2e["d2h_bytes_per_step"] == 0


def test_flop_counts():
    """4 B H Sq Sk D for the plain operator; under the causal rule only the visible (query, key) pairs count, and a
    single new token over a cache sees every key."""
    sys.path.insert(0, ROOT)
    import bench
    w = bench.WORKLOADS["flux_joint"]
    assert bench.flops_of(w) == 4 * 1 * 24 * 4608 * 4608 * 128
    assert bench.flops_of(w, heads=3) == 4 * 1 * 3 * 4608 * 4608 * 128
    d = bench.WORKLOADS["decode_b16"]
    assert d["causal"] and bench.flops_of(d) == 4 * 16 * 32 * 1 * 8192 * 128
    c = dict(B=1, Sq=4, Sk=6, Hq=1, Hkv=1, D=2, causal=True)
    visible = sum(6 - 4 + i + 1 for i in range(4))  # rows see 3, 4, 5, 6 keys
    assert abs(bench.flops_of(c) - 4 * visible * 2) < 1e-9
    for name in ("auraflow_joint_d256", "qwen35_prefill_d256"):
        assert bench.WORKLOADS[name]["D"] == 256 and name in bench.SIDE_SHAPES
