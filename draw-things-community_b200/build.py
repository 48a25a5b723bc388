"""Build lib/libdtattn.so (sm_100a only) from csrc/*.cu with nvcc.  No GPU is needed to build.

    python draw-things-community_b200/build.py [--force] [--verbose] [--define NAME[=VALUE] ...] [--out PATH]

--define adds preprocessor definitions (DT_BRINGUP compiles the timeline probes and the environment overrides of
the bring-up builds in); a build with definitions must name its own --out, and keeps its objects beside it, so it
never replaces the product library.
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB_DIR = os.path.join(HERE, "lib")
LIB = os.path.join(LIB_DIR, "libdtattn.so")
SOURCES = ["api.cu", "generic.cu", "decode_splitkv.cu", "prefill_sm100.cu", "crossattn_short.cu", "sparse_indexed.cu", "comm.cu", "qk_prologue.cu", "out_proj.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]


def _newest(paths):
    return max(os.path.getmtime(p) for p in paths)


def _headers():
    return [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))] + \
           [os.path.join(HERE, "..", "include", "dtattn.h")]


def build(force=False, verbose=False, defines=(), out=None):
    if defines and not out:
        raise ValueError("a build with --define needs its own --out")
    lib = os.path.abspath(out) if out else LIB
    obj_dir = os.path.join(os.path.dirname(lib), "obj_" + os.path.basename(lib)) if out else OBJ
    os.makedirs(obj_dir, exist_ok=True)
    os.makedirs(os.path.dirname(lib), exist_ok=True)
    hdr_time = _newest(_headers())
    jobs = []
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(obj_dir, src.replace(".cu", ".o"))
        if force or not os.path.exists(o) or os.path.getmtime(o) < max(os.path.getmtime(s), hdr_time):
            cmd = ["nvcc", *NVCC_FLAGS, *["-D" + d for d in defines], "-c", s, "-o", o]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)
    objs = [os.path.join(obj_dir, s.replace(".cu", ".o")) for s in SOURCES]

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, r

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for cmd, r in ex.map(run, jobs):
            if verbose or r.returncode:
                sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
            if r.returncode:
                raise RuntimeError("nvcc failed: " + cmd[-3])
    if jobs or force or not os.path.exists(lib):
        cmd = ["nvcc", "-shared", "-o", lib, *objs, "-ldl", "-lpthread"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    return lib


# The wait-runs-out test (tests/test_gpu_wait_limit.py) needs a library whose device-side waits give up after a few
# milliseconds and whose decode kernel can be told by the host to skip its loads: a bring-up build kept beside the product.
WAIT_TEST_LIB = os.path.join(LIB_DIR, "libdtattn_waittest.so")
WAIT_TEST_DEFINES = ("DT_BRINGUP", "DT_WAIT_LIMIT_NS=5000000ull")


def build_all(force=False):
    path = build(force=force)
    build(force=force, defines=WAIT_TEST_DEFINES, out=WAIT_TEST_LIB)
    return path


if __name__ == "__main__":
    argv = sys.argv[1:]
    if "--all" in argv:
        print(build_all(force="--force" in argv))
        sys.exit(0)
    defs = [argv[i + 1] for i, a in enumerate(argv[:-1]) if a == "--define"]
    outs = [argv[i + 1] for i, a in enumerate(argv[:-1]) if a == "--out"]
    print(build(force="--force" in argv, verbose="--verbose" in argv, defines=defs, out=outs[0] if outs else None))
