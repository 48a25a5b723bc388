"""Build oracle/_build/libsdpa_oracle.so from oracle/sdpa_oracle.c (test infrastructure, never shipped).

The reference's own CPU attention cannot be compiled here (its arithmetic is in un-vendored
dependencies and there is no Swift/Bazel toolchain), so there is no oracle/_ref build: this restatement
is the only CPU implementation available.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "sdpa_oracle.c")
OUT_DIR = os.path.join(HERE, "_build")
OUT = os.path.join(OUT_DIR, "libsdpa_oracle.so")


def build(force=False):
    os.makedirs(OUT_DIR, exist_ok=True)
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= os.path.getmtime(SRC):
        return OUT
    # -march=x86-64-v3 (AVX2+FMA) rather than native: the library is built in one container and
    # timed on another machine's host cores.
    cmd = ["gcc", "-O3", "-march=x86-64-v3", "-fopenmp-simd", "-shared", "-fPIC", "-pthread",
           "-o", OUT, SRC, "-lm"]
    subprocess.check_call(cmd)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
