"""The C++ host mirror of the operator (host/ScaledDotProductAttention.hpp) compiles against the C ABI and
rejects misuse the way the header documents (no GPU: only construction and validation run)."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "draw-things-community_b200")

SRC = r'''
#include <cstdio>
#include "host/ScaledDotProductAttention.hpp"
int main() {
  using namespace dt;
  int fails = 0;
  ScaledDotProductAttention op(0.125f, /*isCausal=*/true, /*hasAttentionMask=*/false, kFloat16);
  ScaledDotProductAttention fused(1.f, false, false, kNone, /*multiHeadOutputProjectionFused=*/true);
  alignas(16) static char qb[1 << 12];
  TensorView fq = TensorView::contiguous(qb, 1, 1, 4, 64, DT_F16);
  try { fused(fq, fq, fq, fq, nullptr, 0, nullptr); ++fails; }  // the Dense parameters were never set
  catch (const Error& e) { if (e.status != DT_BAD_ARG) ++fails; }
  fused.withOutputProjection(qb, nullptr, 64);
  if (fused.projectedWorkspaceSize(fq, fq, fq, fq) < 4 * 64 * 2) ++fails;  // room for the attention output
  try { ScaledDotProductAttention bad(1.f, false, false, kInt8 | kFloat16); ++fails; }
  catch (const Error& e) { if (e.status != DT_UNSUPPORTED) ++fails; }
  alignas(16) static char buf[1 << 16];
  TensorView q = TensorView::contiguous(buf, 1, 1, 32, 128, DT_F16);
  TensorView k = TensorView::contiguous(buf, 1, 8192, 8, 128, DT_F16);
  size_t ws = op.workspaceSize(q, k, k, q);
  if (ws == 0) ++fails;                       // the split-KV decode path needs scratch
  TensorView k3 = TensorView::contiguous(buf, 1, 8192, 5, 128, DT_F16);
  try { op.workspaceSize(q, k3, k3, q); ++fails; } catch (const Error& e) { if (e.status != DT_BAD_ARG) ++fails; }
  TensorView r = k.rows(16, 100);
  if (r.S != 100 || r.ptr != buf + 16 * 8 * 128 * 2) ++fails;
  ScaledDotProductAttention masked(1.f, false, true);
  try { masked(q, k, k, q, nullptr, 0, nullptr); ++fails; } catch (const Error& e) { if (e.status != DT_BAD_ARG) ++fails; }
  // free functions for the steps either side of the operator: argument checks happen before any launch
  TensorView cache = TensorView::contiguous(buf, 1, 64, 8, 128, DT_F16);
  TensorView many = TensorView::contiguous(buf, 1, 17, 8, 128, DT_F16);
  try { decodeStep(q, cache, cache, many, many, nullptr, 0, 0, 0.1f, 10, q, nullptr, 0, nullptr); ++fails; }
  catch (const Error& e) { if (e.status != DT_UNSUPPORTED) ++fails; }  // more new rows than one 16-key unit
  TensorView odd = TensorView::contiguous(buf, 1, 4, 2, 60, DT_F16);
  try { qkPrologue(odd, odd, PrologueSpec(), nullptr, nullptr, nullptr, nullptr); ++fails; }
  catch (const Error& e) { if (e.status != DT_UNSUPPORTED) ++fails; }
  std::printf("fails=%d ws=%zu\n", fails, ws);
  return fails;
}
'''


def test_cpp_mirror_compiles_and_validates(tmp_path, dtattn):
    src = tmp_path / "host_test.cpp"
    src.write_text(SRC)
    exe = tmp_path / "host_test"
    lib_dir = os.path.join(PKG, "lib")
    subprocess.check_call(["g++", "-std=c++17", "-O1", "-I", PKG, str(src), "-o", str(exe), "-L", lib_dir, "-ldtattn",
                           f"-Wl,-rpath,{lib_dir}"])
    r = subprocess.run([str(exe)], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "fails=0" in r.stdout


def test_header_is_plain_c(tmp_path):
    """include/dtattn.h must be usable from C (the boundary is a C ABI): compile a C translation unit that fills every
    parameter struct and references every entry point."""
    import re
    header = os.path.join(ROOT, "include", "dtattn.h")
    text = re.sub(r"/\*.*?\*/", "", open(header).read(), flags=re.S)
    names = sorted(set(re.findall(r"\b(dt_[a-z0-9_]+)\s*\(", text)))
    src = tmp_path / "abi.c"
    body = ["#include \"dtattn.h\"", "#include <string.h>", "int probe(void) {",
            "  dt_sdpa_params p; dt_decode_step_params s; dt_qk_prologue_params q; dt_out_proj o;",
            "  memset(&p, 0, sizeof p); memset(&s, 0, sizeof s); memset(&q, 0, sizeof q); memset(&o, 0, sizeof o);",
            "  p.sliding_window = 4; s.T_new = 1; q.post_scale = 1.0f; o.C = 8;",
            "  typedef void (*fn_t)(void);",
            "  fn_t fns[] = {" + ", ".join(f"(fn_t){n}" for n in names) + "};",
            "  return (int)(sizeof fns / sizeof fns[0]) + p.sliding_window + s.T_new + o.C + (int)q.post_scale;", "}"]
    src.write_text("\n".join(body) + "\n")
    r = subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-pedantic", "-I", os.path.join(ROOT, "include"), "-c", str(src), "-o",
                        str(tmp_path / "abi.o")], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    assert len(names) >= 25
