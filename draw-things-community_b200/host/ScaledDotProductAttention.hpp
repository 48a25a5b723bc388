// C++ mirror of the reference's operator surface, header-only, above the C ABI (include/dtattn.h).
//
// The reference builds attention as a graph node of its Swift NNC module:
//   ScaledDotProductAttention(scale:, isCausal:, hasAttentionMask:, flags:, multiHeadOutputProjectionFused:, name:)
//   op(queries, keys, values[, mask])
// (Libraries/SwiftDiffusion/Sources/Models/UNet.swift:139-155, Flux1.swift:224-232, Wan.swift:95-131,
//  Libraries/SwiftLLM/Sources/Models/Qwen3_5.swift:193-196).  No Swift toolchain exists in this build
// environment, so the host side is written in C++ with the same names and argument meaning; the Swift
// facade a maintainer would add is in host/ScaledDotProductAttention.swift.
//
// Error behaviour: the reference traps (precondition / fatalError) on misuse.  Here misuse throws
// dt::Error carrying the dt_status; nothing falls back to another implementation.
#pragma once

#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <string>

#include "../../include/dtattn.h"

namespace dt {

struct Error : std::runtime_error {
  int status;
  Error(int st, const std::string& what) : std::runtime_error(what + ": " + dt_status_string(st)), status(st) {}
};

// Functional.GEMMFlag as passed at the call sites ([.Float16], [], [.Float32], [.Int8, .Float16]).
enum GEMMFlag : unsigned { kNone = 0, kFloat16 = 1, kFloat32 = 2, kInt8 = 4 };

// A [B, S, H, D] tensor view in device memory (element strides, D contiguous): what Model.IO carries
// for this operator.
struct TensorView {
  void* ptr = nullptr;
  int B = 0, S = 0, H = 0, D = 0;
  int64_t stride_b = 0, stride_s = 0, stride_h = 0;
  dt_dtype dtype = DT_F16;
  static TensorView contiguous(void* p, int B, int S, int H, int D, dt_dtype t) {
    TensorView v;
    v.ptr = p; v.B = B; v.S = S; v.H = H; v.D = D; v.dtype = t;
    v.stride_h = D; v.stride_s = (int64_t)H * D; v.stride_b = (int64_t)S * H * D;
    return v;
  }
  // rows [offset, offset + count) of the sequence axis, the reshaped(offset:strides:) views of
  // Flux1.swift:236-243
  TensorView rows(int offset, int count) const {
    TensorView v = *this;
    const size_t es = dtype == DT_F32 ? 4 : 2;
    v.ptr = static_cast<char*>(ptr) + (size_t)offset * stride_s * es;
    v.S = count;
    return v;
  }
  dt_tensor4 abi() const { return dt_tensor4{ptr, stride_b, stride_s, stride_h}; }
};

class ScaledDotProductAttention {
 public:
  ScaledDotProductAttention(float scale, bool isCausal = false, bool hasAttentionMask = false,
                            unsigned flags = kNone, bool multiHeadOutputProjectionFused = false,
                            std::string name = "")
      : scale_(scale), causal_(isCausal), has_mask_(hasAttentionMask), flags_(flags), name_(std::move(name)),
        fused_projection_(multiHeadOutputProjectionFused) {
    if (flags & kInt8) throw Error(DT_UNSUPPORTED, "quantised attention is only selected on Metal in the reference");
  }

  // Bytes of scratch operator() needs for these shapes (the graph compiles once per shape in the
  // reference, UNetProtocol.swift:2954-2965; query this at the same point).
  size_t workspaceSize(const TensorView& q, const TensorView& k, const TensorView& v, const TensorView& o) const {
    dt_sdpa_params p = params(q, k, v, o, nullptr);
    size_t n = 0;
    int st = dt_sdpa_workspace_size(&p, &n);
    if (st != DT_OK) throw Error(st, "dt_sdpa_workspace_size");
    return n;
  }

  // Operator variants of the reference's initialiser: hasAttentionSinks + slidingWindow
  // (SwiftLLM/Sources/Models/DeepSeek4.swift:482-493) and isVariableLength + maxSequenceLength
  // (SwiftLLM/Sources/Models/Qwen3_5VL.swift:428-437).  The inputs they add are set here before the call.
  ScaledDotProductAttention& withSinks(const void* sinks_hq) { sinks_ = sinks_hq; return *this; }
  ScaledDotProductAttention& withSlidingWindow(int window) { window_ = window; return *this; }
  ScaledDotProductAttention& withSequenceOffsets(const int32_t* q_offsets, const int32_t* kv_offsets, int n_seq,
                                                 int max_q, int max_kv) {
    off_q_ = q_offsets; off_k_ = kv_offsets; n_seq_ = n_seq; max_q_ = max_q; max_k_ = max_kv;
    return *this;
  }

  // multiHeadOutputProjectionFused (UNet.swift:122-130): the operator owns the unify-heads Dense.  Its
  // parameters ([C, Hq*D] weight, [C] bias or null, device memory) are set here, as the reference copies them
  // into the model at UNet.swift:865-874; out of operator() is then [B, Sq, 1, C].
  ScaledDotProductAttention& withOutputProjection(const void* weight, const void* bias, int C) {
    proj_weight_ = weight; proj_bias_ = bias; proj_c_ = C;
    return *this;
  }
  size_t projectedWorkspaceSize(const TensorView& q, const TensorView& k, const TensorView& v, const TensorView& out) const {
    dt_sdpa_params p = params(q, k, v, q, nullptr);
    dt_out_proj pr = projection(out);
    size_t n = 0;
    int st = dt_sdpa_projected_workspace_size(&p, &pr, &n);
    if (st != DT_OK) throw Error(st, "dt_sdpa_projected_workspace_size");
    return n;
  }

  // op(queries, keys, values[, mask]) -> out, enqueued on `stream`.
  void operator()(const TensorView& q, const TensorView& k, const TensorView& v, const TensorView& out,
                  void* workspace, size_t workspace_bytes, void* stream, const TensorView* mask = nullptr) const {
    if (has_mask_ != (mask != nullptr)) throw Error(DT_BAD_ARG, "hasAttentionMask and the inputs disagree");
    if (fused_projection_) {
      if (!proj_weight_) throw Error(DT_BAD_ARG, "multiHeadOutputProjectionFused: withOutputProjection() first");
      dt_sdpa_params pp = params(q, k, v, q, mask);
      dt_out_proj pr = projection(out);
      int stp = dt_sdpa_forward_projected(&pp, &pr, workspace, workspace_bytes, stream);
      if (stp != DT_OK) throw Error(stp, "dt_sdpa_forward_projected(" + name_ + ")");
      return;
    }
    dt_sdpa_params p = params(q, k, v, out, mask);
    int st = dt_sdpa_forward(&p, workspace, workspace_bytes, stream);
    if (st != DT_OK) throw Error(st, "dt_sdpa_forward(" + name_ + ")");
  }

 private:
  dt_out_proj projection(const TensorView& out) const {
    dt_out_proj pr{};
    pr.weight = proj_weight_; pr.bias = proj_bias_; pr.C = proj_c_;
    pr.out = out.abi();
    return pr;
  }
  dt_sdpa_params params(const TensorView& q, const TensorView& k, const TensorView& v, const TensorView& o,
                        const TensorView* mask) const {
    if (q.dtype != k.dtype || q.dtype != v.dtype || q.dtype != o.dtype) throw Error(DT_BAD_ARG, "dtype mismatch");
    if (q.B != k.B || k.S != v.S || k.H != v.H || q.D != k.D || q.D != v.D) throw Error(DT_BAD_ARG, "shape mismatch");
    dt_sdpa_params p{};
    p.B = q.B; p.Sq = q.S; p.Sk = k.S; p.Hq = q.H; p.Hkv = k.H; p.D = q.D;
    p.dtype = q.dtype;
    p.scale = scale_;
    p.is_causal = causal_ ? 1 : 0;
    p.flags = (flags_ & kFloat16) ? DT_FLAG_FP16_ACCUM_HINT : 0;
    p.q = q.abi(); p.k = k.abi(); p.v = v.abi(); p.o = o.abi();
    if (mask) {  // [B|1, H|1, Sq, Sk] carried as a TensorView with B, S=H(mask heads), H=Sq, D=Sk
      p.mask = mask->ptr;
      p.mask_stride_b = mask->B > 1 ? mask->stride_b : 0;
      p.mask_stride_h = mask->S > 1 ? mask->stride_s : 0;
      p.mask_stride_q = mask->stride_h;
    }
    p.sinks = sinks_;
    p.sliding_window = window_;
    p.seq_offsets_q = off_q_; p.seq_offsets_k = off_k_;
    p.n_seq = n_seq_; p.max_seq_q = max_q_; p.max_seq_k = max_k_;
    return p;
  }
  float scale_;
  const void* proj_weight_ = nullptr;
  const void* proj_bias_ = nullptr;
  int proj_c_ = 0;
  const void* sinks_ = nullptr;
  int window_ = 0;
  const int32_t* off_q_ = nullptr;
  const int32_t* off_k_ = nullptr;
  int n_seq_ = 0, max_q_ = 0, max_k_ = 0;
  bool causal_, has_mask_;
  unsigned flags_;
  std::string name_;
  bool fused_projection_ = false;
};

// SparseIndexedAttention(scale:, isCausal:, hasAttentionSinks:, slidingWindow:) with the reference's input order
// (SwiftLLM/Sources/Models/DeepSeek4.swift:521-545): op(queries, rawKeys, rawValues, compressedKeys, compressedValues,
// selectedRows, sinks) -> out.  selectedRows: int32 [queryLength, selectedRowCount] (one list per query, shared by the
// batch); entries outside [0, compressed rows) name no row.
class SparseIndexedAttention {
 public:
  SparseIndexedAttention(float scale, bool isCausal = true, bool hasAttentionSinks = true, int slidingWindow = 0,
                         std::string name = "")
      : scale_(scale), causal_(isCausal), has_sinks_(hasAttentionSinks), window_(slidingWindow), name_(std::move(name)) {}
  void operator()(const TensorView& q, const TensorView& rawK, const TensorView& rawV, const TensorView* compK,
                  const TensorView* compV, const int32_t* selectedRows, int selectedRowCount, const void* sinks,
                  const TensorView& out, void* stream) const {
    if (has_sinks_ != (sinks != nullptr)) throw Error(DT_BAD_ARG, "hasAttentionSinks and the inputs disagree");
    dt_sparse_indexed_params p{};
    p.B = q.B; p.Sq = q.S; p.Hq = q.H; p.Hkv = rawK.H; p.D = q.D;
    p.Sr = rawK.S; p.Sc = compK ? compK->S : 0; p.n_selected = selectedRowCount;
    p.dtype = q.dtype; p.scale = scale_; p.is_causal = causal_ ? 1 : 0; p.sliding_window = window_;
    p.q = q.abi(); p.o = out.abi(); p.k_raw = rawK.abi(); p.v_raw = rawV.abi();
    if (compK && compV) { p.k_comp = compK->abi(); p.v_comp = compV->abi(); }
    p.selected = selectedRows; p.selected_stride_b = 0; p.selected_stride_q = selectedRowCount;
    p.sinks = sinks;
    int st = dt_sparse_indexed_attention(&p, stream);
    if (st != DT_OK) throw Error(st, "dt_sparse_indexed_attention(" + name_ + ")");
  }

 private:
  float scale_;
  bool causal_, has_sinks_;
  int window_;
  std::string name_;
};

// ---- the steps either side of the operator, as free functions over the same views --------------------------

// One KV-cache step (Qwen3_5.swift:164-196): optional qNorm / kNorm, rotary cmul on the last q.S queries and the
// new keys, append of the new rows at row `cachedLength` of the caches, causal attention over cachedLength + T_new
// rows.  kCache / vCache are views of the whole cache (capacity rows).
inline void decodeStep(const TensorView& q, const TensorView& kCache, const TensorView& vCache, const TensorView& kNew,
                       const TensorView& vNew, const void* rotary, int64_t rotaryStrideB, int64_t rotaryStrideS,
                       float scale, int cachedLength, const TensorView& out, void* workspace, size_t workspaceBytes,
                       void* stream, const void* qNormWeight = nullptr, const void* kNormWeight = nullptr,
                       float normEps = 1e-6f, unsigned flags = 0) {
  dt_decode_step_params s{};
  dt_sdpa_params& p = s.attn;
  p.B = q.B; p.Sq = q.S; p.Sk = cachedLength + kNew.S; p.Hq = q.H; p.Hkv = kCache.H; p.D = q.D;
  p.dtype = q.dtype; p.scale = scale; p.is_causal = 1; p.flags = flags;
  p.q = q.abi(); p.k = kCache.abi(); p.v = vCache.abi(); p.o = out.abi();
  s.k_new = kNew.abi(); s.v_new = vNew.abi(); s.T_new = kNew.S;
  s.rotary = rotary; s.rotary_stride_b = rotaryStrideB; s.rotary_stride_s = rotaryStrideS;
  s.q_norm_weight = qNormWeight; s.k_norm_weight = kNormWeight; s.norm_eps = normEps;
  int st = dt_sdpa_decode_step(&s, workspace, workspaceBytes, stream);
  if (st != DT_OK) throw Error(st, "dt_sdpa_decode_step");
}

// RMSNorm + rotary + pre-scale of one tensor or of queries and keys together (Flux1.swift:164-188, Wan.swift:86-98).
struct PrologueSpec {
  const void* normWeight = nullptr;  // [D], or [H*D] with normPerToken
  bool normPerToken = false;
  float eps = 1e-6f;
  const void* rotary = nullptr;      // [B|1, S, H|1, D], interleaved (cos, sin); a broadcast axis has stride 0
  int64_t rotaryStrideB = 0, rotaryStrideS = 0, rotaryStrideH = 0;
  float postScale = 1.f;
};
inline dt_qk_prologue_params prologueParams(const TensorView& x, const TensorView& y, const PrologueSpec& spec) {
  dt_qk_prologue_params p{};
  p.B = x.B; p.S = x.S; p.H = x.H; p.D = x.D; p.dtype = x.dtype;
  p.x = x.abi(); p.y = y.abi();
  p.norm_weight = spec.normWeight; p.norm_per_token = spec.normPerToken ? 1 : 0; p.eps = spec.eps;
  p.rotary = spec.rotary; p.rotary_stride_b = spec.rotaryStrideB; p.rotary_stride_s = spec.rotaryStrideS;
  p.rotary_stride_h = spec.rotaryStrideH; p.post_scale = spec.postScale;
  return p;
}
inline void qkPrologue(const TensorView& q, const TensorView& qOut, const PrologueSpec& qSpec, const TensorView* k,
                       const TensorView* kOut, const PrologueSpec* kSpec, void* stream) {
  dt_qk_prologue_params pq = prologueParams(q, qOut, qSpec);
  dt_qk_prologue_params pk{};
  if (k) pk = prologueParams(*k, *kOut, kSpec ? *kSpec : qSpec);
  int st = dt_qk_prologue(&pq, k ? &pk : nullptr, stream);
  if (st != DT_OK) throw Error(st, "dt_qk_prologue");
}

}  // namespace dt
