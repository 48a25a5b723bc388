// Sparse indexed attention: every query attends, in ONE softmax, to a sliding causal window of "raw" key/value rows
// and to a per-query list of selected rows of a second, "compressed" key/value tensor, plus an attention sink.  The
// reference builds it as SparseIndexedAttention(scale:, isCausal: true, hasAttentionSinks: true, slidingWindow:)
// (Libraries/SwiftLLM/Sources/Models/DeepSeek4.swift:521-545; inputs: queries, raw keys, raw values, compressed keys,
// compressed values, selected rows [queryLength, selectedRowCount], sinks) with one shared KV head for 64 query heads of
// dim 512; the selected rows come from a top-k indexer or list every compressed row a query may see (:1080-1133).  Its
// arithmetic is in the absent back end; the definition restated here: an entry of the list outside [0, compressed rows)
// means "no row", a row listed twice counts twice, the sink is an extra unscaled score without a value row.
//
// CUDA-core kernel, any head dim up to 512, fp16 / bf16 / fp32.  One CTA = one query token x up to 16 query heads that
// share a KV head (the whole point of the layout: a gathered key row is read once for all of them); one warp per head.
// The token's keys -- first its window of raw rows, then its selected rows -- are visited 32 at a time from a
// shared-memory tile (fp32, odd row pitch): lane j owns key j of the tile for Q.K^T, then head dims {lane, lane + 32,
// ...} for P.V.  No tensor cores yet: the decode step of the reference's model (one token, 128 + 512 keys) is a few
// microseconds of work, long prefills are not tuned.
#include "common.cuh"

namespace dt {
namespace {

constexpr int kMaxHeadsPerCta = 16;
constexpr int kTileKeys = 32;
constexpr int kMaxDimChunks = 16;  // head dim <= 512

struct SparseArgs {
  const void* q; void* o;
  const void* k_raw; const void* v_raw; const void* k_comp; const void* v_comp;
  const int32_t* selected;
  const void* sinks;
  float* lse;
  int64_t q_sb, q_ss, q_sh, o_sb, o_ss, o_sh;
  int64_t kr_sb, kr_ss, kr_sh, vr_sb, vr_ss, vr_sh, kc_sb, kc_ss, kc_sh, vc_sb, vc_ss, vc_sh;
  int64_t sel_sb, sel_sq;
  int Sq, Hq, Hkv, D, Sr, Sc, n_sel;
  int heads_per_cta;
  float scale_log2;
  int is_causal, window;
};

template <typename T>
__global__ void __launch_bounds__(kMaxHeadsPerCta * 32)
sparse_indexed_kernel(const SparseArgs a) {
  extern __shared__ float smem[];
  const int D = a.D, Dp = D | 1;
  float* Qs = smem;                               // [heads_per_cta][D]
  float* Ks = Qs + a.heads_per_cta * D;           // [32][Dp]
  float* Vs = Ks + kTileKeys * Dp;                // [32][D]
  __shared__ int s_valid[kTileKeys];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int i = blockIdx.x, b = blockIdx.z;       // query token, batch
  const int G = a.Hq / a.Hkv;
  const int chunks_per_kvh = G / a.heads_per_cta;
  const int kvh = blockIdx.y / chunks_per_kvh;
  const int h = kvh * G + (blockIdx.y - kvh * chunks_per_kvh) * a.heads_per_cta + warp;  // this warp's query head
  const bool head_ok = warp < a.heads_per_cta;

  const T* q = reinterpret_cast<const T*>(a.q);
  for (int idx = threadIdx.x; idx < a.heads_per_cta * D; idx += blockDim.x) {
    const int r = idx / D, d = idx - r * D;
    Qs[idx] = to_float(q[b * a.q_sb + (int64_t)i * a.q_ss + (int64_t)(h - warp + r) * a.q_sh + d]);
  }

  // raw rows this token sees: up to and including its own position (bottom-right aligned), the last `window` of them
  const long long last = a.is_causal ? (long long)i + (a.Sr - a.Sq) : (long long)a.Sr - 1;
  long long first = a.window > 0 ? (long long)i + (a.Sr - a.Sq) - a.window + 1 : 0;
  if (first < 0) first = 0;
  const long long last_c = last < (long long)a.Sr - 1 ? last : (long long)a.Sr - 1;
  const int n_raw = last_c >= first ? (int)(last_c - first + 1) : 0;
  const int n_keys = n_raw + (a.Sc > 0 ? a.n_sel : 0);
  const int32_t* sel = a.selected ? a.selected + b * a.sel_sb + (int64_t)i * a.sel_sq : nullptr;

  float m = -INFINITY, l = 0.f;
  float acc[kMaxDimChunks];
#pragma unroll
  for (int c = 0; c < kMaxDimChunks; ++c) acc[c] = 0.f;
  const int nd = (D + 31) / 32;

  const T* kr = reinterpret_cast<const T*>(a.k_raw) + b * a.kr_sb + kvh * a.kr_sh;
  const T* vr = reinterpret_cast<const T*>(a.v_raw) + b * a.vr_sb + kvh * a.vr_sh;
  const T* kc = reinterpret_cast<const T*>(a.k_comp) + b * a.kc_sb + kvh * a.kc_sh;
  const T* vc = reinterpret_cast<const T*>(a.v_comp) + b * a.vc_sb + kvh * a.vc_sh;

  for (int t0 = 0; t0 < n_keys; t0 += kTileKeys) {
    __syncthreads();
    // which global row each of the tile's 32 keys is: one thread per key decides, then everybody copies
    if (threadIdx.x < kTileKeys) {
      const int vkey = t0 + threadIdx.x;
      int code = -1;  // -1: no key; >= 0: raw row; <= -2: compressed row -(code + 2)
      if (vkey < n_raw) {
        code = (int)(first + vkey);
      } else if (vkey < n_keys) {
        const int idx = sel[vkey - n_raw];
        if (idx >= 0 && idx < a.Sc) code = -(idx + 2);
      }
      s_valid[threadIdx.x] = code;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < kTileKeys * D; idx += blockDim.x) {
      const int r = idx / D, d = idx - r * D;
      const int code = s_valid[r];
      float kv = 0.f, vv = 0.f;
      if (code >= 0) {
        kv = to_float(kr[(int64_t)code * a.kr_ss + d]);
        vv = to_float(vr[(int64_t)code * a.vr_ss + d]);
      } else if (code <= -2) {
        const int row = -(code + 2);
        kv = to_float(kc[(int64_t)row * a.kc_ss + d]);
        vv = to_float(vc[(int64_t)row * a.vc_ss + d]);
      }
      Ks[r * Dp + d] = kv;
      Vs[r * D + d] = vv;
    }
    __syncthreads();
    if (!head_ok) continue;

    float s = 0.f;
    const float* qr = Qs + warp * D;
    const float* krow = Ks + lane * Dp;
    for (int d = 0; d < D; ++d) s = fmaf(qr[d], krow[d], s);
    s *= a.scale_log2;
    if (s_valid[lane] == -1) s = -INFINITY;

    float tmax = s;
#pragma unroll
    for (int off = 16; off; off >>= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, off));
    const float m_new = fmaxf(m, tmax);
    if (m_new == -INFINITY) continue;  // nothing visible so far (warp-uniform)
    const float alpha = exp2f(m - m_new);
    const float p = exp2f(s - m_new);
    float psum = p;
#pragma unroll
    for (int off = 16; off; off >>= 1) psum += __shfl_xor_sync(0xffffffffu, psum, off);
    l = l * alpha + psum;
    m = m_new;
#pragma unroll
    for (int c = 0; c < kMaxDimChunks; ++c) acc[c] *= alpha;
    for (int jj = 0; jj < kTileKeys; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const float* vrow = Vs + jj * D;
#pragma unroll
      for (int c = 0; c < kMaxDimChunks; ++c) {
        const int d = lane + 32 * c;
        if (c < nd && d < D) acc[c] = fmaf(pj, vrow[d], acc[c]);
      }
    }
  }

  if (!head_ok) return;
  if (a.sinks) {  // one more score column without a value row
    const float sl = to_float(reinterpret_cast<const T*>(a.sinks)[h]) * kLog2e;
    const float m_f = fmaxf(m, sl);
    const float alpha = exp2f(m - m_f);
    l = l * alpha + exp2f(sl - m_f);
    m = m_f;
#pragma unroll
    for (int c = 0; c < kMaxDimChunks; ++c) acc[c] *= alpha;
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  T* orow = reinterpret_cast<T*>(a.o) + b * a.o_sb + (int64_t)i * a.o_ss + (int64_t)h * a.o_sh;
#pragma unroll
  for (int c = 0; c < kMaxDimChunks; ++c) {
    const int d = lane + 32 * c;
    if (c < nd && d < D) orow[d] = from_float<T>(acc[c] * inv);
  }
  if (a.lse && lane == 0) a.lse[((int64_t)b * a.Hq + h) * a.Sq + i] = l > 0.f ? m * kLn2 + logf(l) : -INFINITY;
}

template <typename T>
int launch_sparse_t(const dt_sparse_indexed_params& p, cudaStream_t stream) {
  SparseArgs a{};
  a.q = p.q.ptr; a.o = p.o.ptr;
  a.k_raw = p.k_raw.ptr; a.v_raw = p.v_raw.ptr; a.k_comp = p.k_comp.ptr; a.v_comp = p.v_comp.ptr;
  a.selected = p.selected; a.sinks = p.sinks; a.lse = p.lse;
  a.q_sb = p.q.stride_b; a.q_ss = p.q.stride_s; a.q_sh = p.q.stride_h;
  a.o_sb = p.o.stride_b; a.o_ss = p.o.stride_s; a.o_sh = p.o.stride_h;
  a.kr_sb = p.k_raw.stride_b; a.kr_ss = p.k_raw.stride_s; a.kr_sh = p.k_raw.stride_h;
  a.vr_sb = p.v_raw.stride_b; a.vr_ss = p.v_raw.stride_s; a.vr_sh = p.v_raw.stride_h;
  a.kc_sb = p.k_comp.stride_b; a.kc_ss = p.k_comp.stride_s; a.kc_sh = p.k_comp.stride_h;
  a.vc_sb = p.v_comp.stride_b; a.vc_ss = p.v_comp.stride_s; a.vc_sh = p.v_comp.stride_h;
  a.sel_sb = p.selected_stride_b; a.sel_sq = p.selected_stride_q;
  a.Sq = p.Sq; a.Hq = p.Hq; a.Hkv = p.Hkv; a.D = p.D; a.Sr = p.Sr; a.Sc = p.Sc; a.n_sel = p.n_selected;
  const int G = p.Hq / p.Hkv;
  int hpc = G < kMaxHeadsPerCta ? G : kMaxHeadsPerCta;
  while (G % hpc) --hpc;  // the heads of a CTA share one KV head
  a.heads_per_cta = hpc;
  a.scale_log2 = p.scale * kLog2e;
  a.is_causal = p.is_causal;
  a.window = p.sliding_window;
  const size_t smem = sizeof(float) * ((size_t)hpc * p.D + (size_t)kTileKeys * (p.D | 1) + (size_t)kTileKeys * p.D);
  auto kern = sparse_indexed_kernel<T>;
  if (smem > 48 * 1024) DT_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid(p.Sq, p.Hkv * (G / hpc), p.B);
  kern<<<grid, hpc * 32 < 32 ? 32 : hpc * 32, smem, stream>>>(a);
  DT_CUDA_TRY(cudaGetLastError());
  return DT_OK;
}

}  // namespace
}  // namespace dt

using namespace dt;

extern "C" int dt_sparse_indexed_attention(const dt_sparse_indexed_params* p, void* cuda_stream) {
  if (!p) return DT_BAD_ARG;
  if (p->B <= 0 || p->Sq <= 0 || p->Hq <= 0 || p->Hkv <= 0 || p->D <= 0 || p->Sr < 0 || p->Sc < 0 || p->n_selected < 0)
    return DT_BAD_ARG;
  if (p->Hq % p->Hkv) return DT_BAD_ARG;
  if (p->dtype != DT_F16 && p->dtype != DT_BF16 && p->dtype != DT_F32) return DT_BAD_ARG;
  if (!p->q.ptr || !p->o.ptr) return DT_BAD_ARG;
  if (p->Sr > 0 && (!p->k_raw.ptr || !p->v_raw.ptr)) return DT_BAD_ARG;
  if (p->Sc > 0 && p->n_selected > 0 && (!p->k_comp.ptr || !p->v_comp.ptr || !p->selected)) return DT_BAD_ARG;
  if (!(p->scale == p->scale) || p->sliding_window < 0) return DT_BAD_ARG;
  const size_t es = dtype_size(p->dtype);
  const void* ptrs[] = {p->q.ptr, p->o.ptr, p->k_raw.ptr, p->v_raw.ptr, p->k_comp.ptr, p->v_comp.ptr, p->sinks};
  for (const void* x : ptrs)
    if (x && reinterpret_cast<uintptr_t>(x) % es) return DT_BAD_ARG;
  if (p->selected && reinterpret_cast<uintptr_t>(p->selected) % 4) return DT_BAD_ARG;
  if (p->lse && reinterpret_cast<uintptr_t>(p->lse) % 4) return DT_BAD_ARG;
  if (p->D > 32 * kMaxDimChunks) return DT_UNSUPPORTED;
  if (p->Sq > 0x7fffffff / 2 || p->B > 65535 || p->Hq > 65535) return DT_UNSUPPORTED;
  cudaStream_t s = (cudaStream_t)cuda_stream;
  switch (p->dtype) {
    case DT_F32: return launch_sparse_t<float>(*p, s);
    case DT_F16: return launch_sparse_t<__half>(*p, s);
    default: return launch_sparse_t<__nv_bfloat16>(*p, s);
  }
}
