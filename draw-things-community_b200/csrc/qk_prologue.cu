// The step immediately before the attention node: Q/K normalisation, rotary embedding and pre-scale in one
// pass over HBM.  The reference builds it from separate graph nodes, each reading and writing the whole tensor:
//   Flux   (Libraries/SwiftDiffusion/Sources/Models/Flux1.swift:164-188): RMSNorm(epsilon 1e-6, axis [3]) on the
//          per-head rows of K and Q, concat of text and image tokens, Functional.cmul with the rotary table;
//   Wan    (Libraries/SwiftDiffusion/Sources/Models/Wan.swift:86-98): RMSNorm(axis [2]) over all h*k channels of a
//          token, reshape to heads, cmul, then Q and K each times D^(-1/4);
//   Qwen   (Libraries/SwiftLLM/Sources/Models/Qwen3_5.swift:164-182): RMSNorm(axis [3]) then cmul.
// Here one launch reads each element once and writes it once (HBM bound: 2 * bytes(Q) + 2 * bytes(K) plus the
// table).  Every node's output is rounded to the tensors' 16-bit type before the next step uses it, as a graph of
// 16-bit tensors does, and cmul avoids fused multiply-add so its result does not depend on contraction.  The inverse
// RMS uses the hardware reciprocal square root (2 ulp of fp32), far below the 16-bit rounding that follows.
// The output may be a strided view, e.g. a row-offset view of the joint text+image buffer, which fuses the concat.
#include <stdlib.h>

#include "common.cuh"

namespace dt {
namespace {

struct PrologueTensor {
  const void* x;
  void* y;
  const void* weight;  // [D] (per head row) or [H*D] (per token), nullptr = no normalisation
  const void* rot;     // interleaved (cos, sin), nullptr = no rotation
  int64_t x_sb, x_ss, x_sh, y_sb, y_ss, y_sh, r_sb, r_ss, r_sh;
  int B, S, H, D;
  int per_token;  // normalise over all H*D channels of a token instead of each head's D
  float eps, post_scale;
};

struct PrologueArgs {
  PrologueTensor t[2];
  int n;
};

template <typename T>
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if constexpr (std::is_same<T, __half>::value) {
      const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      f[2 * i] = a.x;
      f[2 * i + 1] = a.y;
    } else {
      const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
      f[2 * i] = a.x;
      f[2 * i + 1] = a.y;
    }
  }
}

// hardware reciprocal square root (2 ulp); the argument is mean(x^2) + eps, never subnormal
__device__ __forceinline__ float rsqrt_fast(float x) {
  float y;
  asm("rsqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <typename T>
__device__ __forceinline__ float2 unpack2(uint32_t w) {
  if constexpr (std::is_same<T, __half>::value) return __half22float2(*reinterpret_cast<const __half2*>(&w));
  else return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w));
}

// Two fp32 values -> one packed pair, round to nearest even.  One conversion instruction serves both values:
// the conversion unit is the scarce resource of this kernel, so every stage rounds pairwise and hands the packed
// pair to the next stage (unpacking is plain integer work for bf16).
template <typename T>
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  if constexpr (std::is_same<T, __half>::value) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
  } else {
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
  }
}

// normalise (inv already known), rotate, scale: eight consecutive channels of one row, each stage rounded to T
template <typename T>
__device__ __forceinline__ uint4 finish8(const uint4& xin, float post_scale, float inv, bool has_w, const uint4& wv,
                                         bool has_r, const uint4& rv) {
  uint32_t w[4] = {xin.x, xin.y, xin.z, xin.w};
  if (has_w) {
    const uint32_t g[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 v = unpack2<T>(w[i]), gw = unpack2<T>(g[i]);
      w[i] = pack2<T>(__fmul_rn(__fmul_rn(v.x, inv), gw.x), __fmul_rn(__fmul_rn(v.y, inv), gw.y));
    }
  }
  if (has_r) {
    const uint32_t r[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 v = unpack2<T>(w[i]), cs = unpack2<T>(r[i]);
      w[i] = pack2<T>(__fsub_rn(__fmul_rn(v.x, cs.x), __fmul_rn(v.y, cs.y)), __fadd_rn(__fmul_rn(v.x, cs.y), __fmul_rn(v.y, cs.x)));
    }
  }
  if (post_scale != 1.f) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 v = unpack2<T>(w[i]);
      w[i] = pack2<T>(__fmul_rn(v.x, post_scale), __fmul_rn(v.y, post_scale));
    }
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// ---- per-head rows: LANES lanes (8 channels each) per row, 32 / LANES rows per warp ----------------------------
// Persistent warps sweep the rows; the loads of the next row are issued before the current row is worked on, so
// every thread keeps one row piece and its table piece in flight while it computes.
template <typename T, int LANES>
__global__ void __launch_bounds__(256, 4) qk_prologue_rows_kernel(const PrologueArgs a) {
  const PrologueTensor& t = a.t[blockIdx.y];
  const int lane = threadIdx.x & 31, warp_in_cta = threadIdx.x >> 5;
  constexpr int kRowsPerWarp = 32 / LANES;
  const int sub = lane / LANES, l = lane % LANES;
  const uint32_t n_rows = (uint32_t)t.B * t.S * t.H;
  const uint32_t stride = gridDim.x * (blockDim.x >> 5) * kRowsPerWarp;  // rows covered by one sweep of the grid
  const bool lane_on = l * 8 < t.D;
  const T* x = reinterpret_cast<const T*>(t.x);
  T* y = reinterpret_cast<T*>(t.y);
  const T* rot = reinterpret_cast<const T*>(t.rot);
  const bool has_w = t.weight != nullptr, has_r = rot != nullptr;
  uint4 wv = make_uint4(0u, 0u, 0u, 0u);
  if (has_w && lane_on) wv = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(t.weight) + l * 8);
  const float post_scale = t.post_scale, eps = t.eps, inv_d = 1.f / (float)t.D;

  uint4 v_next = make_uint4(0u, 0u, 0u, 0u), r_next = v_next;
  int64_t y_next = 0;
  bool on_next = false;
  // (batch, token, head) of this lane's row, advanced by `stride` rows per sweep without dividing again
  const uint32_t H = (uint32_t)t.H, S = (uint32_t)t.S;
  const uint32_t dh = stride % H, ds = (stride / H) % S, db = stride / H / S;
  uint32_t r0 = (blockIdx.x * (blockDim.x >> 5) + warp_in_cta) * kRowsPerWarp;
  uint32_t h = (r0 + sub) % H, s = ((r0 + sub) / H) % S, b = (r0 + sub) / H / S;
  auto fetch = [&]() {  // loads for row r0 + sub, whose coordinates are (b, s, h)
    on_next = lane_on && r0 + sub < n_rows;
    if (on_next) {
      v_next = *reinterpret_cast<const uint4*>(x + b * t.x_sb + (int64_t)s * t.x_ss + (int64_t)h * t.x_sh + l * 8);
      if (has_r) r_next = *reinterpret_cast<const uint4*>(rot + b * t.r_sb + (int64_t)s * t.r_ss + (int64_t)h * t.r_sh + l * 8);
      y_next = b * t.y_sb + (int64_t)s * t.y_ss + (int64_t)h * t.y_sh + l * 8;
    } else {
      v_next = make_uint4(0u, 0u, 0u, 0u);
    }
  };
  auto advance = [&]() {
    r0 += stride;
    h += dh;
    const uint32_t c0 = h >= H ? 1u : 0u;
    h -= c0 * H;
    s += ds + c0;
    const uint32_t c1 = s >= S ? 1u : 0u;
    s -= c1 * S;
    b += db + c1;
  };
  if (r0 < n_rows) fetch();
  while (r0 < n_rows) {  // warp-uniform
    const uint4 v = v_next, rv = r_next;
    const int64_t yo = y_next;
    const bool on = on_next;
    advance();
    if (r0 < n_rows) fetch();
    float inv = 1.f;
    if (has_w) {
      float f[8];
      unpack8<T>(v, f);
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) ss = fmaf(f[i], f[i], ss);
#pragma unroll
      for (int o = LANES / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      inv = rsqrt_fast(fmaf(ss, inv_d, eps));
    }
    if (on) *reinterpret_cast<uint4*>(y + yo) = finish8<T>(v, post_scale, inv, has_w, wv, has_r, rv);
  }
}

// ---- per-token normalisation over all H*D channels: a group of G threads per token, 256 / G tokens per CTA ------
constexpr int kTokThreads = 256;
constexpr int kTokVecs = 8;  // 16-byte pieces held per thread at most: H*D <= 256 * 8 * 8 = 16384 channels

template <typename T, int VECS>
__global__ void __launch_bounds__(kTokThreads) qk_prologue_tokens_kernel(const PrologueArgs a, const int G) {
  const PrologueTensor& t = a.t[blockIdx.y];
  __shared__ float red[kTokThreads / 32];
  const int vecs_per_head = t.D / 8, n_vec = t.H * vecs_per_head;
  const int tokens_per_cta = kTokThreads / G;
  const int group = threadIdx.x / G, tig = threadIdx.x % G;
  const int warps_per_group = G / 32;
  const int64_t n_tok = (int64_t)t.B * t.S;
  const int64_t sweep = (int64_t)gridDim.x * tokens_per_cta;
  const T* x = reinterpret_cast<const T*>(t.x);
  T* y = reinterpret_cast<T*>(t.y);
  const T* w = reinterpret_cast<const T*>(t.weight);
  const T* rot = reinterpret_cast<const T*>(t.rot);
  const float n_f = (float)(t.H * t.D);
  // this thread's pieces sit at fixed (head, channel) positions of every token
  int xo[VECS], yo[VECS], ro[VECS];  // element offsets inside one token (the host checks that they fit 32 bits)
  int wo[VECS];  // into weight[H*D]
  bool piece_on[VECS];
#pragma unroll
  for (int i = 0; i < VECS; ++i) {
    const int vi = tig + i * G;
    piece_on[i] = vi < n_vec;
    const int h = piece_on[i] ? vi / vecs_per_head : 0, d = piece_on[i] ? (vi - h * vecs_per_head) * 8 : 0;
    xo[i] = (int)(h * t.x_sh) + d;
    yo[i] = (int)(h * t.y_sh) + d;
    ro[i] = (int)(h * t.r_sh) + d;
    wo[i] = h * t.D + d;
  }
  // 32-bit token arithmetic (the host refuses tensors with 2^31 rows or more); one division per token
  uint4 v_next[VECS];
  int64_t yb_next = 0, rb_next = 0;
  bool on_next = false;
  auto fetch = [&](uint32_t tok) {
    on_next = tok < (uint32_t)n_tok;
    const uint32_t b = tok / (uint32_t)t.S, s = tok - b * (uint32_t)t.S;
    const T* xb = x + b * t.x_sb + (int64_t)s * t.x_ss;
    yb_next = b * t.y_sb + (int64_t)s * t.y_ss;
    rb_next = b * t.r_sb + (int64_t)s * t.r_ss;
#pragma unroll
    for (int i = 0; i < VECS; ++i) {
      v_next[i] = make_uint4(0u, 0u, 0u, 0u);
      if (on_next && piece_on[i]) v_next[i] = *reinterpret_cast<const uint4*>(xb + xo[i]);
    }
  };
  int64_t base = (int64_t)blockIdx.x * tokens_per_cta;
  if (base < n_tok) fetch((uint32_t)(base + group));
  while (base < n_tok) {  // uniform over the CTA
    const bool tok_on = on_next;
    uint4 v[VECS], rv[VECS];
    const T* rb = rot ? rot + rb_next : nullptr;
    T* yb = y + yb_next;
#pragma unroll
    for (int i = 0; i < VECS; ++i) {
      v[i] = v_next[i];
      rv[i] = make_uint4(0u, 0u, 0u, 0u);
      if (rb && tok_on && piece_on[i]) rv[i] = *reinterpret_cast<const uint4*>(rb + ro[i]);
    }
    base += sweep;
    if (base < n_tok) fetch((uint32_t)(base + group));
    float inv[VECS];
#pragma unroll
    for (int i = 0; i < VECS; ++i) inv[i] = 1.f;
    if (w) {  // uniform over the CTA
      float sq[VECS];
#pragma unroll
      for (int i = 0; i < VECS; ++i) {
        float f[8];
        unpack8<T>(v[i], f);
        sq[i] = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) sq[i] = fmaf(f[e], f[e], sq[i]);
      }
      {
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < VECS; ++i) ss += sq[i];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (warps_per_group > 1) {
          if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
          __syncthreads();
          ss = 0.f;
          for (int i = 0; i < warps_per_group; ++i) ss += red[group * warps_per_group + i];
          __syncthreads();  // red is reused by the next sweep
        }
        const float inv_tok = rsqrt_fast(fmaf(ss, 1.f / n_f, t.eps));
#pragma unroll
        for (int i = 0; i < VECS; ++i) inv[i] = inv_tok;
      }
    }
    if (tok_on) {
#pragma unroll
      for (int i = 0; i < VECS; ++i) {
        if (piece_on[i]) {
          uint4 wv = make_uint4(0u, 0u, 0u, 0u);
          if (w) wv = *reinterpret_cast<const uint4*>(w + wo[i]);
          *reinterpret_cast<uint4*>(yb + yo[i]) = finish8<T>(v[i], t.post_scale, inv[i], w != nullptr, wv, rb != nullptr, rv[i]);
        }
      }
    }
  }
}

int sm_count_prologue() {
  int dev = 0, n = 0;
  cudaGetDevice(&dev);
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
  return n;
}

int check_one(const dt_qk_prologue_params* p) {
  if (!p->x.ptr || !p->y.ptr) return DT_BAD_ARG;
  if (p->B <= 0 || p->S <= 0 || p->H <= 0 || p->D <= 0) return DT_BAD_ARG;
  if (p->dtype != DT_F16 && p->dtype != DT_BF16) return DT_UNSUPPORTED;
  if (p->D % 8 || p->D > 256) return DT_UNSUPPORTED;
  auto ok = [](const dt_tensor4& t) {
    return reinterpret_cast<uintptr_t>(t.ptr) % 16 == 0 && t.stride_b % 8 == 0 && t.stride_s % 8 == 0 &&
           t.stride_h % 8 == 0;
  };
  if (!ok(p->x) || !ok(p->y)) return DT_UNSUPPORTED;
  if (p->norm_weight && reinterpret_cast<uintptr_t>(p->norm_weight) % 16) return DT_UNSUPPORTED;
  if (p->rotary && (reinterpret_cast<uintptr_t>(p->rotary) % 16 || p->rotary_stride_b % 8 || p->rotary_stride_s % 8 ||
                    p->rotary_stride_h % 8))
    return DT_UNSUPPORTED;
  if (p->norm_per_token && (int64_t)p->H * p->D > (int64_t)kTokThreads * kTokVecs * 8) return DT_UNSUPPORTED;
  if ((int64_t)p->B * p->S * p->H >= (int64_t)1 << 31) return DT_UNSUPPORTED;  // 32-bit row index
  const int64_t lim = (int64_t)1 << 30;  // 32-bit element offsets inside one token
  if (p->H * p->x.stride_h >= lim || p->H * p->y.stride_h >= lim || p->H * p->rotary_stride_h >= lim) return DT_UNSUPPORTED;
  if (p->x.stride_h < 0 || p->y.stride_h < 0 || p->rotary_stride_h < 0) return DT_UNSUPPORTED;
  return DT_OK;
}

PrologueTensor to_arg(const dt_qk_prologue_params* p) {
  PrologueTensor t{};
  t.x = p->x.ptr; t.y = p->y.ptr; t.weight = p->norm_weight; t.rot = p->rotary;
  t.x_sb = p->x.stride_b; t.x_ss = p->x.stride_s; t.x_sh = p->x.stride_h;
  t.y_sb = p->y.stride_b; t.y_ss = p->y.stride_s; t.y_sh = p->y.stride_h;
  t.r_sb = p->rotary_stride_b; t.r_ss = p->rotary_stride_s; t.r_sh = p->rotary_stride_h;
  t.B = p->B; t.S = p->S; t.H = p->H; t.D = p->D;
  t.per_token = p->norm_per_token;
  t.eps = p->eps;
  t.post_scale = p->post_scale == 0.f ? 1.f : p->post_scale;
  return t;
}

template <typename T>
int launch_rows(const PrologueArgs& a, int D, int64_t max_rows, cudaStream_t stream) {
  const int lanes = D <= 64 ? 8 : (D <= 128 ? 16 : 32);
  const int rows_per_cta = 8 * (32 / lanes);
  int64_t ctas = (max_rows + rows_per_cta - 1) / rows_per_cta;
  const int64_t cap = (int64_t)sm_count_prologue() * 4;  // persistent: four CTAs per SM sweep the rows
  if (ctas > cap) ctas = cap;
  dim3 grid((unsigned)ctas, a.n);
  if (lanes == 8) qk_prologue_rows_kernel<T, 8><<<grid, 256, 0, stream>>>(a);
  else if (lanes == 16) qk_prologue_rows_kernel<T, 16><<<grid, 256, 0, stream>>>(a);
  else qk_prologue_rows_kernel<T, 32><<<grid, 256, 0, stream>>>(a);
  DT_CUDA_TRY(cudaGetLastError());
  return DT_OK;
}

}  // namespace
}  // namespace dt

extern "C" int dt_qk_prologue(const dt_qk_prologue_params* q, const dt_qk_prologue_params* k, void* cuda_stream) {
  using namespace dt;
  if (!q) return DT_BAD_ARG;
  int st = check_one(q);
  if (st != DT_OK) return st;
  if (k) {
    st = check_one(k);
    if (st != DT_OK) return st;
    // one launch serves both tensors: same element type, same kind of normalisation, same lane mapping
    if (k->dtype != q->dtype || k->norm_per_token != q->norm_per_token) return DT_BAD_ARG;
    const int lq = q->D <= 64 ? 8 : (q->D <= 128 ? 16 : 32), lk = k->D <= 64 ? 8 : (k->D <= 128 ? 16 : 32);
    if (lq != lk) return DT_BAD_ARG;
  }
  PrologueArgs a{};
  a.t[0] = to_arg(q);
  a.n = 1;
  if (k) {
    a.t[1] = to_arg(k);
    a.n = 2;
  }
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(cuda_stream);
  if (q->norm_per_token) {
    int n_vec = q->H * (q->D / 8);
    if (k && k->H * (k->D / 8) > n_vec) n_vec = k->H * (k->D / 8);
    int64_t toks = (int64_t)q->B * q->S;
    if (k && (int64_t)k->B * k->S > toks) toks = (int64_t)k->B * k->S;
    // threads per token: the smallest power of two >= 32 that leaves at most 4 pieces per thread (8 at 256 threads)
    int G = 32;
    while (G < kTokThreads && n_vec > G * 4) G *= 2;
    const int vecs = (n_vec + G - 1) / G;
    const int tokens_per_cta = kTokThreads / G;
    const int64_t ctas = (toks + tokens_per_cta - 1) / tokens_per_cta;
    const bool f16 = q->dtype == DT_F16;
    const int sms = sm_count_prologue();
#define DT_TOK_LAUNCH(V)                                                                                          \
  do {                                                                                                            \
    auto kern = f16 ? qk_prologue_tokens_kernel<__half, V> : qk_prologue_tokens_kernel<__nv_bfloat16, V>;         \
    int per_sm = 0;                                                                                               \
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kTokThreads, 0) != cudaSuccess || per_sm < 1) \
      per_sm = 1;                                                                                                 \
    const int64_t cap = (int64_t)sms * per_sm; /* persistent: resident CTAs sweep the tokens */                   \
    dim3 grid((unsigned)(ctas < cap ? ctas : cap), a.n);                                                          \
    kern<<<grid, kTokThreads, 0, stream>>>(a, G);                                                     \
  } while (0)
    if (vecs <= 1) DT_TOK_LAUNCH(1);
    else if (vecs <= 2) DT_TOK_LAUNCH(2);
    else if (vecs <= 3) DT_TOK_LAUNCH(3);
    else if (vecs <= 4) DT_TOK_LAUNCH(4);
    else DT_TOK_LAUNCH(8);
#undef DT_TOK_LAUNCH
    DT_CUDA_TRY(cudaGetLastError());
    return DT_OK;
  }
  int64_t rows = (int64_t)q->B * q->S * q->H;
  if (k && (int64_t)k->B * k->S * k->H > rows) rows = (int64_t)k->B * k->S * k->H;
  return q->dtype == DT_F16 ? launch_rows<__half>(a, q->D, rows, stream) : launch_rows<__nv_bfloat16>(a, q->D, rows, stream);
}
