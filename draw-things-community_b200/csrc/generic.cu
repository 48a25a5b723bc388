// CUDA-core flash attention: the any-shape kernel (D <= 256, fp32/fp16/bf16, additive mask, causal,
// grouped KV heads, attention sinks, sliding window, variable-length batches).  It covers what the tensor-core kernels do not (SD1.5's D = 40/80/160, fp32
// "upcastAttention" I/O, masked text encoders) and serves as an independent on-GPU second opinion in
// the tests.  Semantics follow the reference's explicit graph
// (Libraries/SwiftDiffusion/Sources/Models/UNet.swift:217-265): fp32 scores, softmax over keys, P*V.
//
// Mapping: one CTA = 8 query rows of one (batch, head); one warp per query row.  Keys are visited 32 at
// a time from a shared-memory tile (fp32, odd row pitch so that lane j reading key row j is conflict
// free); lane j owns key j of the tile for Q.K^T, then owns head dims {lane, lane+32, ...} for P.V.
#include "common.cuh"

namespace dt {
namespace {

constexpr int kRows = 8;    // query rows (= warps) per CTA
constexpr int kKeys = 32;   // keys per tile

template <typename T>
__global__ void __launch_bounds__(kRows * 32)
generic_sdpa_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, T* __restrict__ o,
                    const T* __restrict__ mask, float* __restrict__ lse,
                    int64_t q_sb, int64_t q_ss, int64_t q_sh, int64_t k_sb, int64_t k_ss, int64_t k_sh,
                    int64_t v_sb, int64_t v_ss, int64_t v_sh, int64_t o_sb, int64_t o_ss, int64_t o_sh,
                    int64_t m_sb, int64_t m_sh, int64_t m_sq,
                    int Sq, int Sk, int Hq, int Hkv, int D, float scale_log2, int is_causal,
                    const T* __restrict__ sinks, int window, const int32_t* __restrict__ off_q,
                    const int32_t* __restrict__ off_k) {
  extern __shared__ float smem[];
  const int Dp = D | 1;
  float* Qs = smem;                    // [kRows][D]
  float* Ks = Qs + kRows * D;          // [kKeys][Dp]
  float* Vs = Ks + kKeys * Dp;         // [kKeys][D]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int b = blockIdx.z;
  const int h = blockIdx.y;
  const int kvh = h / (Hq / Hkv);
  const int row0 = blockIdx.x * kRows;
  const int lse_rows = Sq;  // rows per head of the lse output (packed rows for variable-length batches)
  int lse_row0 = 0;
  if (off_q) {
    // variable-length batch: blockIdx.z is the sequence; its rows are a slice of the packed tensors
    const int q0 = off_q[b], k0 = off_k[b];
    Sq = off_q[b + 1] - q0;
    Sk = off_k[b + 1] - k0;
    if (row0 >= Sq) return;  // whole CTA, before any barrier
    q += (int64_t)q0 * q_ss;
    o += (int64_t)q0 * o_ss;
    k += (int64_t)k0 * k_ss;
    v += (int64_t)k0 * v_ss;
    lse_row0 = q0;
    b = 0;
  }
  const int row = row0 + warp;
  const bool row_ok = row < Sq;

  for (int idx = threadIdx.x; idx < kRows * D; idx += blockDim.x) {
    int r = idx / D, d = idx - r * D;
    int rr = row0 + r;
    Qs[idx] = rr < Sq ? to_float(q[b * q_sb + (int64_t)rr * q_ss + h * q_sh + d]) : 0.f;
  }

  // keys this CTA needs: with a causal mask the last row of the CTA bounds it
  int k_end = Sk;
  if (is_causal) {
    int last = min(row0 + kRows, Sq) - 1;
    long long lim = (long long)last + (Sk - Sq) + 1;
    k_end = (int)max(0LL, min((long long)Sk, lim));
  }
  const long long vis = is_causal ? (long long)row + (Sk - Sq) : (long long)Sk;  // keys j <= vis visible
  // sliding window: keys below `lo` are hidden; the CTA starts at the tile holding its first row's bound
  const long long lo = window > 0 ? (long long)row + (Sk - Sq) - window + 1 : 0;
  int k_begin = 0;
  if (window > 0) {
    const long long first = (long long)row0 + (Sk - Sq) - window + 1;
    k_begin = (int)(max(0LL, min(first, (long long)Sk)) / kKeys) * kKeys;
  }

  float m = -INFINITY, l = 0.f;
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  const int nd = (D + 31) / 32;

  const T* kb = k + b * k_sb + kvh * k_sh;
  const T* vb = v + b * v_sb + kvh * v_sh;
  const T* mrow = (mask && row_ok) ? mask + b * m_sb + h * m_sh + (int64_t)row * m_sq : nullptr;

  for (int j0 = k_begin; j0 < k_end; j0 += kKeys) {
    __syncthreads();
    for (int idx = threadIdx.x; idx < kKeys * D; idx += blockDim.x) {
      int r = idx / D, d = idx - r * D;
      int j = j0 + r;
      float kv = 0.f, vv = 0.f;
      if (j < Sk) {
        kv = to_float(kb[(int64_t)j * k_ss + d]);
        vv = to_float(vb[(int64_t)j * v_ss + d]);
      }
      Ks[r * Dp + d] = kv;
      Vs[r * D + d] = vv;
    }
    __syncthreads();
    if (!row_ok) continue;

    const int j = j0 + lane;
    float s = 0.f;
    const float* qr = Qs + warp * D;
    const float* kr = Ks + lane * Dp;
    for (int d = 0; d < D; ++d) s = fmaf(qr[d], kr[d], s);
    s *= scale_log2;
    if (mrow && j < Sk) s += to_float(mrow[j]) * kLog2e;
    if (j >= Sk || (is_causal && (long long)j > vis) || (long long)j < lo) s = -INFINITY;

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
    for (int i = 0; i < 8; ++i) acc[i] *= alpha;
    for (int jj = 0; jj < kKeys; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const float* vr = Vs + jj * D;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        int d = lane + 32 * i;
        if (i < nd && d < D) acc[i] = fmaf(pj, vr[d], acc[i]);
      }
    }
  }

  if (row_ok) {
    if (sinks) {  // one more score column without a value row
      const float sl = to_float(sinks[h]) * kLog2e;
      const float m_f = fmaxf(m, sl);
      const float alpha = exp2f(m - m_f);
      l = l * alpha + exp2f(sl - m_f);
      m = m_f;
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] *= alpha;
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
    T* orow = o + b * o_sb + (int64_t)row * o_ss + h * o_sh;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      int d = lane + 32 * i;
      if (i < nd && d < D) orow[d] = from_float<T>(acc[i] * inv);
    }
    if (lse && lane == 0) lse[((int64_t)b * Hq + h) * lse_rows + lse_row0 + row] = l > 0.f ? m * kLn2 + logf(l) : -INFINITY;
  }
}

template <typename T>
int launch_t(const dt_sdpa_params& p, cudaStream_t stream) {
  const int D = p.D;
  const size_t smem = sizeof(float) * ((size_t)kRows * D + (size_t)kKeys * (D | 1) + (size_t)kKeys * D);
  auto kern = generic_sdpa_kernel<T>;
  if (smem > 48 * 1024) DT_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const bool varlen = p.seq_offsets_q != nullptr;
  dim3 grid(((varlen ? p.max_seq_q : p.Sq) + kRows - 1) / kRows, p.Hq, varlen ? p.n_seq : p.B);
  kern<<<grid, kRows * 32, smem, stream>>>(
      (const T*)p.q.ptr, (const T*)p.k.ptr, (const T*)p.v.ptr, (T*)p.o.ptr, (const T*)p.mask, p.lse,
      p.q.stride_b, p.q.stride_s, p.q.stride_h, p.k.stride_b, p.k.stride_s, p.k.stride_h,
      p.v.stride_b, p.v.stride_s, p.v.stride_h, p.o.stride_b, p.o.stride_s, p.o.stride_h,
      p.mask_stride_b, p.mask_stride_h, p.mask_stride_q, p.Sq, p.Sk, p.Hq, p.Hkv, D, p.scale * kLog2e,
      p.is_causal, (const T*)p.sinks, p.sliding_window, p.seq_offsets_q, p.seq_offsets_k);
  DT_CUDA_TRY(cudaGetLastError());
  return DT_OK;
}

}  // namespace

int launch_generic(const dt_sdpa_params& p, cudaStream_t stream) {
  if (p.D > 256) return DT_UNSUPPORTED;
  if (p.Hq > 65535 || p.B > 65535 || p.n_seq > 65535) return DT_UNSUPPORTED;
  switch (p.dtype) {
    case DT_F32: return launch_t<float>(p, stream);
    case DT_F16: return launch_t<__half>(p, stream);
    case DT_BF16: return launch_t<__nv_bfloat16>(p, stream);
  }
  return DT_BAD_ARG;
}

}  // namespace dt
