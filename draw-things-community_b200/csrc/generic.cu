// CUDA-core flash attention: the any-shape kernels (D <= 256, fp32/fp16/bf16, additive mask of any row stride,
// causal, grouped KV heads, attention sinks, sliding window, variable-length batches).  They cover what the
// tensor-core kernels do not (fp32 "upcastAttention" I/O, head dims that are not a multiple of 8, masks whose
// rows are not 16-byte aligned) and serve as an independent on-GPU second opinion in the tests.  Semantics follow the reference's
// explicit graph (Libraries/SwiftDiffusion/Sources/Models/UNet.swift:217-265): fp32 scores, softmax over keys, P*V.
//
// Two mappings.  Register-tiled (D a multiple of 4, at least 32 query rows): described at generic_tiled_kernel.
// One warp per query row (everything else): one CTA = 8 query rows of one (batch, head); keys are visited 32 at
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

// ---------------------------------------------------------------------------------------------------------------
// Register-tiled variant for D a multiple of 4 and at least a few dozen query rows: one CTA = 64 query rows x 64 keys
// per step, 256 threads as a 16 x 16 grid.  Thread (ty, tx) owns the scores of rows ty + 16 i and keys tx + 16 j
// (i, j < 4) and, for P.V, the same four rows times the 4-wide column groups tx + 16 r.  Q, K, V and P sit in shared
// memory as fp32 and are read with 16-byte loads along the contracted index, so that one load feeds four
// multiply-adds per row/column pair; the K pitch is an odd number of 16-byte units, which spreads the 16 key rows a
// warp reads over all banks.  A row's 64 probabilities are written and read by the same half-warp.
constexpr int kTM = 64, kTN = 64, kTThreads = 256, kPPitch = kTN + 4;

__host__ __device__ inline int tiled_pitch(int D) {  // multiple of 4, >= D + 4, odd number of float4 per row
  int p = D + 4;
  if (((p >> 2) & 1) == 0) p += 4;
  return p;
}

template <typename T, int R>  // R = 4-wide output column groups per thread (D <= 64 R)
__global__ void __launch_bounds__(kTThreads)
generic_tiled_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, T* __restrict__ o,
                     const T* __restrict__ mask, float* __restrict__ lse,
                     int64_t q_sb, int64_t q_ss, int64_t q_sh, int64_t k_sb, int64_t k_ss, int64_t k_sh,
                     int64_t v_sb, int64_t v_ss, int64_t v_sh, int64_t o_sb, int64_t o_ss, int64_t o_sh,
                     int64_t m_sb, int64_t m_sh, int64_t m_sq,
                     int Sq, int Sk, int Hq, int Hkv, int D, float scale_log2, int is_causal,
                     const T* __restrict__ sinks, int window, const int32_t* __restrict__ off_q,
                     const int32_t* __restrict__ off_k) {
  extern __shared__ __align__(16) float smem[];
  const int P1 = tiled_pitch(D);
  float* Qs = smem;              // [64][P1]
  float* Ks = Qs + kTM * P1;     // [64][P1]
  float* Vs = Ks + kTN * P1;     // [64][D]
  float* Ps = Vs + kTN * D;      // [64][68]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tx = tid & 15, ty = tid >> 4;
  int b = blockIdx.z;
  const int h = blockIdx.y;
  const int kvh = h / (Hq / Hkv);
  const int row0 = blockIdx.x * kTM;
  const int lse_rows = Sq;
  int lse_row0 = 0;
  if (off_q) {
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
  const int off = Sk - Sq;

  {  // Q tile: one warp per row at a time, lanes along the head dim
    const T* qb = q + b * q_sb + h * q_sh;
    for (int r = warp; r < kTM; r += kTThreads / 32) {
      const int rr = row0 + r;
      for (int d = lane; d < D; d += 32) Qs[r * P1 + d] = rr < Sq ? to_float(qb[(int64_t)rr * q_ss + d]) : 0.f;
    }
  }

  int k_end = Sk;
  if (is_causal) {
    const int last = min(row0 + kTM, Sq) - 1;
    k_end = (int)max(0LL, min((long long)Sk, (long long)last + off + 1));
  }
  int k_begin = 0;
  if (window > 0) {
    const long long first = (long long)row0 + off - window + 1;
    k_begin = (int)(max(0LL, min(first, (long long)Sk)) / kTN) * kTN;
  }

  float m[4], l[4], acc[4][R][4];
  long long vis[4], lo[4];
  const T* mrow[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = row0 + ty + 16 * i;
    m[i] = -INFINITY;
    l[i] = 0.f;
    vis[i] = is_causal ? (long long)row + off : (long long)Sk;
    lo[i] = window > 0 ? (long long)row + off - window + 1 : 0;
    mrow[i] = (mask && row < Sq) ? mask + b * m_sb + h * m_sh + (int64_t)row * m_sq : nullptr;
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[i][r][e] = 0.f;
  }

  const T* kb = k + b * k_sb + kvh * k_sh;
  const T* vb = v + b * v_sb + kvh * v_sh;

  for (int j0 = k_begin; j0 < k_end; j0 += kTN) {
    __syncthreads();  // the previous step's reads of K and V are over (and Q is in place)
    for (int r = warp; r < kTN; r += kTThreads / 32) {
      const int j = j0 + r;
      for (int d = lane; d < D; d += 32) {
        float kv = 0.f, vv = 0.f;
        if (j < Sk) {
          kv = to_float(kb[(int64_t)j * k_ss + d]);
          vv = to_float(vb[(int64_t)j * v_ss + d]);
        }
        Ks[r * P1 + d] = kv;
        Vs[r * D + d] = vv;
      }
    }
    __syncthreads();

    // ---- S = Q K^T for this thread's 4 x 4 scores ----
    float s[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
    for (int d = 0; d < D; d += 4) {
      float4 qv[4], kv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) qv[i] = *reinterpret_cast<const float4*>(Qs + (ty + 16 * i) * P1 + d);
#pragma unroll
      for (int j = 0; j < 4; ++j) kv[j] = *reinterpret_cast<const float4*>(Ks + (tx + 16 * j) * P1 + d);
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          s[i][j] = fmaf(qv[i].x, kv[j].x, s[i][j]);
          s[i][j] = fmaf(qv[i].y, kv[j].y, s[i][j]);
          s[i][j] = fmaf(qv[i].z, kv[j].z, s[i][j]);
          s[i][j] = fmaf(qv[i].w, kv[j].w, s[i][j]);
        }
    }

    // ---- online softmax per row (a row's 64 scores live in the 16 lanes of one half-warp) ----
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float tmax = -INFINITY;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int key = j0 + tx + 16 * j;
        float x = s[i][j] * scale_log2;
        if (mrow[i] && key < Sk) x += to_float(mrow[i][key]) * kLog2e;
        if (key >= Sk || (long long)key > vis[i] || (long long)key < lo[i]) x = -INFINITY;
        s[i][j] = x;
        tmax = fmaxf(tmax, x);
      }
#pragma unroll
      for (int sh = 8; sh; sh >>= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, sh));
      const float m_new = fmaxf(m[i], tmax);
      const bool none = m_new == -INFINITY;  // nothing visible in this row so far
      const float alpha = none ? 1.f : exp2f(m[i] - m_new);
      float psum = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float pj = none ? 0.f : exp2f(s[i][j] - m_new);
        psum += pj;
        Ps[(ty + 16 * i) * kPPitch + tx + 16 * j] = pj;
      }
#pragma unroll
      for (int sh = 8; sh; sh >>= 1) psum += __shfl_xor_sync(0xffffffffu, psum, sh);
      l[i] = l[i] * alpha + psum;
      m[i] = m_new;
#pragma unroll
      for (int r = 0; r < R; ++r)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[i][r][e] *= alpha;
    }
    __syncwarp();  // a row's probabilities are written and read by the same half-warp

    // ---- O += P V ----
    for (int kk = 0; kk < kTN; kk += 4) {
      float4 pv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) pv[i] = *reinterpret_cast<const float4*>(Ps + (ty + 16 * i) * kPPitch + kk);
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int col = 4 * (tx + 16 * r);
        if (col < D) {
          const float4 v0 = *reinterpret_cast<const float4*>(Vs + (kk + 0) * D + col);
          const float4 v1 = *reinterpret_cast<const float4*>(Vs + (kk + 1) * D + col);
          const float4 v2 = *reinterpret_cast<const float4*>(Vs + (kk + 2) * D + col);
          const float4 v3 = *reinterpret_cast<const float4*>(Vs + (kk + 3) * D + col);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            acc[i][r][0] = fmaf(pv[i].x, v0.x, fmaf(pv[i].y, v1.x, fmaf(pv[i].z, v2.x, fmaf(pv[i].w, v3.x, acc[i][r][0]))));
            acc[i][r][1] = fmaf(pv[i].x, v0.y, fmaf(pv[i].y, v1.y, fmaf(pv[i].z, v2.y, fmaf(pv[i].w, v3.y, acc[i][r][1]))));
            acc[i][r][2] = fmaf(pv[i].x, v0.z, fmaf(pv[i].y, v1.z, fmaf(pv[i].z, v2.z, fmaf(pv[i].w, v3.z, acc[i][r][2]))));
            acc[i][r][3] = fmaf(pv[i].x, v0.w, fmaf(pv[i].y, v1.w, fmaf(pv[i].z, v2.w, fmaf(pv[i].w, v3.w, acc[i][r][3]))));
          }
        }
      }
    }
    __syncwarp();  // P is rewritten in the next step
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = row0 + ty + 16 * i;
    if (row >= Sq) continue;
    float mi = m[i], li = l[i], alpha = 1.f;
    if (sinks) {  // one more score column without a value row
      const float sl = to_float(sinks[h]) * kLog2e;
      const float m_f = fmaxf(mi, sl);
      alpha = exp2f(mi - m_f);
      li = li * alpha + exp2f(sl - m_f);
      mi = m_f;
    }
    const float inv = li > 0.f ? alpha / li : 0.f;
    T* orow = o + b * o_sb + (int64_t)row * o_ss + h * o_sh;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int col = 4 * (tx + 16 * r);
      if (col < D) {
#pragma unroll
        for (int e = 0; e < 4; ++e) orow[col + e] = from_float<T>(acc[i][r][e] * inv);
      }
    }
    if (lse && tx == 0) lse[((int64_t)b * Hq + h) * lse_rows + lse_row0 + row] = li > 0.f ? mi * kLn2 + logf(li) : -INFINITY;
  }
}

template <typename T, int R>
int launch_tiled(const dt_sdpa_params& p, cudaStream_t stream) {
  const int D = p.D;
  const size_t smem = sizeof(float) * ((size_t)(kTM + kTN) * tiled_pitch(D) + (size_t)kTN * D + (size_t)kTM * kPPitch);
  auto kern = generic_tiled_kernel<T, R>;
  if (smem > 48 * 1024) DT_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const bool varlen = p.seq_offsets_q != nullptr;
  dim3 grid(((varlen ? p.max_seq_q : p.Sq) + kTM - 1) / kTM, p.Hq, varlen ? p.n_seq : p.B);
  kern<<<grid, kTThreads, smem, stream>>>(
      (const T*)p.q.ptr, (const T*)p.k.ptr, (const T*)p.v.ptr, (T*)p.o.ptr, (const T*)p.mask, p.lse,
      p.q.stride_b, p.q.stride_s, p.q.stride_h, p.k.stride_b, p.k.stride_s, p.k.stride_h,
      p.v.stride_b, p.v.stride_s, p.v.stride_h, p.o.stride_b, p.o.stride_s, p.o.stride_h,
      p.mask_stride_b, p.mask_stride_h, p.mask_stride_q, p.Sq, p.Sk, p.Hq, p.Hkv, D, p.scale * kLog2e,
      p.is_causal, (const T*)p.sinks, p.sliding_window, p.seq_offsets_q, p.seq_offsets_k);
  DT_CUDA_TRY(cudaGetLastError());
  return DT_OK;
}

template <typename T>
int launch_t(const dt_sdpa_params& p, cudaStream_t stream) {
  const int D = p.D;
  // enough query rows to fill 64-row tiles (a variable-length batch: by its longest sequence) and 16-byte rows of fp32
  const int rows = p.seq_offsets_q ? p.max_seq_q : p.Sq;
  if (D % 4 == 0 && rows >= 32) {
    if (D <= 64) return launch_tiled<T, 1>(p, stream);
    if (D <= 128) return launch_tiled<T, 2>(p, stream);
    return launch_tiled<T, 4>(p, stream);
  }
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
