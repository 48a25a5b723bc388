// Sparse indexed attention: every query attends, in ONE softmax, to a sliding causal window of "raw" key/value rows
// and to a per-query list of selected rows of a second, "compressed" key/value tensor, plus an attention sink.  The
// reference builds it as SparseIndexedAttention(scale:, isCausal: true, hasAttentionSinks: true, slidingWindow:)
// (Libraries/SwiftLLM/Sources/Models/DeepSeek4.swift:521-545; inputs: queries, raw keys, raw values, compressed keys,
// compressed values, selected rows [queryLength, selectedRowCount], sinks) with one shared KV head for 64 query heads of
// dim 512; the selected rows come from a top-k indexer or list every compressed row a query may see (:1080-1133).  Its
// arithmetic is in the absent back end; the definition restated here: an entry of the list outside [0, compressed rows)
// means "no row", a row listed twice counts twice, the sink is an extra unscaled score without a value row.
//
// Two kernels: a tensor-core one (described at sparse_mma_kernel) for 16-bit tensors with a head dim that is a multiple
// of 64 and 16-byte aligned rows, and a CUDA-core one for everything else (any head dim up to 512, fp16 / bf16 / fp32):
// one CTA = one query token x up to 16 query heads that share a KV head (a gathered key row is read once for all of
// them); one warp per head.  The token's keys -- first its window of raw rows, then its selected rows -- are visited
// 32 at a time from a shared-memory tile (fp32, odd row pitch): lane j owns key j of the tile for Q.K^T, then head
// dims {lane, lane + 32, ...} for P.V.
#include "sm100_ptx.cuh"

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

// ---------------------------------------------------------------------------------------------------------------
// Tensor-core variant (mma.sync m16n8k16, fp32 accumulate) for 16-bit tensors whose head dim is a multiple of 64 and
// whose rows are 16-byte aligned: the reference's shape (64 heads over one KV head, dim 512) is a [heads x keys x dim]
// matrix product per token, and the decode step needs the token's keys spread over several CTAs.
//
// One CTA = one token x 16 query heads of one KV head x one share of the token's keys; 4 warps.  Keys are gathered 32 at
// a time into shared memory (16-byte pieces, 16-bit, row pitch D + 8 so that ldmatrix rows fall on distinct banks);
// 64 at a time where two buffers of that size fit (keys and values in one tensor): a warp then takes 16 keys.
// S = Q K^T: warp w takes keys 8 w .. 8 w + 7 of the tile over the whole head dim (one n-tile, D / 16 k-steps; Q and K
// fragments by ldmatrix).  The row maxima of the four warps meet in shared memory, every warp then holds the tile's
// maximum, exponentiates its 8 keys and writes them as 16-bit P into a [16 x 32] exchange tile.  O += P V: warp w owns
// head dims [w D / 4, (w + 1) D / 4) (D / 32 n-tiles of fp32 accumulators), P by ldmatrix, V by ldmatrix.trans.
// With more than one share per token the CTAs of a token form a thread-block cluster: each leaves (m, l, O) in its
// shared memory and CTA r of the cluster combines and stores columns [r D / n, (r + 1) D / n) of the 16 rows from all
// of them through distributed shared memory (ordinary ld.shared::cluster loads).
constexpr int kMmaMaxSplit = 8;
constexpr int kMmaMaxGroups = 4;  // head groups of 16 per CTA

struct SparseMmaExtra {
  int n_split;   // CTAs (= cluster size) per token and head group; > 1 only with one head group per CTA
  int same_kv;   // values are the keys (one gathered tile serves both)
  int gpc;       // head groups of 16 per CTA (4 warps each); they share the gathered tiles
};

template <typename T, int TK>  // TK keys per tile: 32, or 64 (every Q fragment then feeds two score MMAs)
__global__ void __launch_bounds__(128 * kMmaMaxGroups)
sparse_mma_kernel(const SparseArgs a, const SparseMmaExtra x) {
  constexpr bool kBf16 = !std::is_same<T, __half>::value;
  constexpr int NT = TK / 32;        // n-tiles of 8 keys per warp in Q K^T
  constexpr int PP = TK + 8;         // row pitch of the P exchange tile
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int D = a.D, P = D + 8;  // row pitch in elements
  const int gpc = x.gpc, nthreads = 128 * gpc;
  uint16_t* Qs = reinterpret_cast<uint16_t*>(smem_raw);                 // [gpc * 16][P]
  uint16_t* Kb = Qs + gpc * 16 * P;                                      // [2][32][P]
  uint16_t* Vb = x.same_kv ? Kb : Kb + 2 * TK * P;                 // [2][32][P]
  uint16_t* Pex = Kb + (x.same_kv ? 2 : 4) * TK * P;               // [gpc][16][40]
  float* mxs = reinterpret_cast<float*>(Pex + gpc * 16 * PP);            // [gpc][4][16] row maxima, one set per warp
  float* ls = mxs + gpc * 64;                                            // [gpc][4][16] row sums
  int* codes = reinterpret_cast<int*>(ls + gpc * 64);                    // [2][32]
  // cluster path (one head group per CTA): after the key loop the first K buffer holds this CTA's partial result
  float* Opart = reinterpret_cast<float*>(Kb);                           // [16][D] fp32
  float* mpart = reinterpret_cast<float*>(codes + 2 * TK);               // [16]
  float* lpart = mpart + 16;                                             // [16]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tg = lane & 3;
  const int gi = warp >> 2, w = warp & 3;  // head group within the CTA, warp within the group
  const int i = blockIdx.x / x.n_split, split = blockIdx.x % x.n_split, b = blockIdx.z;
  const int G = a.Hq / a.Hkv;
  const int ng = (G + 15) / 16, gy = (ng + gpc - 1) / gpc;
  const int kvh = blockIdx.y / gy;
  const int hg0 = (blockIdx.y - kvh * gy) * gpc;         // first head group of this CTA
  const int hg = hg0 + gi;
  const int h0 = kvh * G + hg * 16;
  const int nh = hg < ng ? min(16, G - hg * 16) : 0;     // query heads of this warp's group (rows beyond them hold zeros)
  const int chunks = D / 8;                              // 16-byte pieces per row

  {
    const T* q = reinterpret_cast<const T*>(a.q) + b * a.q_sb + (int64_t)i * a.q_ss;
    for (int c = tid; c < gpc * 16 * chunks; c += nthreads) {
      const int r = c / chunks, ch = c - r * chunks;
      const int head = kvh * G + hg0 * 16 + r;  // rows of all groups of the CTA are consecutive heads
      // asynchronous like the key rows below (the first wait covers both); rows beyond the heads are zero-filled
      const bool on = hg0 * 16 + r < G;
      ptx::cp_async_16(ptx::smem_u32(Qs + r * P + ch * 8), on ? (const void*)(q + (int64_t)head * a.q_sh + ch * 8) : (const void*)q,
                       on ? 16 : 0);
    }
    ptx::cp_async_commit();
  }

  const long long last = a.is_causal ? (long long)i + (a.Sr - a.Sq) : (long long)a.Sr - 1;
  long long first = a.window > 0 ? (long long)i + (a.Sr - a.Sq) - a.window + 1 : 0;
  if (first < 0) first = 0;
  const long long last_c = last < (long long)a.Sr - 1 ? last : (long long)a.Sr - 1;
  const int n_raw = last_c >= first ? (int)(last_c - first + 1) : 0;
  const int n_keys = n_raw + (a.Sc > 0 ? a.n_sel : 0);
  const int32_t* sel = a.selected ? a.selected + b * a.sel_sb + (int64_t)i * a.sel_sq : nullptr;
  const int n_tiles = (n_keys + TK - 1) / TK;
  const int per = (n_tiles + x.n_split - 1) / x.n_split;
  const int t_begin = split * per, t_end = min(n_tiles, t_begin + per);

  const T* kr = reinterpret_cast<const T*>(a.k_raw) + b * a.kr_sb + kvh * a.kr_sh;
  const T* vr = reinterpret_cast<const T*>(a.v_raw) + b * a.vr_sb + kvh * a.vr_sh;
  const T* kc = reinterpret_cast<const T*>(a.k_comp) + b * a.kc_sb + kvh * a.kc_sh;
  const T* vc = reinterpret_cast<const T*>(a.v_comp) + b * a.vc_sb + kvh * a.vc_sh;

  const int g_r0 = tid / chunks, g_ch0 = tid - g_r0 * chunks, g_dr = nthreads / chunks, g_dch = nthreads - g_dr * chunks;
  // which row each of a tile's 32 keys is: -1 no key, >= 0 raw row, <= -2 compressed row -(code + 2)
  auto set_codes = [&](int tile, int buf) {
    if (tid < TK) {
      const int vkey = tile * TK + tid;
      int code = -1;
      if (vkey < n_raw) {
        code = (int)(first + vkey);
      } else if (vkey < n_keys) {
        const int idx = sel[vkey - n_raw];
        if (idx >= 0 && idx < a.Sc) code = -(idx + 2);
      }
      codes[buf * TK + tid] = code;
    }
  };
  // the tile's rows into buffer `buf`: asynchronous 16-byte copies, zero fill where there is no key
  auto gather = [&](int buf) {
    const uint32_t kdst = ptx::smem_u32(Kb + buf * TK * P), vdst = ptx::smem_u32(Vb + buf * TK * P);
    int r = g_r0, ch = g_ch0;  // (row, 16-byte piece) of this thread's first copy; they advance without dividing
    for (int c = tid; c < TK * chunks; c += nthreads, r += g_dr, ch += g_dch) {
      if (ch >= chunks) {
        ch -= chunks;
        ++r;
      }
      const int code = codes[buf * TK + r];
      const T* ksrc = reinterpret_cast<const T*>(a.q);  // any valid address when nothing is copied (the raw tensors may be absent)
      const T* vsrc = ksrc;
      int nbytes = 0;
      if (code >= 0) {
        ksrc = kr + (int64_t)code * a.kr_ss + ch * 8;
        vsrc = vr + (int64_t)code * a.vr_ss + ch * 8;
        nbytes = 16;
      } else if (code <= -2) {
        const int row = -(code + 2);
        ksrc = kc + (int64_t)row * a.kc_ss + ch * 8;
        vsrc = vc + (int64_t)row * a.vc_ss + ch * 8;
        nbytes = 16;
      }
      const uint32_t off = (uint32_t)((r * P + ch * 8) * 2);
      ptx::cp_async_16(kdst + off, ksrc, nbytes);
      if (!x.same_kv) ptx::cp_async_16(vdst + off, vsrc, nbytes);
    }
    ptx::cp_async_commit();
  };

  const int Dq = D / 4, ntl = Dq / 8;  // this warp's head dims and its n-tiles of 8 (D = 512: 16)
  const int dim0 = w * Dq;
  float acc[16][4];
#pragma unroll
  for (int nt = 0; nt < 16; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[nt][e] = 0.f;
  float m_row[2] = {-INFINITY, -INFINITY};  // rows g and g + 8: the same in the four warps of a group
  float l_lane[2] = {0.f, 0.f};             // this lane's share of the row sums (its two keys of every tile)

  const uint32_t qs_addr = ptx::smem_u32(Qs) + (uint32_t)(((gi * 16 + (lane & 15)) * P + (lane >> 4) * 8) * 2);
  const uint32_t ks_off = (uint32_t)(((8 * NT * w + (lane & 7)) * P + (lane >> 3) * 8) * 2);
  const uint32_t vs_off = (uint32_t)((((lane & 7) + ((lane >> 3) & 1) * 8) * P + dim0 + (lane >> 4) * 8) * 2);
  uint16_t* pex = Pex + gi * 16 * PP;
  const uint32_t pex_addr = ptx::smem_u32(pex) + (uint32_t)(((lane & 15) * PP + (lane >> 4) * 8) * 2);
  float* mx_g = mxs + gi * 64;

  if (t_begin < t_end) {
    set_codes(t_begin, 0);
    __syncthreads();
    gather(0);
  }
  for (int tile = t_begin; tile < t_end; ++tile) {
    const int cur = (tile - t_begin) & 1;
    const bool more = tile + 1 < t_end;
    if (more) set_codes(tile + 1, cur ^ 1);
    ptx::cp_async_wait<0>();
    __syncthreads();  // this tile has landed for everybody, the previous tile is used up, the next codes are visible
    if (more) gather(cur ^ 1);  // travels while this tile is worked on
    const uint32_t ks_addr = ptx::smem_u32(Kb + cur * TK * P) + ks_off;
    const uint32_t vs_addr = ptx::smem_u32(Vb + cur * TK * P) + vs_off;
    const int* code_cur = codes + cur * TK;

    // ---- scores of this warp's 8 NT keys, the group's 16 heads, the whole head dim ----
    float sc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) sc[j][e] = 0.f;
    for (int ks = 0; ks < D / 16; ks += 2) {
      uint32_t a0[4], a1[4];
      ptx::ldmatrix_x4(a0[0], a0[1], a0[2], a0[3], qs_addr + (uint32_t)(ks * 32));
      ptx::ldmatrix_x4(a1[0], a1[1], a1[2], a1[3], qs_addr + (uint32_t)(ks * 32 + 32));
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        uint32_t b0, b1, b2, b3;
        ptx::ldmatrix_x4(b0, b1, b2, b3, ks_addr + (uint32_t)(ks * 32 + j * 8 * P * 2));
        ptx::mma_m16n8k16<kBf16>(sc[j], a0, b0, b1);
        ptx::mma_m16n8k16<kBf16>(sc[j], a1, b2, b3);
      }
    }
    // this lane's scores: rows g (s[j][0], s[j][1]) and g + 8 (s[j][2], s[j][3]) of keys 8 NT w + 8 j + 2 tg + {0, 1}
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      const int key = 8 * NT * w + 8 * j + 2 * tg;
      const bool v0 = code_cur[key] != -1, v1 = code_cur[key + 1] != -1;
      sc[j][0] = v0 ? sc[j][0] * a.scale_log2 : -INFINITY;
      sc[j][1] = v1 ? sc[j][1] * a.scale_log2 : -INFINITY;
      sc[j][2] = v0 ? sc[j][2] * a.scale_log2 : -INFINITY;
      sc[j][3] = v1 ? sc[j][3] * a.scale_log2 : -INFINITY;
      mx0 = fmaxf(mx0, fmaxf(sc[j][0], sc[j][1]));
      mx1 = fmaxf(mx1, fmaxf(sc[j][2], sc[j][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    if (tg == 0) {
      mx_g[w * 16 + g] = mx0;
      mx_g[w * 16 + g + 8] = mx1;
    }
    __syncthreads();
    const float mt0 = fmaxf(fmaxf(mx_g[g], mx_g[16 + g]), fmaxf(mx_g[32 + g], mx_g[48 + g]));
    const float mt1 = fmaxf(fmaxf(mx_g[g + 8], mx_g[24 + g]), fmaxf(mx_g[40 + g], mx_g[56 + g]));
    const float mn0 = fmaxf(m_row[0], mt0), mn1 = fmaxf(m_row[1], mt1);
    const float al0 = mn0 == -INFINITY ? 1.f : exp2f(m_row[0] - mn0), al1 = mn1 == -INFINITY ? 1.f : exp2f(m_row[1] - mn1);
    float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      const float p00 = mn0 == -INFINITY ? 0.f : exp2f(sc[j][0] - mn0), p01 = mn0 == -INFINITY ? 0.f : exp2f(sc[j][1] - mn0);
      const float p10 = mn1 == -INFINITY ? 0.f : exp2f(sc[j][2] - mn1), p11 = mn1 == -INFINITY ? 0.f : exp2f(sc[j][3] - mn1);
      sum0 += p00 + p01;
      sum1 += p10 + p11;
      uint32_t w0, w1;
      if constexpr (kBf16) {
        w0 = ptx::cvt_pack_bf16(p00, p01);
        w1 = ptx::cvt_pack_bf16(p10, p11);
      } else {
        w0 = ptx::cvt_pack_f16(p00, p01);
        w1 = ptx::cvt_pack_f16(p10, p11);
      }
      const int key = 8 * NT * w + 8 * j + 2 * tg;
      *reinterpret_cast<uint32_t*>(pex + g * PP + key) = w0;
      *reinterpret_cast<uint32_t*>(pex + (g + 8) * PP + key) = w1;
    }
    l_lane[0] = l_lane[0] * al0 + sum0;
    l_lane[1] = l_lane[1] * al1 + sum1;
    m_row[0] = mn0;
    m_row[1] = mn1;
    __syncthreads();

    // ---- O += P V over this warp's head dims ----
    uint32_t pa[TK / 16][4];
#pragma unroll
    for (int k2 = 0; k2 < TK / 16; ++k2) ptx::ldmatrix_x4(pa[k2][0], pa[k2][1], pa[k2][2], pa[k2][3], pex_addr + (uint32_t)(k2 * 32));
    if (__any_sync(0xffffffffu, al0 != 1.f || al1 != 1.f)) {  // some row's maximum moved (rare once it has settled)
#pragma unroll
      for (int nt = 0; nt < 16; ++nt) {
        if (nt < ntl) {
          acc[nt][0] *= al0; acc[nt][1] *= al0; acc[nt][2] *= al1; acc[nt][3] *= al1;
        }
      }
    }
#pragma unroll
    for (int nt = 0; nt < 16; nt += 2) {
      if (nt < ntl) {
#pragma unroll
        for (int k2 = 0; k2 < TK / 16; ++k2) {
          uint32_t b0, b1, b2, b3;
          ptx::ldmatrix_x4_trans(b0, b1, b2, b3, vs_addr + (uint32_t)(nt * 16 + k2 * 16 * P * 2));
          ptx::mma_m16n8k16<kBf16>(acc[nt], pa[k2], b0, b1);
          ptx::mma_m16n8k16<kBf16>(acc[nt + 1], pa[k2], b2, b3);
        }
      }
    }
  }

  // ---- row sums over the four warps' keys ----
  float l0 = l_lane[0], l1 = l_lane[1];
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  float* ls_g = ls + gi * 64;
  ptx::cp_async_wait<0>();  // (a CTA without tiles still has its Q copies in flight)
  __syncthreads();  // the last tile is used up: the K buffers may be overwritten below
  if (tg == 0) {
    ls_g[w * 16 + g] = l0;
    ls_g[w * 16 + g + 8] = l1;
  }
  __syncthreads();
  l0 = (ls_g[g] + ls_g[16 + g]) + (ls_g[32 + g] + ls_g[48 + g]);
  l1 = (ls_g[g + 8] + ls_g[24 + g]) + (ls_g[40 + g] + ls_g[56 + g]);

  const T* sinks = reinterpret_cast<const T*>(a.sinks);
  T* obase = reinterpret_cast<T*>(a.o) + b * a.o_sb + (int64_t)i * a.o_ss;
  if (x.n_split == 1) {
    float inv[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = g + 8 * r;
      float m = m_row[r], l = r ? l1 : l0, alpha = 1.f;
      if (sinks && row < nh) {  // one more score column without a value row
        const float sl = to_float(sinks[h0 + row]) * kLog2e;
        const float m_f = fmaxf(m, sl);
        alpha = exp2f(m - m_f);
        l = l * alpha + exp2f(sl - m_f);
        m = m_f;
      }
      inv[r] = l > 0.f ? alpha / l : 0.f;
      if (a.lse && w == 0 && tg == 0 && row < nh)
        a.lse[((int64_t)b * a.Hq + h0 + row) * a.Sq + i] = l > 0.f ? m * kLn2 + logf(l) : -INFINITY;
    }
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) {
      if (nt < ntl) {
        const int col = dim0 + nt * 8 + 2 * tg;
        uint32_t w0, w1;
        if constexpr (kBf16) {
          w0 = ptx::cvt_pack_bf16(acc[nt][0] * inv[0], acc[nt][1] * inv[0]);
          w1 = ptx::cvt_pack_bf16(acc[nt][2] * inv[1], acc[nt][3] * inv[1]);
        } else {
          w0 = ptx::cvt_pack_f16(acc[nt][0] * inv[0], acc[nt][1] * inv[0]);
          w1 = ptx::cvt_pack_f16(acc[nt][2] * inv[1], acc[nt][3] * inv[1]);
        }
        if (g < nh) *reinterpret_cast<uint32_t*>(obase + (int64_t)(h0 + g) * a.o_sh + col) = w0;
        if (g + 8 < nh) *reinterpret_cast<uint32_t*>(obase + (int64_t)(h0 + g + 8) * a.o_sh + col) = w1;
      }
    }
    return;
  }

  // ---- several CTAs per token (one head group each): partial results to shared memory, combined over the cluster ----
#pragma unroll
  for (int nt = 0; nt < 16; ++nt) {
    if (nt < ntl) {
      const int col = dim0 + nt * 8 + 2 * tg;
      *reinterpret_cast<float2*>(Opart + g * D + col) = make_float2(acc[nt][0], acc[nt][1]);
      *reinterpret_cast<float2*>(Opart + (g + 8) * D + col) = make_float2(acc[nt][2], acc[nt][3]);
    }
  }
  if (w == 0 && tg == 0) {
    mpart[g] = m_row[0];
    mpart[g + 8] = m_row[1];
    lpart[g] = l0;
    lpart[g + 8] = l1;
  }
  ptx::cluster_sync();  // every CTA of the token has written its partial result
  {
    const uint32_t rank = ptx::cluster_ctarank();
    const int cols = D / x.n_split;  // this CTA's share of the columns (D is a multiple of 64, n_split <= 8: at least 8)
    const int vecs = cols / 4;
    const uint32_t o_loc = ptx::smem_u32(Opart), m_loc = ptx::smem_u32(mpart), l_loc = ptx::smem_u32(lpart);
    for (int e = tid; e < 16 * vecs; e += nthreads) {  // four columns of one row per step
      const int row = e / vecs, col = (int)rank * cols + (e - row * vecs) * 4;
      float ms[kMmaMaxSplit], lp[kMmaMaxSplit];
      float4 op[kMmaMaxSplit];
#pragma unroll
      for (int sIdx = 0; sIdx < kMmaMaxSplit; ++sIdx) {  // all loads first: they are independent of each other
        if (sIdx < x.n_split) {
          ms[sIdx] = ptx::ld_cluster_f32(ptx::map_to_cta(m_loc + (uint32_t)row * 4u, (uint32_t)sIdx));
          lp[sIdx] = ptx::ld_cluster_f32(ptx::map_to_cta(l_loc + (uint32_t)row * 4u, (uint32_t)sIdx));
          op[sIdx] = ptx::ld_cluster_f32x4(ptx::map_to_cta(o_loc + (uint32_t)(row * D + col) * 4u, (uint32_t)sIdx));
        } else {
          ms[sIdx] = -INFINITY;
          lp[sIdx] = 0.f;
          op[sIdx] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
      float m = -INFINITY;
#pragma unroll
      for (int sIdx = 0; sIdx < kMmaMaxSplit; ++sIdx) m = fmaxf(m, ms[sIdx]);
      float sl = -INFINITY;
      if (sinks && row < nh) sl = to_float(sinks[h0 + row]) * kLog2e;
      const float m_f = fmaxf(m, sl);
      float l = (sl == -INFINITY) ? 0.f : exp2f(sl - m_f);  // the sink: a score without a value row
      float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int sIdx = 0; sIdx < kMmaMaxSplit; ++sIdx) {
        const float wgt = ms[sIdx] == -INFINITY ? 0.f : exp2f(ms[sIdx] - m_f);
        l += wgt * lp[sIdx];
        o.x += wgt * op[sIdx].x; o.y += wgt * op[sIdx].y; o.z += wgt * op[sIdx].z; o.w += wgt * op[sIdx].w;
      }
      if (row < nh) {
        const float inv = l > 0.f ? 1.f / l : 0.f;
        T* dst = obase + (int64_t)(h0 + row) * a.o_sh + col;
        uint2 pk;
        if constexpr (kBf16) {
          pk.x = ptx::cvt_pack_bf16(o.x * inv, o.y * inv);
          pk.y = ptx::cvt_pack_bf16(o.z * inv, o.w * inv);
        } else {
          pk.x = ptx::cvt_pack_f16(o.x * inv, o.y * inv);
          pk.y = ptx::cvt_pack_f16(o.z * inv, o.w * inv);
        }
        *reinterpret_cast<uint2*>(dst) = pk;
        if (a.lse && col == 0) a.lse[((int64_t)b * a.Hq + h0 + row) * a.Sq + i] = l > 0.f ? m_f * kLn2 + logf(l) : -INFINITY;
      }
    }
  }
  ptx::cluster_sync();  // nobody leaves while its shared memory is still being read
}

// What the tensor-core variant needs: 16-bit tensors, head dim a multiple of 64, every row it gathers 16-byte aligned.
bool sparse_mma_supported(const dt_sparse_indexed_params& p) {
  if (p.dtype != DT_F16 && p.dtype != DT_BF16) return false;
  if (p.D % 64 || p.D > 512) return false;
  auto ok = [](const dt_tensor4& t) {
    return t.ptr == nullptr || (reinterpret_cast<uintptr_t>(t.ptr) % 16 == 0 && t.stride_b % 8 == 0 && t.stride_s % 8 == 0 &&
                                t.stride_h % 8 == 0);
  };
  return ok(p.q) && ok(p.o) && ok(p.k_raw) && ok(p.v_raw) && ok(p.k_comp) && ok(p.v_comp);
}

template <typename T, int TK>
int launch_sparse_mma_tk(const dt_sparse_indexed_params& p, const SparseArgs& a, cudaStream_t stream) {
  auto same = [](const dt_tensor4& u, const dt_tensor4& v) {
    return u.ptr == v.ptr && u.stride_b == v.stride_b && u.stride_s == v.stride_s && u.stride_h == v.stride_h;
  };
  SparseMmaExtra x{};
  x.same_kv = same(p.k_raw, p.v_raw) && (p.Sc == 0 || p.n_selected == 0 || same(p.k_comp, p.v_comp));
  const int G = p.Hq / p.Hkv, ng = (G + 15) / 16;
  const long long ctas = (long long)p.Sq * ng * p.Hkv * p.B;
  // few tokens (the decode step): a token's keys are shared out over a cluster of CTAs, as long as every CTA still gets
  // a few tiles and the grid stays within about two rounds over the SMs
  const int keys = (p.sliding_window > 0 ? (p.sliding_window < p.Sr ? p.sliding_window : p.Sr) : p.Sr) + (p.Sc > 0 ? p.n_selected : 0);
  const int tiles = (keys + TK - 1) / TK;
  int split = 1;
  const int sms = device_sm_count();
  while (split < kMmaMaxSplit && ctas * (split * 2) <= 2LL * sms && tiles >= 2 * (split * 2)) split *= 2;
  x.n_split = split;
  // many tokens: all head groups of a KV head (up to four: 64 heads) in one CTA, so that a gathered row is fetched
  // from L2 once for all of them; with a cluster one group per CTA (more CTAs is what the decode step wants)
  x.gpc = split > 1 ? 1 : (ng < kMmaMaxGroups ? ng : kMmaMaxGroups);
  const int gy = (ng + x.gpc - 1) / x.gpc;
  const int P = p.D + 8;
  const size_t smem = 2 * ((size_t)x.gpc * 16 * P + (size_t)(x.same_kv ? 2 : 4) * TK * P + (size_t)x.gpc * 16 * (TK + 8)) +
                      4 * ((size_t)x.gpc * 128 + 2 * TK + 32);
  auto kern = sparse_mma_kernel<T, TK>;
  if (smem > 48 * 1024) DT_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(p.Sq * split), (unsigned)(p.Hkv * gy), (unsigned)p.B);
  cfg.blockDim = dim3(128 * x.gpc);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = split;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = split > 1 ? 1 : 0;
  DT_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, a, x));
  return DT_OK;
}

// 64 keys per tile when the two K buffers of that size fit beside Q (keys and values in one tensor; otherwise 32)
template <typename T>
int launch_sparse_mma_t(const dt_sparse_indexed_params& p, const SparseArgs& a, cudaStream_t stream) {
  auto same = [](const dt_tensor4& u, const dt_tensor4& v) {
    return u.ptr == v.ptr && u.stride_b == v.stride_b && u.stride_s == v.stride_s && u.stride_h == v.stride_h;
  };
  const bool same_kv = same(p.k_raw, p.v_raw) && (p.Sc == 0 || p.n_selected == 0 || same(p.k_comp, p.v_comp));
  const int keys = (p.sliding_window > 0 ? (p.sliding_window < p.Sr ? p.sliding_window : p.Sr) : p.Sr) + (p.Sc > 0 ? p.n_selected : 0);
  if (same_kv && keys >= 256 && (long long)p.Sq * p.B >= 64) return launch_sparse_mma_tk<T, 64>(p, a, stream);
  return launch_sparse_mma_tk<T, 32>(p, a, stream);
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
  if constexpr (!std::is_same<T, float>::value) {
    if (sparse_mma_supported(p) && !(p.flags & DT_FLAG_FORCE_GENERIC)) return launch_sparse_mma_t<T>(p, a, stream);
  }
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
