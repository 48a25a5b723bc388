// Split-KV grouped-query decode attention (the KV-cache step of
// Libraries/SwiftLLM/Sources/Models/Qwen3_5.swift:183-196: a few new query tokens over T cached rows).
//
// The path is bound by streaming the K and V cache once from HBM.  Layout in HBM is the reference's
// cache layout [B, T, Hkv, D] (Qwen3_5TextGeneration.swift:1639-1655), so one KV head's rows are 2*D-byte
// segments `stride_s` elements apart.
//
//   grid  = (splits, Hkv, B); one CTA streams a contiguous range of 16-key units of ONE KV head and
//           serves all M = Sq * (Hq/Hkv) <= 16 query rows that read it, so K/V are read exactly once.
//   CTA   = 4 consumer warps + 1 producer warp.  The producer issues TMA tile loads (boxes of
//           16 keys x 64 dims, 128-byte swizzle, per-CTA loads) into a ring of stages; each consumer warp
//           owns one 16-key unit per stage: S^T = Q K^T and O += P V with mma.sync m16n8k16 (fp32
//           accumulate) fed by ldmatrix from the swizzled tiles, online softmax in registers with
//           warp-shuffle reductions.
//   merge = the 4 warps' (m, l, O) are merged through shared memory.  Up to 8 splits per (batch, KV head) are
//           launched as ONE thread-block cluster along the split axis: after a cluster barrier every CTA
//           combines its share of the output elements straight out of the other CTAs' shared memory
//           (distributed shared memory, ordinary ld.shared::cluster loads) and stores the result; no partial
//           reaches global memory.  With more splits (few (batch, KV head) pairs, e.g. batch 1) each CTA writes
//           an fp32 partial to the workspace and takes a ticket (atomicAdd), and the CTA that draws the last
//           ticket of its (batch, KV head) combines all partials.  (Measured on B200: clusters of 16, or
//           several clusters per pair, cost more in scheduling than they save: 14.1 - 22 us against 13.4 at
//           batch 1.)  Apart from the hardware cluster barrier (which every CTA reaches unconditionally, also
//           after a wait that ran out) nothing waits on another CTA, so nothing can hang.
#include <stdlib.h>

#include <mutex>

#include "sm100_ptx.cuh"

namespace dt {
namespace {

#ifndef DT_DECODE_MAX_CLUSTER
#define DT_DECODE_MAX_CLUSTER 8  // the portable cluster size; one cluster must hold all splits of a (batch, KV head)
#endif
constexpr int kUnitKeys = 16;
constexpr int kConsumerWarps = 4;
constexpr int kThreads = (kConsumerWarps + 1) * 32;
constexpr int kBoxBytes = kUnitKeys * 128;  // one TMA box: 16 keys x 64 dims x 2 B
constexpr int kMaxRows = 16;
// Ticket counters sit in a fixed-size area at the start of the workspace, so that calls with different
// shapes that share one workspace never see another call's partials where they expect zeroed counters.
constexpr size_t kCounterBytes = 4096;
constexpr int kMaxSplitPairs = (int)(kCounterBytes / sizeof(unsigned int));

template <int D>
struct Cfg {
  static constexpr int kHalves = D / 64;
  static constexpr int kWarpTileBytes = 2 * kHalves * kBoxBytes;  // one 16-key unit: K boxes then V boxes
  // D = 256: two warps share a unit (both compute the scores, each accumulates 128 of the 256 output dims),
  // so that the per-thread accumulators stay at 64 registers
  static constexpr int kDimSplit = D > 128 ? 2 : 1;
  static constexpr int kUnitsPerStage = kConsumerWarps / kDimSplit;
  static constexpr int kDW = D / kDimSplit;  // output dims accumulated by one warp
  static constexpr int kStageBytes = kUnitsPerStage * kWarpTileBytes;
  // A stage is filled by one TMA box per (K | V, 64-dim half) that covers all its units: [K half 0][K half 1]..[V half 0]..,
  // each kStageBox bytes = units x 16 keys x 128 bytes; unit u sits u * kBoxBytes into every box.
  static constexpr int kStageBox = kUnitsPerStage * kBoxBytes;
  // Measured on B200: stage-wide boxes help head dim 256 (16.4 -> 15.2 us at B=1) and cost 3 % at D=128, B=16, where
  // one box per unit streams more evenly; so only D=256 uses them.
  static constexpr bool kStageBoxes = D > 128;
  static constexpr int kHalfStride = kStageBoxes ? kStageBox : kBoxBytes;   // bytes between 64-dim halves of a tile
  static constexpr int kUnitStride = kStageBoxes ? kBoxBytes : kWarpTileBytes;  // bytes between units of a stage
  static constexpr int kBoxRows = kStageBoxes ? kUnitKeys * kUnitsPerStage : kUnitKeys;
  // (A deeper ring for grids that leave every CTA an SM of its own was measured on B200 and changed nothing.)
  static constexpr int kStages = D == 64 ? 4 : 3;
  static constexpr int kRingBytes = kStages * kStageBytes;
  static constexpr int kSmemBytes = kRingBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

struct DecodeArgs {
  const void* q;
  void* o;
  float* lse;
  int64_t q_sb, q_ss, q_sh, o_sb, o_ss, o_sh;
  unsigned int* counters;  // [B*Hkv]
  float* part_ml;          // [B*Hkv][nparts][M][2]
  float* part_o;           // [B*Hkv][nparts][M][D]
  unsigned int* status;
#ifdef DT_BRINGUP
  unsigned long long* dbg;  // optional per-CTA timeline (bring-up probe)
  int skip_loads;           // failure injection on the host's request: the producer lane issues no loads, so the
                            // consumers' bounded wait runs out and the kernel reports it and returns
#endif
  // decode-step fusion (all null / 0 for a plain attention call): new K/V rows to rotate, append and attend
  const void* k_new; const void* v_new; const void* rotary; void* k_cache; void* v_cache;
  int64_t kn_sb, kn_ss, kn_sh, vn_sb, vn_ss, vn_sh, rot_sb, rot_ss, kc_sb, kc_ss, kc_sh, vc_sb, vc_ss, vc_sh;
  int Sq, Sk, Hq, Hkv, G, M;
  int stream_keys;  // cache rows streamed through the ring: Sk, or Sk - Tn with the step fusion
  int unit_first;   // first 16-key unit that any row can see (sliding window), 0 otherwise
  int window;       // sliding window W (0 = off): row i sees keys j > i + (Sk - Sq) - W
  const void* sinks;  // [Hq] attention sinks, or null
  const void* q_norm_w;  // [D] RMSNorm weights applied to the queries / new keys before the rotation, or null
  const void* k_norm_w;
  float norm_eps;
  int Tn;           // new rows appended by the step fusion (<= 16), 0 otherwise
  int nsplit, units_per_split, total_units;
  int cluster;  // nsplit when the splits of a (batch, KV head) form one thread-block cluster, else 1
  int nparts;   // partials per (batch, KV head) that go through global memory: nsplit without a cluster, else none
  float scale_log2;
  int is_causal;
};

#ifdef DT_BRINGUP
#define DT_STAMP(slot) do { if (dbg && threadIdx.x == 0) dbg[slot] = ptx::globaltimer_ns(); } while (0)
#else
#define DT_STAMP(slot) do { } while (0)
#endif

__device__ __forceinline__ uint32_t pack2(float lo, float hi, bool bf16) {
  if (bf16) {
    __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&t);
  }
  __half2 t = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&t);
}

// (x0 + i x1) * (cos + i sin) on one packed 16-bit pair: fp32 products and sum without fused multiply-add
// (so that the result does not depend on how the compiler contracts it), rounded once to T: the reference's
// Functional.cmul (Libraries/SwiftLLM/Sources/Models/Qwen3_5.swift:170-182) on adjacent head dims.
template <typename T>
__device__ __forceinline__ uint32_t cmul_pair(uint32_t x, uint32_t cs) {
  float x0, x1, c, s;
  if constexpr (std::is_same<T, __half>::value) {
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&x));
    const float2 r = __half22float2(*reinterpret_cast<const __half2*>(&cs));
    x0 = a.x; x1 = a.y; c = r.x; s = r.y;
  } else {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&x));
    const float2 r = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&cs));
    x0 = a.x; x1 = a.y; c = r.x; s = r.y;
  }
  return pack2(__fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s)), __fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c)),
               !std::is_same<T, __half>::value);
}

// Attention sink: one more score (natural-log domain logit `sink`) without a value row joins a finished row whose
// running max is `m` (log2 domain), denominator `l` and un-normalised output `o`.
__device__ __forceinline__ void sink_merge(float sink, float& m, float& l, float& o) {
  const float sl = sink * kLog2e;
  const float m2 = fmaxf(m, sl);
  const float down = m == -INFINITY ? 0.f : fast_exp2(m - m2);
  l = l * down + fast_exp2(sl - m2);
  o *= down;
  m = m2;
}

// RMSNorm of one packed pair: (x * inv) * w in fp32 without contraction, rounded once to T (the node the reference
// runs before the rotation, Qwen3_5.swift:164-167).
template <typename T>
__device__ __forceinline__ uint32_t norm_pair(uint32_t x, float inv, uint32_t w) {
  float x0, x1, w0, w1;
  if constexpr (std::is_same<T, __half>::value) {
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&x));
    const float2 g = __half22float2(*reinterpret_cast<const __half2*>(&w));
    x0 = a.x; x1 = a.y; w0 = g.x; w1 = g.y;
  } else {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&x));
    const float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w));
    x0 = a.x; x1 = a.y; w0 = g.x; w1 = g.y;
  }
  return pack2(__fmul_rn(__fmul_rn(x0, inv), w0), __fmul_rn(__fmul_rn(x1, inv), w1), !std::is_same<T, __half>::value);
}

template <typename T>
__device__ __forceinline__ float sumsq_pair(uint32_t x) {
  float2 a;
  if constexpr (std::is_same<T, __half>::value) a = __half22float2(*reinterpret_cast<const __half2*>(&x));
  else a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&x));
  return fmaf(a.x, a.x, a.y * a.y);
}

__device__ __forceinline__ float rsqrt_approx(float x) {
  float y;
  asm("rsqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <typename T, int D>
__global__ void __launch_bounds__(kThreads)
decode_splitkv_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                      const DecodeArgs a) {
  using C = Cfg<D>;
  constexpr bool kBf16 = sizeof(T) == 2 && !std::is_same<T, __half>::value;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t ring = (raw + 1023u) & ~1023u;
  uint8_t* ring_ptr = smem_raw + (ring - raw);
  constexpr int nst = C::kStages;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(ring_ptr + C::kRingBytes);
  uint64_t* empty_bar = full_bar + nst;
  __shared__ int s_abort;
  __shared__ int s_is_last;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
#ifdef DT_BRINGUP
  unsigned long long* dbg = a.dbg ? a.dbg + ((size_t)(b * gridDim.y + kvh) * gridDim.x + split) * 8 : nullptr;
#endif
  DT_STAMP(0);
  const int unit_begin = a.unit_first + split * a.units_per_split;
  const int unit_end = min(a.total_units, unit_begin + a.units_per_split);
  const int n_units = max(0, unit_end - unit_begin);
  const int n_stages = (n_units + C::kUnitsPerStage - 1) / C::kUnitsPerStage;

  // A kernel launched behind this one with programmatic stream serialization (the next decode call, see
  // DT_FLAG_KV_PREFIX_STABLE) may be scheduled as soon as every CTA of this grid has got here; it takes the SM slots
  // that this grid's CTAs free when they exit, while the last CTAs still combine.
  if (threadIdx.x == 0) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (threadIdx.x == kConsumerWarps * 32) {  // the producer lane: the descriptor fetch (about 1 us when cold) starts at once
    ptx::prefetch_tensormap(&map_k);
    ptx::prefetch_tensormap(&map_v);
  }
  if (threadIdx.x == 0) {
    s_abort = 0;
    s_is_last = 0;
    for (int i = 0; i < nst; ++i) {
      ptx::mbar_init(&full_bar[i], 1);
      ptx::mbar_init(&empty_bar[i], kConsumerWarps);
    }
    ptx::fence_mbar_init();
  }
  __syncthreads();

  // per-lane running state of rows lane/4 (lo) and lane/4 + 8 (hi)
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
  float oacc[C::kDW / 8][4];
#pragma unroll
  for (int i = 0; i < C::kDW / 8; ++i) oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.f;
  const int uslot = warp % C::kUnitsPerStage;  // which unit of a stage this warp works on
  const int dhalf = warp / C::kUnitsPerStage;  // which slice of the output dims it accumulates (consumer warps)

  // ---------------- per-warp set-up of the consumer warps (declared here so that the streamed units and
  // the optional extra unit of freshly appended rows share one code path) ----------------
  const int r_lo = lane >> 2, r_hi = r_lo + 8;
  const int cq = (lane & 3) * 2;
  // Q fragments (A operand, rows = (query token, group head), k = head dim)
  uint32_t qa[D / 16][4];
  if (warp < kConsumerWarps) {
    // Programmatic dependent launch (DT_FLAG_KV_PREFIX_STABLE): this grid may have started while the kernel before
    // it in the stream was still running.  The producer warp streams the K/V prefix at once (the caller guarantees
    // that kernel does not write it); everything else -- Q, the new rows, the workspace, the outputs -- is
    // touched only after the preceding grid has completed.  Without the launch attribute this returns at once.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const T* q = reinterpret_cast<const T*>(a.q);
    const T* rot = reinterpret_cast<const T*>(a.rotary);
    const T* p_lo = nullptr;
    const T* p_hi = nullptr;
    const T* t_lo = nullptr;
    const T* t_hi = nullptr;
    if (r_lo < a.M) {
      p_lo = q + b * a.q_sb + (int64_t)(r_lo / a.G) * a.q_ss + (int64_t)(kvh * a.G + r_lo % a.G) * a.q_sh;
      if (rot) t_lo = rot + b * a.rot_sb + (int64_t)(a.Tn - a.Sq + r_lo / a.G) * a.rot_ss;
    }
    if (r_hi < a.M) {
      p_hi = q + b * a.q_sb + (int64_t)(r_hi / a.G) * a.q_ss + (int64_t)(kvh * a.G + r_hi % a.G) * a.q_sh;
      if (rot) t_hi = rot + b * a.rot_sb + (int64_t)(a.Tn - a.Sq + r_hi / a.G) * a.rot_ss;
    }
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      qa[ks][0] = p_lo ? *reinterpret_cast<const uint32_t*>(p_lo + ks * 16 + cq) : 0u;
      qa[ks][1] = p_hi ? *reinterpret_cast<const uint32_t*>(p_hi + ks * 16 + cq) : 0u;
      qa[ks][2] = p_lo ? *reinterpret_cast<const uint32_t*>(p_lo + ks * 16 + cq + 8) : 0u;
      qa[ks][3] = p_hi ? *reinterpret_cast<const uint32_t*>(p_hi + ks * 16 + cq + 8) : 0u;
    }
    if (a.q_norm_w) {
      // per-row RMSNorm: a row's D elements sit in the four lanes that share lane >> 2
      const T* gw = reinterpret_cast<const T*>(a.q_norm_w);
      float ss_lo = 0.f, ss_hi = 0.f;
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        ss_lo += sumsq_pair<T>(qa[ks][0]) + sumsq_pair<T>(qa[ks][2]);
        ss_hi += sumsq_pair<T>(qa[ks][1]) + sumsq_pair<T>(qa[ks][3]);
      }
      ss_lo += __shfl_xor_sync(0xffffffffu, ss_lo, 1);
      ss_lo += __shfl_xor_sync(0xffffffffu, ss_lo, 2);
      ss_hi += __shfl_xor_sync(0xffffffffu, ss_hi, 1);
      ss_hi += __shfl_xor_sync(0xffffffffu, ss_hi, 2);
      const float inv_lo = rsqrt_approx(fmaf(ss_lo, 1.f / (float)D, a.norm_eps));
      const float inv_hi = rsqrt_approx(fmaf(ss_hi, 1.f / (float)D, a.norm_eps));
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const uint32_t g0 = *reinterpret_cast<const uint32_t*>(gw + ks * 16 + cq);
        const uint32_t g1 = *reinterpret_cast<const uint32_t*>(gw + ks * 16 + cq + 8);
        qa[ks][0] = norm_pair<T>(qa[ks][0], inv_lo, g0);
        qa[ks][1] = norm_pair<T>(qa[ks][1], inv_hi, g0);
        qa[ks][2] = norm_pair<T>(qa[ks][2], inv_lo, g1);
        qa[ks][3] = norm_pair<T>(qa[ks][3], inv_hi, g1);
      }
    }
    // rotation as a second pass, so that the loads above stay back to back when there is no table: a fragment
    // register holds head dims (d, d+1) with d even, exactly one (cos, sin) pair of the rotary table
    if (rot) {
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const uint32_t c0 = t_lo ? *reinterpret_cast<const uint32_t*>(t_lo + ks * 16 + cq) : 0u;
        const uint32_t c1 = t_hi ? *reinterpret_cast<const uint32_t*>(t_hi + ks * 16 + cq) : 0u;
        const uint32_t c2 = t_lo ? *reinterpret_cast<const uint32_t*>(t_lo + ks * 16 + cq + 8) : 0u;
        const uint32_t c3 = t_hi ? *reinterpret_cast<const uint32_t*>(t_hi + ks * 16 + cq + 8) : 0u;
        qa[ks][0] = cmul_pair<T>(qa[ks][0], c0);
        qa[ks][1] = cmul_pair<T>(qa[ks][1], c1);
        qa[ks][2] = cmul_pair<T>(qa[ks][2], c2);
        qa[ks][3] = cmul_pair<T>(qa[ks][3], c3);
      }
    }
  }
  // last visible key per row (inclusive)
  const int off = a.Sk - a.Sq;
  const int vis_lo = a.is_causal ? min(a.Sk - 1, r_lo / a.G + off) : a.Sk - 1;
  const int vis_hi = a.is_causal ? min(a.Sk - 1, r_hi / a.G + off) : a.Sk - 1;
  // first visible key per row (sliding window)
  const int lo_lo = a.window > 0 ? r_lo / a.G + off - a.window + 1 : 0;
  const int lo_hi = a.window > 0 ? r_hi / a.G + off - a.window + 1 : 0;

  // one 16-key unit: scores, online softmax, P V.  kbase / vbase: swizzled K and V tiles in shared memory.
  // Keys beyond `last_key` are masked on top of the causal rule (rows past the streamed range are TMA zero fill).
  // half_stride: bytes between the 64-dim halves of a tile (a whole stage box for streamed units).
  auto process_unit = [&](uint32_t kbase, uint32_t vbase, int key0, int last_key, uint32_t half_stride) {
    const int vl_lo = min(vis_lo, last_key), vl_hi = min(vis_hi, last_key);
    float sacc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    {
      const int key = ((lane >> 4) << 3) + (lane & 7);
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const int chunk = ks * 2 + ((lane >> 3) & 1);
        const uint32_t addr = kbase + (chunk >> 3) * half_stride + key * 128 + (((chunk & 7) ^ (key & 7)) << 4);
        uint32_t b00, b01, b10, b11;
        ptx::ldmatrix_x4(b00, b01, b10, b11, addr);
        ptx::mma_m16n8k16<kBf16>(sacc[0], qa[ks], b00, b01);
        ptx::mma_m16n8k16<kBf16>(sacc[1], qa[ks], b10, b11);
      }
    }
    // scale, mask, online softmax
    float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int j = key0 + nt * 8 + cq + e;
        float s0 = sacc[nt][e] * a.scale_log2;
        float s1 = sacc[nt][2 + e] * a.scale_log2;
        if (j > vl_lo || j < lo_lo) s0 = -INFINITY;
        if (j > vl_hi || j < lo_hi) s1 = -INFINITY;
        sacc[nt][e] = s0;
        sacc[nt][2 + e] = s1;
        mx_lo = fmaxf(mx_lo, s0);
        mx_hi = fmaxf(mx_hi, s1);
      }
    }
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
    const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
    const float ms_lo = mn_lo == -INFINITY ? 0.f : mn_lo;
    const float ms_hi = mn_hi == -INFINITY ? 0.f : mn_hi;
    const float al_lo = fast_exp2(m_lo - ms_lo), al_hi = fast_exp2(m_hi - ms_hi);
    m_lo = mn_lo;
    m_hi = mn_hi;
    float ps_lo = 0.f, ps_hi = 0.f;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float p0 = fast_exp2(sacc[nt][e] - ms_lo);
        const float p1 = fast_exp2(sacc[nt][2 + e] - ms_hi);
        sacc[nt][e] = p0;
        sacc[nt][2 + e] = p1;
        ps_lo += p0;
        ps_hi += p1;
      }
    }
    l_lo = l_lo * al_lo + ps_lo;
    l_hi = l_hi * al_hi + ps_hi;
    uint32_t pa[4];
    pa[0] = pack2(sacc[0][0], sacc[0][1], kBf16);
    pa[1] = pack2(sacc[0][2], sacc[0][3], kBf16);
    pa[2] = pack2(sacc[1][0], sacc[1][1], kBf16);
    pa[3] = pack2(sacc[1][2], sacc[1][3], kBf16);
#pragma unroll
    for (int i = 0; i < C::kDW / 8; ++i) {
      oacc[i][0] *= al_lo;
      oacc[i][1] *= al_lo;
      oacc[i][2] *= al_hi;
      oacc[i][3] *= al_hi;
    }
    {
      const int key = (((lane >> 3) & 1) << 3) + (lane & 7);
#pragma unroll
      for (int dp = 0; dp < C::kDW / 16; ++dp) {
        const int chunk = dhalf * (C::kDW / 8) + dp * 2 + (lane >> 4);
        const uint32_t addr = vbase + (chunk >> 3) * half_stride + key * 128 + (((chunk & 7) ^ (key & 7)) << 4);
        uint32_t v00, v01, v10, v11;
        ptx::ldmatrix_x4_trans(v00, v01, v10, v11, addr);
        ptx::mma_m16n8k16<kBf16>(oacc[2 * dp], pa, v00, v01);
        ptx::mma_m16n8k16<kBf16>(oacc[2 * dp + 1], pa, v10, v11);
      }
    }
  };

  if (warp == kConsumerWarps) {
    // ---------------- producer ----------------
#ifdef DT_BRINGUP
    if (lane == 0 && !a.skip_loads) {
#else
    if (lane == 0) {
#endif
      for (int st = 0; st < n_stages; ++st) {
        const int slot = st % nst;
        if (st >= nst) {
          if (!ptx::mbar_wait(&empty_bar[slot], ((st / nst) - 1) & 1, &s_abort)) {
            atomicCAS(a.status, 0u, 2u);
            s_abort = 1;
            break;
          }
        }
        const int u0 = unit_begin + st * C::kUnitsPerStage;
        if constexpr (C::kStageBoxes) {
          // one box per (K | V, half) covers the stage's units; rows past the streamed range are zero fill and units
          // past this split's end are simply not consumed
          const int key0 = u0 * kUnitKeys;
          ptx::mbar_arrive_expect_tx(&full_bar[slot], (uint32_t)C::kStageBytes);
          uint8_t* dst = ring_ptr + slot * C::kStageBytes;
#pragma unroll
          for (int hf = 0; hf < C::kHalves; ++hf) {
            ptx::tma_load_4d(dst + hf * C::kStageBox, &map_k, &full_bar[slot], hf * 64, kvh, key0, b);
            ptx::tma_load_4d(dst + (C::kHalves + hf) * C::kStageBox, &map_v, &full_bar[slot], hf * 64, kvh, key0, b);
          }
        } else {
          const int nu = min(C::kUnitsPerStage, unit_end - u0);
          ptx::mbar_arrive_expect_tx(&full_bar[slot], (uint32_t)(nu * C::kWarpTileBytes));
          for (int w = 0; w < nu; ++w) {
            uint8_t* dst = ring_ptr + slot * C::kStageBytes + w * C::kWarpTileBytes;
            const int key0 = (u0 + w) * kUnitKeys;
#pragma unroll
            for (int hf = 0; hf < C::kHalves; ++hf) {
              ptx::tma_load_4d(dst + hf * kBoxBytes, &map_k, &full_bar[slot], hf * 64, kvh, key0, b);
              ptx::tma_load_4d(dst + (C::kHalves + hf) * kBoxBytes, &map_v, &full_bar[slot], hf * 64, kvh, key0, b);
            }
          }
        }
      }
    }
  } else {
    // ---------------- consumers ----------------
    for (int st = 0; st < n_stages; ++st) {
      const int slot = st % nst;
      if (!ptx::mbar_wait(&full_bar[slot], (st / nst) & 1, &s_abort)) {
        atomicCAS(a.status, 0u, 1u);
        s_abort = 1;
        break;
      }
      if (st == 0) DT_STAMP(1);
      const int unit = unit_begin + st * C::kUnitsPerStage + uslot;
      if (unit < unit_end) {
        const uint32_t kbase = ring + slot * C::kStageBytes + uslot * C::kUnitStride;
        process_unit(kbase, kbase + C::kHalves * C::kHalfStride, unit * kUnitKeys, a.stream_keys - 1, (uint32_t)C::kHalfStride);
      }
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&empty_bar[slot]);
    }
  }

  // ---------------- decode step fusion: rotate, append and attend the new K/V rows ----------------
  // The cache rows streamed above end at Sk - Tn; the Tn new rows come from k_new / v_new.  The last split of
  // each (batch, KV head) rotates the new keys, stores new keys and values into the cache for later steps and
  // attends to them as one more unit built in shared memory (the ring is idle after the barrier).
  if (a.k_new != nullptr) {
    __syncthreads();
    if (split == a.nsplit - 1 && warp < kConsumerWarps && uslot == 0) {
      const uint32_t tile = ring + dhalf * C::kWarpTileBytes;  // with D = 256 the two warps of the pair build one copy each
      const T* kn = reinterpret_cast<const T*>(a.k_new);
      const T* vn = reinterpret_cast<const T*>(a.v_new);
      const T* rot = reinterpret_cast<const T*>(a.rotary);
      T* kc = reinterpret_cast<T*>(a.k_cache);
      T* vc = reinterpret_cast<T*>(a.v_cache);
      const int t_old = a.stream_keys;
      constexpr int kChunks = D / 8;  // 16-byte chunks per row
      // RMSNorm of the new keys: lanes l and l + 16 each sum half of row l's squares; lane l then holds 1 / rms
      const T* kw = reinterpret_cast<const T*>(a.k_norm_w);
      float inv_row = 1.f;
      if (kw) {
        const int row = lane & 15, half = lane >> 4;
        float ss = 0.f;
        if (row < a.Tn) {
          const T* src = kn + b * a.kn_sb + (int64_t)row * a.kn_ss + (int64_t)kvh * a.kn_sh + half * (D / 2);
#pragma unroll
          for (int c = 0; c < D / 16; ++c) {
            const uint4 x = *reinterpret_cast<const uint4*>(src + c * 8);
            ss += sumsq_pair<T>(x.x) + sumsq_pair<T>(x.y) + sumsq_pair<T>(x.z) + sumsq_pair<T>(x.w);
          }
        }
        ss += __shfl_xor_sync(0xffffffffu, ss, 16);
        inv_row = rsqrt_approx(fmaf(ss, 1.f / (float)D, a.norm_eps));
      }
      for (int it = lane; it < kUnitKeys * kChunks; it += 32) {
        const int row = it / kChunks, ch = it - row * kChunks;
        const float inv_k = __shfl_sync(0xffffffffu, inv_row, row);  // uniform trip count: every lane takes part
        uint4 kq = make_uint4(0u, 0u, 0u, 0u), vq = make_uint4(0u, 0u, 0u, 0u);
        if (row < a.Tn) {
          kq = *reinterpret_cast<const uint4*>(kn + b * a.kn_sb + (int64_t)row * a.kn_ss + (int64_t)kvh * a.kn_sh + ch * 8);
          vq = *reinterpret_cast<const uint4*>(vn + b * a.vn_sb + (int64_t)row * a.vn_ss + (int64_t)kvh * a.vn_sh + ch * 8);
          if (kw) {
            const uint4 g = *reinterpret_cast<const uint4*>(kw + ch * 8);
            kq.x = norm_pair<T>(kq.x, inv_k, g.x);
            kq.y = norm_pair<T>(kq.y, inv_k, g.y);
            kq.z = norm_pair<T>(kq.z, inv_k, g.z);
            kq.w = norm_pair<T>(kq.w, inv_k, g.w);
          }
          if (rot) {
            const uint4 rq = *reinterpret_cast<const uint4*>(rot + b * a.rot_sb + (int64_t)row * a.rot_ss + ch * 8);
            kq.x = cmul_pair<T>(kq.x, rq.x);
            kq.y = cmul_pair<T>(kq.y, rq.y);
            kq.z = cmul_pair<T>(kq.z, rq.z);
            kq.w = cmul_pair<T>(kq.w, rq.w);
          }
          if (dhalf == 0) {
            *reinterpret_cast<uint4*>(kc + b * a.kc_sb + (int64_t)(t_old + row) * a.kc_ss + (int64_t)kvh * a.kc_sh + ch * 8) = kq;
            *reinterpret_cast<uint4*>(vc + b * a.vc_sb + (int64_t)(t_old + row) * a.vc_ss + (int64_t)kvh * a.vc_sh + ch * 8) = vq;
          }
        }
        const uint32_t o = (uint32_t)(ch >> 3) * kBoxBytes + (uint32_t)row * 128 + ((((uint32_t)ch & 7u) ^ ((uint32_t)row & 7u)) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(tile + o), "r"(kq.x), "r"(kq.y), "r"(kq.z), "r"(kq.w) : "memory");
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(tile + C::kHalves * kBoxBytes + o), "r"(vq.x), "r"(vq.y),
                     "r"(vq.z), "r"(vq.w)
                     : "memory");
      }
      __syncwarp();
      process_unit(tile, tile + C::kHalves * kBoxBytes, t_old, a.Sk - 1, (uint32_t)kBoxBytes);
    }
  }
  if (warp < kConsumerWarps) {
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
  }

  // ---------------- merge the consumer warps through shared memory (ring is idle now) ----------------
  __syncthreads();
  DT_STAMP(2);
  float* obuf = reinterpret_cast<float*>(ring_ptr);                    // [units per stage][16][D]
  float* mbuf = obuf + C::kUnitsPerStage * kMaxRows * D;               // [units per stage][16]
  float* lbuf = mbuf + C::kUnitsPerStage * kMaxRows;                   // [units per stage][16]
  float* cta_o = lbuf + C::kUnitsPerStage * kMaxRows;                  // [16][D]  this CTA's merged O (cluster mode)
  float* cta_ml = cta_o + kMaxRows * D;                                // [16][2]  this CTA's merged (m, l)
  float* comb = cta_ml + 2 * kMaxRows;                                 // scratch of the final combine
  if (warp < kConsumerWarps) {
    const int r_lo = lane >> 2, r_hi = r_lo + 8, cq = (lane & 3) * 2;
    float* ob = obuf + uslot * kMaxRows * D + dhalf * C::kDW;
    // only the M valid rows are merged; float2 stores, row pitch D floats
    if (r_lo < a.M) {
#pragma unroll
      for (int i = 0; i < C::kDW / 8; ++i) *reinterpret_cast<float2*>(&ob[r_lo * D + i * 8 + cq]) = make_float2(oacc[i][0], oacc[i][1]);
    }
    if (r_hi < a.M) {
#pragma unroll
      for (int i = 0; i < C::kDW / 8; ++i) *reinterpret_cast<float2*>(&ob[r_hi * D + i * 8 + cq]) = make_float2(oacc[i][2], oacc[i][3]);
    }
    if ((lane & 3) == 0 && dhalf == 0) {
      mbuf[uslot * kMaxRows + r_lo] = m_lo;
      mbuf[uslot * kMaxRows + r_hi] = m_hi;
      lbuf[uslot * kMaxRows + r_lo] = l_lo;
      lbuf[uslot * kMaxRows + r_hi] = l_hi;
    }
  }
  __syncthreads();

  const int pair = b * a.Hkv + kvh;
  const int MD = a.M * D;
  T* o = reinterpret_cast<T*>(a.o);
  // final result of one output element: sink, normalisation, store (and the row's log-sum-exp once per row)
  auto store_final = [&](int r, int d, float mstar, float lt, float ot) {
    const int sq = r / a.G, h = kvh * a.G + r % a.G;
    if (a.sinks) sink_merge(to_float(reinterpret_cast<const T*>(a.sinks)[h]), mstar, lt, ot);
    o[b * a.o_sb + (int64_t)sq * a.o_ss + (int64_t)h * a.o_sh + d] = from_float<T>(lt > 0.f ? ot / lt : 0.f);
    if (a.lse && d == 0) a.lse[((int64_t)b * a.Hq + h) * a.Sq + sq] = lt > 0.f ? mstar * kLn2 + logf(lt) : -INFINITY;
  };
  for (int idx = threadIdx.x; idx < MD; idx += kThreads) {
    const int r = idx / D, d = idx - r * D;
    float mstar = -INFINITY;
#pragma unroll
    for (int w = 0; w < C::kUnitsPerStage; ++w) mstar = fmaxf(mstar, mbuf[w * kMaxRows + r]);
    float lt = 0.f, ot = 0.f;
    if (mstar != -INFINITY) {
#pragma unroll
      for (int w = 0; w < C::kUnitsPerStage; ++w) {
        const float wgt = fast_exp2(mbuf[w * kMaxRows + r] - mstar);
        lt += wgt * lbuf[w * kMaxRows + r];
        ot += wgt * obuf[(w * kMaxRows + r) * D + d];
      }
    }
    if (a.cluster > 1) {
      cta_o[idx] = ot;
      if (d == 0) {
        cta_ml[2 * r] = mstar;
        cta_ml[2 * r + 1] = lt;
      }
    } else if (a.nsplit == 1) {
      store_final(r, d, mstar, lt, ot);
    } else {
      const int64_t slot = (int64_t)pair * a.nparts + split;
      a.part_o[slot * MD + idx] = ot;
      if (d == 0) {
        a.part_ml[(slot * a.M + r) * 2] = mstar;
        a.part_ml[(slot * a.M + r) * 2 + 1] = lt;
      }
    }
  }
  if (a.cluster == 1 && a.nsplit == 1) return;

  if (a.cluster > 1) {
    // ---------------- cluster combine through distributed shared memory ----------------
    // Every CTA of the cluster gets here whatever happened before (a wait that ran out falls through to this
    // point), so the hardware barrier always completes.  After it, CTA c of the cluster owns output elements
    // [c * per, (c + 1) * per) and reads them, and every CTA's (m, l), from all the cluster's shared memories.
    ptx::cluster_sync();
    DT_STAMP(3);
    const int crank = (int)ptx::cluster_ctarank();
    const int per = (MD + a.cluster - 1) / a.cluster;
    const uint32_t o_local = ptx::smem_u32(cta_o), ml_local = ptx::smem_u32(cta_ml);
    const int idx_end = min(MD, (crank + 1) * per);
    for (int idx = crank * per + threadIdx.x; idx < idx_end; idx += kThreads) {
      const int r = idx / D, d = idx - r * D;
      float mv[DT_DECODE_MAX_CLUSTER], lv[DT_DECODE_MAX_CLUSTER], ov[DT_DECODE_MAX_CLUSTER];
#pragma unroll
      for (int c = 0; c < DT_DECODE_MAX_CLUSTER; ++c) {
        if (c < a.cluster) {
          const uint32_t ml_remote = ptx::map_to_cta(ml_local + (uint32_t)r * 8u, (uint32_t)c);
          mv[c] = ptx::ld_cluster_f32(ml_remote);
          lv[c] = ptx::ld_cluster_f32(ml_remote + 4u);
          ov[c] = ptx::ld_cluster_f32(ptx::map_to_cta(o_local + (uint32_t)idx * 4u, (uint32_t)c));
        } else {
          mv[c] = -INFINITY;
          lv[c] = 0.f;
          ov[c] = 0.f;
        }
      }
      float mstar = -INFINITY;
#pragma unroll
      for (int c = 0; c < DT_DECODE_MAX_CLUSTER; ++c) mstar = fmaxf(mstar, mv[c]);
      float lt = 0.f, ot = 0.f;
      if (mstar != -INFINITY) {
#pragma unroll
        for (int c = 0; c < DT_DECODE_MAX_CLUSTER; ++c) {
          const float wgt = fast_exp2(mv[c] - mstar);  // exp2(-inf) = 0 for the unused slots
          lt = fmaf(wgt, lv[c], lt);
          ot = fmaf(wgt, ov[c], ot);
        }
      }
      store_final(r, d, mstar, lt, ot);
    }
    // no CTA may exit while another still reads its shared memory
    ptx::cluster_sync();
    DT_STAMP(4);
    return;
  }

  // ---------------- ticket: the last partial of this (batch, KV head) to arrive combines ----------------
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int ticket = atomicAdd(&a.counters[pair], 1u);
    s_is_last = (ticket == (unsigned int)(a.nparts - 1));
  }
  __syncthreads();
  if (!s_is_last) return;
  __threadfence();
  // Combine.  Up to 32 partials: one warp per output row, one round trip.  Lane s fetches partial s's (m, l) of the row
  // while every lane fetches its float4 column of all the partials' O; the weights come out of warp reductions and
  // travel by shuffle, so nothing waits on a second dependent load or on shared memory.  (B=1, D=128: 13.4 -> 12.9 us
  // per call; head dim 256 would need two column passes per row and measured slower this way, it keeps the form below.)
  if (D <= 128 && a.nparts <= 32) {
    const int np = a.nparts;
    const int64_t base = (int64_t)pair * np;
    constexpr int kVec = D / 4;
    const int64_t part_stride = (int64_t)a.M * kVec;
    for (int r = warp; r < a.M; r += kThreads / 32) {
      float2 ml = make_float2(-INFINITY, 0.f);
      if (lane < np) ml = __ldcg(reinterpret_cast<const float2*>(&a.part_ml[((base + lane) * a.M + r) * 2]));
#pragma unroll 1
      for (int c0 = 0; c0 < kVec; c0 += 32) {
        const int d4 = c0 + lane;
        const bool col_ok = d4 < kVec;
        const float4* src = reinterpret_cast<const float4*>(a.part_o) + (base * a.M + r) * kVec + (col_ok ? d4 : 0);
        float4 v[32];
#pragma unroll
        for (int u = 0; u < 32; ++u)
          v[u] = (u < np && col_ok) ? __ldcg(src + u * part_stride) : make_float4(0.f, 0.f, 0.f, 0.f);
        float mstar = ml.x;
#pragma unroll
        for (int o2 = 16; o2 > 0; o2 >>= 1) mstar = fmaxf(mstar, __shfl_xor_sync(0xffffffffu, mstar, o2));
        float wgt = mstar == -INFINITY ? 0.f : fast_exp2(ml.x - mstar);
        float lt = wgt * ml.y;
#pragma unroll
        for (int o2 = 16; o2 > 0; o2 >>= 1) lt += __shfl_xor_sync(0xffffffffu, lt, o2);
        if (a.sinks) {
          // the sink is one more partial: weight 1 for it, every partial's weight rescaled to the common max
          const float sl = to_float(reinterpret_cast<const T*>(a.sinks)[kvh * a.G + r % a.G]) * kLog2e;
          const float m2 = fmaxf(mstar, sl);
          const float down = mstar == -INFINITY ? 0.f : fast_exp2(mstar - m2);
          wgt *= down;
          lt = lt * down + fast_exp2(sl - m2);
          mstar = m2;
        }
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int u = 0; u < 32; ++u) {
          const float wu = __shfl_sync(0xffffffffu, wgt, u);
          acc.x = fmaf(wu, v[u].x, acc.x);
          acc.y = fmaf(wu, v[u].y, acc.y);
          acc.z = fmaf(wu, v[u].z, acc.z);
          acc.w = fmaf(wu, v[u].w, acc.w);
        }
        const float inv = lt > 0.f ? 1.f / lt : 0.f;
        const int sq = r / a.G, h = kvh * a.G + r % a.G;
        if (col_ok) {
          T* dst = o + b * a.o_sb + (int64_t)sq * a.o_ss + (int64_t)h * a.o_sh + d4 * 4;
          dst[0] = from_float<T>(acc.x * inv);
          dst[1] = from_float<T>(acc.y * inv);
          dst[2] = from_float<T>(acc.z * inv);
          dst[3] = from_float<T>(acc.w * inv);
        }
        if (a.lse && c0 == 0 && lane == 0) a.lse[((int64_t)b * a.Hq + h) * a.Sq + sq] = lt > 0.f ? mstar * kLn2 + logf(lt) : -INFINITY;
      }
    }
  } else {
  // More partials than lanes.  All loads of a phase are independent so they overlap: first every (partial, row) pair's (m, l) lands in
  // shared memory and one warp per row turns them into weights (lanes over partials, shuffle reductions); then each
  // thread owns one float4 of one output row and streams the partial O, 32 loads in flight.
  {
    const int np = a.nparts;
    const int64_t base = (int64_t)pair * np;
    float* wbuf = comb;                      // [np][M] weights
    float* lsm = wbuf + np * a.M;            // [np][M] l
    float* rowinfo = lsm + np * a.M;         // [M][2]: m*, L
    const int nm = np * a.M;
    constexpr int kVec = D / 4;
    const int64_t part_stride = (int64_t)a.M * kVec;
    for (int idx = threadIdx.x; idx < nm; idx += kThreads) {
      const float2 ml = __ldcg(reinterpret_cast<const float2*>(&a.part_ml[(base * a.M + idx) * 2]));
      wbuf[idx] = ml.x;
      lsm[idx] = ml.y;
    }
    __syncthreads();
    for (int r = warp; r < a.M; r += kThreads / 32) {
      float mstar = -INFINITY;
      for (int sp = lane; sp < np; sp += 32) mstar = fmaxf(mstar, wbuf[sp * a.M + r]);
#pragma unroll
      for (int o2 = 16; o2 > 0; o2 >>= 1) mstar = fmaxf(mstar, __shfl_xor_sync(0xffffffffu, mstar, o2));
      float lt = 0.f;
      for (int sp = lane; sp < np; sp += 32) {
        const float wgt = mstar == -INFINITY ? 0.f : fast_exp2(wbuf[sp * a.M + r] - mstar);
        wbuf[sp * a.M + r] = wgt;
        lt += wgt * lsm[sp * a.M + r];
      }
#pragma unroll
      for (int o2 = 16; o2 > 0; o2 >>= 1) lt += __shfl_xor_sync(0xffffffffu, lt, o2);
      if (a.sinks) {
        // the sink is one more partial: weight 1 for it, every partial's weight rescaled to the common max
        const float sl = to_float(reinterpret_cast<const T*>(a.sinks)[kvh * a.G + r % a.G]) * kLog2e;
        const float m2 = fmaxf(mstar, sl);
        const float down = mstar == -INFINITY ? 0.f : fast_exp2(mstar - m2);
        for (int sp = lane; sp < np; sp += 32) wbuf[sp * a.M + r] *= down;
        lt = lt * down + fast_exp2(sl - m2);
        mstar = m2;
      }
      if (lane == 0) {
        rowinfo[2 * r] = mstar;
        rowinfo[2 * r + 1] = lt;
      }
    }
    __syncthreads();
    for (int item = threadIdx.x; item < a.M * kVec; item += kThreads) {
      const int r = item / kVec, d4 = item - r * kVec;
      const float4* src = reinterpret_cast<const float4*>(a.part_o) + (base * a.M + r) * kVec + d4;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int s0 = 0; s0 < np; s0 += 32) {  // up to 32 independent loads in flight per thread
        float4 v[32];
#pragma unroll
        for (int u = 0; u < 32; ++u)
          v[u] = (s0 + u < np) ? __ldcg(src + (s0 + u) * part_stride) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int u = 0; u < 32; ++u) {
          const float wgt = (s0 + u < np) ? wbuf[(s0 + u) * a.M + r] : 0.f;
          acc.x = fmaf(wgt, v[u].x, acc.x);
          acc.y = fmaf(wgt, v[u].y, acc.y);
          acc.z = fmaf(wgt, v[u].z, acc.z);
          acc.w = fmaf(wgt, v[u].w, acc.w);
        }
      }
      const float mstar = rowinfo[2 * r], lt = rowinfo[2 * r + 1];
      const float inv = lt > 0.f ? 1.f / lt : 0.f;
      const int sq = r / a.G, h = kvh * a.G + r % a.G;
      T* dst = o + b * a.o_sb + (int64_t)sq * a.o_ss + (int64_t)h * a.o_sh + d4 * 4;
      dst[0] = from_float<T>(acc.x * inv);
      dst[1] = from_float<T>(acc.y * inv);
      dst[2] = from_float<T>(acc.z * inv);
      dst[3] = from_float<T>(acc.w * inv);
      if (a.lse && d4 == 0) a.lse[((int64_t)b * a.Hq + h) * a.Sq + sq] = lt > 0.f ? mstar * kLn2 + logf(lt) : -INFINITY;
    }
  }
  }
  DT_STAMP(5);
  if (threadIdx.x == 0) a.counters[pair] = 0u;  // leave the workspace ready for the next call
}

// ---- host side ---------------------------------------------------------------------------------------

constexpr int kMaxParts = 256;    // partials per (batch, KV head) the final combine has shared memory for
constexpr int kMaxDevices = 64;
constexpr int kVariants = 6;      // (fp16 | bf16) x (D = 64, 128, 256)

// What the host side remembers per device: cudaFuncSetAttribute and the cluster occupancy answer are per device,
// and a process may drive several devices (one host thread per GPU).
struct DeviceState {
  int sm_count = 0;
  bool attr_set[kVariants] = {false, false, false, false, false, false};
  int max_cluster[kVariants] = {0, 0, 0, 0, 0, 0};  // 0 = not asked yet
  unsigned char* noalloc_scratch = nullptr;         // device addresses of the built-in scratch and its status word
  unsigned int* noalloc_status = nullptr;
};
DeviceState g_dev[kMaxDevices];
std::mutex g_dev_mu;

// Current device's slot, or null when there is no usable device (sizes are then computed for a 148-SM part).
DeviceState* device_state() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    cudaGetLastError();
    return nullptr;
  }
  DeviceState* d = &g_dev[dev];
  std::lock_guard<std::mutex> lk(g_dev_mu);
  if (d->sm_count == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    d->sm_count = n;
  }
  return d;
}

int sm_count() {
  DeviceState* d = device_state();
  return d ? d->sm_count : 148;
}

#ifdef DT_BRINGUP
unsigned long long* g_decode_dbg = nullptr;
int g_decode_skip_loads = 0;
#endif

struct Plan {
  int nsplit, units_per_split, total_units;
  int cluster;  // nsplit when the splits should form one cluster, else 1 (the launch falls back to 1 when the device cannot co-schedule it)
};

// first 16-key unit any row of the call can see: row 0's window bound
int first_unit(const dt_sdpa_params& p) {
  if (p.sliding_window <= 0) return 0;
  const long long lo = (long long)(p.Sk - p.Sq) - p.sliding_window + 1;
  return lo <= 0 ? 0 : (int)(lo / kUnitKeys);
}

// Split count: the path is bound by HBM, and what costs is the fixed part of a CTA (start-up, merge, combine), so
// use as few CTAs as keep every SM streaming: the largest power of two with pairs * splits <= the CTAs that are
// resident at once (one wave), and at least four 16-key units per split.  (Measured on B200: B=16 runs at 99% of
// the copy peak with 2 splits and at 57% with 37.)  The caller may fix the count with DT_FLAG_DECODE_SPLITS.
Plan make_plan(const dt_sdpa_params& p, int stream_keys) {
  Plan pl;
  pl.cluster = 1;
  pl.total_units = (stream_keys + kUnitKeys - 1) / kUnitKeys - min((stream_keys + kUnitKeys - 1) / kUnitKeys, first_unit(p));
  if (pl.total_units == 0) {  // empty cache (first step of a sequence): one CTA per pair, nothing streamed
    pl.nsplit = 1;
    pl.units_per_split = 0;
    return pl;
  }
  const int pairs = p.B * p.Hkv;
  // resident CTAs per SM: two, except head dim 256 whose 215 registers per thread leave room for one
  const int slots = (p.D > 128 ? 1 : 2) * sm_count();
  int ns = 1;
  while (pairs * ns * 2 <= slots && pl.total_units / (ns * 2) >= 4) ns *= 2;
  int forced = (int)((p.flags >> 16) & 0xFFFu);
#ifdef DT_BRINGUP
  if (const char* env = getenv("DTATTN_DECODE_SPLITS")) forced = atoi(env);
#endif
  if (forced > 0) ns = min(min(forced, kMaxParts), pl.total_units);
  if (pairs > kMaxSplitPairs) ns = 1;  // more (batch, KV head) pairs than counters: plenty of CTAs anyway
  pl.units_per_split = (pl.total_units + ns - 1) / ns;
  // a power-of-two count is kept as it is (trailing splits may be empty) so that it still forms clusters
  pl.nsplit = (ns & (ns - 1)) == 0 ? ns : (pl.total_units + pl.units_per_split - 1) / pl.units_per_split;
  int cap = DT_DECODE_MAX_CLUSTER;
#ifdef DT_BRINGUP
  if (const char* env = getenv("DTATTN_DECODE_CLUSTER")) cap = max(1, atoi(env));
#endif
  // one cluster for all splits of a pair, or none
  pl.cluster = pl.nsplit > 1 && pl.nsplit <= cap && (pl.nsplit & (pl.nsplit - 1)) == 0 ? pl.nsplit : 1;
  return pl;
}

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// Bytes of scratch for `nparts` global partials per (batch, KV head).
size_t scratch_bytes(const dt_sdpa_params& p, int nparts) {
  if (nparts <= 1) return 0;
  const size_t pairs = (size_t)p.B * p.Hkv;
  const size_t M = (size_t)p.Sq * (p.Hq / p.Hkv);
  return kCounterBytes + align_up(pairs * nparts * M * 2 * sizeof(float), 256) +
         align_up(pairs * nparts * M * p.D * sizeof(float), 256);
}

// What dt_sdpa_workspace_size reports: enough for every cluster size the launch may end up with (a device that
// cannot co-schedule the wanted cluster falls back to a smaller one and then writes more partials).
size_t plan_workspace_bytes(const dt_sdpa_params& p, const Plan& pl) { return scratch_bytes(p, pl.nsplit); }

// Where the partials live: the caller's workspace, or the library's built-in array (dt_sdpa_decode_noalloc).
struct Scratch {
  void* ptr;
  size_t bytes;
  unsigned int* status;    // device status word the kernel reports to
  bool stale;              // the memory keeps an earlier call's contents: clear the ticket counters first
  bool reported_size;      // a caller workspace must hold what dt_sdpa_workspace_size reported, whatever this launch uses
  int too_small;           // status returned when the partials do not fit
};

template <typename T, int D>
constexpr int variant_index() {
  return (std::is_same<T, __half>::value ? 0 : 3) + (D == 64 ? 0 : D == 128 ? 1 : 2);
}

// Largest cluster size <= `want` this device can co-schedule for this kernel (asked once per device and variant).
template <typename T, int D>
int usable_cluster(DeviceState* dev, int want) {
  using C = Cfg<D>;
  constexpr int vi = variant_index<T, D>();
  auto kern = decode_splitkv_kernel<T, D>;
  std::lock_guard<std::mutex> lk(g_dev_mu);
  if (dev->max_cluster[vi] == 0) {
    int best = 1;
    for (int c = DT_DECODE_MAX_CLUSTER; c > 1; c /= 2) {
      if (c > 8 && cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) {
        cudaGetLastError();
        continue;
      }
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(c, 1, 1);
      cfg.blockDim = dim3(kThreads);
      cfg.dynamicSmemBytes = C::kSmemBytes;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = c;
      attr[0].val.clusterDim.y = 1;
      attr[0].val.clusterDim.z = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) == cudaSuccess && n > 0) {
        best = c;
        break;
      }
      cudaGetLastError();
    }
    dev->max_cluster[vi] = best;
  }
  return want <= dev->max_cluster[vi] ? want : 1;
}

template <typename T, int D>
int launch_t(const dt_sdpa_params& p, const dt_decode_step_params* step, const Scratch& scratch, cudaStream_t stream) {
  using C = Cfg<D>;
  DeviceState* dev = device_state();
  if (!dev) return DT_NO_DEVICE;
  auto kern = decode_splitkv_kernel<T, D>;
  constexpr int vi = variant_index<T, D>();
  {
    std::lock_guard<std::mutex> lk(g_dev_mu);
    if (!dev->attr_set[vi]) {
      DT_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
      dev->attr_set[vi] = true;
    }
  }
  const int Tn = step ? step->T_new : 0;
  const int stream_keys = p.Sk - Tn;
  const Plan pl = make_plan(p, stream_keys);
  const int G = p.Hq / p.Hkv, M = p.Sq * G;
  const size_t pairs = (size_t)p.B * p.Hkv;
  DecodeArgs a{};
  a.cluster = pl.cluster > 1 ? usable_cluster<T, D>(dev, pl.cluster) : 1;
  a.nparts = a.cluster > 1 ? 1 : pl.nsplit;
  if (scratch.reported_size) {
    const size_t reported = plan_workspace_bytes(p, pl);
    if (reported > 0 && (!scratch.ptr || scratch.bytes < reported)) return scratch.too_small;
  }
  if (a.nparts > 1) {
    const size_t need = scratch_bytes(p, a.nparts);
    if (!scratch.ptr || scratch.bytes < need) return scratch.too_small;
    uint8_t* w = reinterpret_cast<uint8_t*>(scratch.ptr);
    a.counters = reinterpret_cast<unsigned int*>(w);
    size_t off = kCounterBytes;
    a.part_ml = reinterpret_cast<float*>(w + off);
    off += align_up(pairs * a.nparts * M * 2 * sizeof(float), 256);
    a.part_o = reinterpret_cast<float*>(w + off);
    if (scratch.stale) DT_CUDA_TRY(cudaMemsetAsync(a.counters, 0, pairs * sizeof(unsigned int), stream));
  }
  // The maps cover exactly the streamed rows: what a unit reads past them is TMA zero fill, never the rows
  // another CTA of this launch is appending.  (An empty cache still needs a valid map; it is never read.)
  CUtensorMap mk, mv;
  const int map_rows = stream_keys > 0 ? stream_keys : 1;
  if (!make_bshd_tensor_map(&mk, p.k, p.B, map_rows, p.Hkv, D, p.dtype, C::kBoxRows)) return DT_UNSUPPORTED;
  if (!make_bshd_tensor_map(&mv, p.v, p.B, map_rows, p.Hkv, D, p.dtype, C::kBoxRows)) return DT_UNSUPPORTED;
  a.q = p.q.ptr; a.o = p.o.ptr; a.lse = p.lse;
  a.q_sb = p.q.stride_b; a.q_ss = p.q.stride_s; a.q_sh = p.q.stride_h;
  a.o_sb = p.o.stride_b; a.o_ss = p.o.stride_s; a.o_sh = p.o.stride_h;
  a.status = scratch.status;
  if (!a.status) return DT_CUDA;
#ifdef DT_BRINGUP
  a.dbg = g_decode_dbg;
  a.skip_loads = g_decode_skip_loads;
#endif
  a.Sq = p.Sq; a.Sk = p.Sk; a.Hq = p.Hq; a.Hkv = p.Hkv; a.G = G; a.M = M;
  a.stream_keys = stream_keys;
  a.Tn = Tn;
  if (step) {
    a.k_new = step->k_new.ptr; a.v_new = step->v_new.ptr; a.rotary = step->rotary;
    a.k_cache = p.k.ptr; a.v_cache = p.v.ptr;
    a.kn_sb = step->k_new.stride_b; a.kn_ss = step->k_new.stride_s; a.kn_sh = step->k_new.stride_h;
    a.vn_sb = step->v_new.stride_b; a.vn_ss = step->v_new.stride_s; a.vn_sh = step->v_new.stride_h;
    a.rot_sb = step->rotary_stride_b; a.rot_ss = step->rotary_stride_s;
    a.q_norm_w = step->q_norm_weight; a.k_norm_w = step->k_norm_weight; a.norm_eps = step->norm_eps;
    a.kc_sb = p.k.stride_b; a.kc_ss = p.k.stride_s; a.kc_sh = p.k.stride_h;
    a.vc_sb = p.v.stride_b; a.vc_ss = p.v.stride_s; a.vc_sh = p.v.stride_h;
  }
  a.nsplit = pl.nsplit; a.units_per_split = pl.units_per_split;
  a.unit_first = min(first_unit(p), (a.stream_keys + kUnitKeys - 1) / kUnitKeys);
  a.total_units = a.unit_first + pl.total_units;  // one past the last streamed unit
  a.window = p.sliding_window;
  a.sinks = p.sinks;
  a.scale_log2 = p.scale * kLog2e;
  a.is_causal = p.is_causal;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(pl.nsplit, p.Hkv, p.B);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = C::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n_attr = 0;
  if (a.cluster > 1) {
    attr[n_attr].id = cudaLaunchAttributeClusterDimension;
    attr[n_attr].val.clusterDim.x = a.cluster;
    attr[n_attr].val.clusterDim.y = 1;
    attr[n_attr].val.clusterDim.z = 1;
    ++n_attr;
  }
  if (p.flags & DT_FLAG_KV_PREFIX_STABLE) {
    attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
    ++n_attr;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n_attr;
  DT_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, mk, mv, a));
  return DT_OK;
}

}  // namespace

bool decode_supported(const dt_sdpa_params& p) {
  if (p.seq_offsets_q) return false;  // variable-length batches: generic kernel
  if (p.dtype != DT_F16 && p.dtype != DT_BF16) return false;
  if (p.D != 64 && p.D != 128 && p.D != 256) return false;  // 256: the reference's Qwen3.5 configs (Qwen3_5.swift:59-82)
  if (p.mask) return false;
  if (p.Hq % p.Hkv) return false;
  const int M = p.Sq * (p.Hq / p.Hkv);
  if (M > kMaxRows) return false;
  if (p.Hkv > 65535 || p.B > 65535) return false;
  // TMA and 32-bit fragment loads: 16-byte aligned bases, strides multiples of 8 elements
  auto ok = [](const dt_tensor4& t) {
    return (reinterpret_cast<uintptr_t>(t.ptr) % 16 == 0) && t.stride_b % 8 == 0 && t.stride_s % 8 == 0 &&
           t.stride_h % 8 == 0;
  };
  return ok(p.q) && ok(p.k) && ok(p.v);
}

size_t decode_workspace_bytes(const dt_sdpa_params& p) { return plan_workspace_bytes(p, make_plan(p, p.Sk)); }

namespace {
int dispatch_decode(const dt_sdpa_params& p, const dt_decode_step_params* step, const Scratch& scratch,
                    cudaStream_t stream) {
  if (p.dtype == DT_F16) {
    if (p.D == 256) return launch_t<__half, 256>(p, step, scratch, stream);
    return p.D == 128 ? launch_t<__half, 128>(p, step, scratch, stream) : launch_t<__half, 64>(p, step, scratch, stream);
  }
  if (p.D == 256) return launch_t<__nv_bfloat16, 256>(p, step, scratch, stream);
  return p.D == 128 ? launch_t<__nv_bfloat16, 128>(p, step, scratch, stream)
                    : launch_t<__nv_bfloat16, 64>(p, step, scratch, stream);
}

Scratch caller_workspace(void* workspace, size_t bytes) {
  return Scratch{workspace, bytes, device_status_word(), false, true, DT_WORKSPACE};
}

// Argument rules of the fused decode step on top of decode_supported().
int validate_step(const dt_decode_step_params* s) {
  if (!s) return DT_BAD_ARG;
  const dt_sdpa_params& p = s->attn;
  const int base = validate_params(&p);
  if (base != DT_OK) return base;
  if (!s->k_new.ptr || !s->v_new.ptr) return DT_BAD_ARG;
  if (s->T_new < p.Sq || s->T_new > p.Sk) return DT_BAD_ARG;
  if (s->T_new > kUnitKeys) return DT_UNSUPPORTED;  // the new rows form one 16-key unit
  if (!p.is_causal && s->T_new != p.Sq) return DT_BAD_ARG;
  if (!decode_supported(p)) return DT_UNSUPPORTED;
  auto ok = [](const dt_tensor4& t) {
    return (reinterpret_cast<uintptr_t>(t.ptr) % 16 == 0) && t.stride_b % 8 == 0 && t.stride_s % 8 == 0 &&
           t.stride_h % 8 == 0;
  };
  if (!ok(s->k_new) || !ok(s->v_new)) return DT_UNSUPPORTED;
  if (s->rotary && (reinterpret_cast<uintptr_t>(s->rotary) % 16 || s->rotary_stride_b % 8 || s->rotary_stride_s % 8))
    return DT_UNSUPPORTED;
  if ((s->q_norm_weight && reinterpret_cast<uintptr_t>(s->q_norm_weight) % 16) ||
      (s->k_norm_weight && reinterpret_cast<uintptr_t>(s->k_norm_weight) % 16))
    return DT_UNSUPPORTED;
  if ((s->q_norm_weight || s->k_norm_weight) && !(s->norm_eps >= 0.f)) return DT_BAD_ARG;
  return DT_OK;
}
}  // namespace

int launch_decode(const dt_sdpa_params& p, void* workspace, size_t bytes, cudaStream_t stream) {
  return dispatch_decode(p, nullptr, caller_workspace(workspace, bytes), stream);
}

}  // namespace dt

// ---- fused decode step -------------------------------------------------------------------------------
extern "C" int dt_sdpa_decode_step_workspace_size(const dt_decode_step_params* s, size_t* bytes) {
  using namespace dt;
  if (!bytes) return DT_BAD_ARG;
  const int st = validate_step(s);
  if (st != DT_OK) return st;
  *bytes = plan_workspace_bytes(s->attn, make_plan(s->attn, s->attn.Sk - s->T_new));
  return DT_OK;
}

extern "C" int dt_sdpa_decode_step(const dt_decode_step_params* s, void* workspace, size_t workspace_bytes,
                                   void* cuda_stream) {
  using namespace dt;
  const int st = validate_step(s);
  if (st != DT_OK) return st;
  return dispatch_decode(s->attn, s, caller_workspace(workspace, workspace_bytes), reinterpret_cast<cudaStream_t>(cuda_stream));
}

// ---- entry point that allocates nothing ----------------------------------------------------------------
// Scratch for the split-KV partials lives in a file-scope device array instead of a caller workspace.
// Every GPU that loads the library holds these DT_NOALLOC_SCRATCH_BYTES until the process exits.
namespace dt {
namespace {

static __device__ __align__(256) unsigned char g_noalloc_scratch[DT_NOALLOC_SCRATCH_BYTES];
static __device__ __align__(256) unsigned int g_noalloc_status[64];

// In host code the two names above are host-side stand-ins, not device addresses: the real addresses come
// from cudaGetSymbolAddress, once per device, with that device current.
int noalloc_setup(DeviceState* d) {
  std::lock_guard<std::mutex> lk(g_dev_mu);
  if (!d->noalloc_scratch) {
    void* ps = nullptr;
    void* pst = nullptr;
    DT_CUDA_TRY(cudaGetSymbolAddress(&ps, g_noalloc_scratch));
    DT_CUDA_TRY(cudaGetSymbolAddress(&pst, g_noalloc_status));
    d->noalloc_status = reinterpret_cast<unsigned int*>(pst);
    d->noalloc_scratch = reinterpret_cast<unsigned char*>(ps);
  }
  return DT_OK;
}

}  // namespace
}  // namespace dt

extern "C" int dt_sdpa_decode_noalloc(const dt_sdpa_params* p, void* cuda_stream) {
  using namespace dt;
  // the same argument rules as dt_sdpa_forward (null / misaligned pointers, NaN scale, negative window ...)
  int st = validate_params(p);
  if (st != DT_OK) return st;
  if (p->lse && reinterpret_cast<uintptr_t>(p->lse) % sizeof(float)) return DT_BAD_ARG;
  if (!decode_supported(*p)) return DT_UNSUPPORTED;
  DeviceState* d = device_state();
  if (!d) return DT_NO_DEVICE;
  st = noalloc_setup(d);
  if (st != DT_OK) return st;
  const Scratch scratch{d->noalloc_scratch, (size_t)DT_NOALLOC_SCRATCH_BYTES, d->noalloc_status, true, false, DT_SCRATCH_LIMIT};
  return dispatch_decode(*p, nullptr, scratch, (cudaStream_t)cuda_stream);
}

// Reads and clears the status word of the entry point above: a device-side wait that ran out in one of its
// launches left a non-zero code there.  Copies four bytes into the caller's variable; allocates nothing.
extern "C" int dt_sdpa_decode_noalloc_status(void* cuda_stream, int* code) {
  using namespace dt;
  if (!code) return DT_BAD_ARG;
  DeviceState* d = device_state();
  if (!d) return DT_NO_DEVICE;
  int st = noalloc_setup(d);
  if (st != DT_OK) return st;
  cudaStream_t s = (cudaStream_t)cuda_stream;
  unsigned int h = 0;
  DT_CUDA_TRY(cudaMemcpyAsync(&h, d->noalloc_status, sizeof(h), cudaMemcpyDeviceToHost, s));
  DT_CUDA_TRY(cudaStreamSynchronize(s));
  *code = (int)h;
  if (h) {
    DT_CUDA_TRY(cudaMemsetAsync(d->noalloc_status, 0, sizeof(h), s));
    DT_CUDA_TRY(cudaStreamSynchronize(s));
    return DT_TIMEOUT;
  }
  return DT_OK;
}

#ifdef DT_BRINGUP
// Bring-up builds only: host-made failure for the wait-runs-out test (see DecodeArgs::skip_loads).
extern "C" int dt_internal_set_decode_skip_loads(int on) {
  dt::g_decode_skip_loads = on;
  return 0;
}
// Bring-up builds only: per-CTA timeline buffer for the decode kernel.
extern "C" int dt_internal_set_decode_dump(unsigned long long* device_buffer) {
  dt::g_decode_dbg = device_buffer;
  return 0;
}
#endif
