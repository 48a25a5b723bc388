// Flash-attention forward for sm_100a: TMA-staged Q/K/V tiles, tcgen05.mma with TMEM accumulators,
// warp-specialised online softmax.  Serves the diffusion shapes of the reference
// (Libraries/SwiftDiffusion/Sources/Models/Flux1.swift:224-232 joint attention, Wan.swift:95-131 video
// self-attention, UNetXL.swift:67-185 cross-attention) and the masked text encoders (an additive mask as 4th
// input, alone or with isCausal: Llama.swift:70-73, CLIPTextModel.swift:46-51): fp16/bf16 I/O, fp32 accumulation,
// head dim up to 256, grouped KV heads, optional bottom-right causal rule, BSHD strided views.
//
// One CTA = one (batch, head, pair of 128-row query tiles); at head dim 256 (AuraFlow.swift:358, Gemma3.swift:148,
// Qwen3_5.swift:59-82) one tile, because TMEM holds S and O of only one.  12 warps:
//   warp 0      TMA producer: Q tiles once, then K(j), V(j) blocks of 128 keys through a ring of slots
//   warp 1      MMA issuer (one thread): S_t = Q_t K(j)^T  (operands in shared memory) and
//               O_t += P_t V(j) (P read from TMEM, V from shared memory), interleaved over the two tiles so
//               that the tensor pipe works on one tile while the other tile's softmax runs
//   warp 2      TMEM allocation / release
//   warps 4-7   softmax of tile 0: one thread per query row; reads its S row from TMEM, keeps the running
//               max / sum, rescales O in TMEM only when the max grew by more than 2^8 (the final 1/l
//               normalisation makes the result independent of that choice), writes P as 16-bit back to
//               TMEM over the S columns, and at the end normalises O and stores it
//   warps 8-11  the same for tile 1
// TMEM (512 columns x 128 lanes, fp32): S0 [0,128) S1 [128,256) O0 [256,256+D) O1 [256+D,256+2D).
// Every mbarrier wait is bounded; a wait that runs out stores a code into the device status word and the
// CTA unwinds (TMEM is released on that path too).
#include <stdlib.h>

#include <type_traits>

#include "sm100_ptx.cuh"

namespace dt {
namespace {

constexpr int kBM = 128;       // query rows per tile
constexpr int kBN = 128;       // keys per block
constexpr int kThreads = 384;
constexpr int kHalfBytes = 128 * 128;  // [128 rows][64 x 16-bit] = 16 KB, one TMA box
constexpr float kRescaleThreshold = 8.f;
constexpr int kMaxExtraOutputs = 7;
// every kPolyPeriod-th pair of exponentials is evaluated with the polynomial instead of MUFU.EX2 (1 of 16 pairs with
// period 16).  The softmax warps are bound by the number of instructions they issue, not by the special-function unit
// (measured on B200, Flux shape, TFLOP/s: period 1 (all polynomial) 996, 2: 1066, 3: 1123, 4: 1140, 6: 1157, 8: 1149,
// 16: 1160, none: 1147; with the softmax and the MMA warps free-running, never waiting for each other, the same order)
#ifndef DT_POLY_PERIOD
#define DT_POLY_PERIOD 16
#endif
constexpr int kPolyPeriod = DT_POLY_PERIOD;
// 128 * kRegsLow + 256 * kRegsHigh must not exceed what the CTA was launched with (384 threads * 168)
constexpr int kRegsLow = 80, kRegsHigh = 208;

template <int D, bool kMask = false>
struct Cfg {
  // Query tiles per work item.  TMEM (512 columns) holds S (128 columns) and O (D columns) of two tiles up to
  // D = 128; at D = 256 it holds one tile, whose softmax is run by the first softmax warpgroup alone (the second
  // one idles), and the columns of the second tile's S hold a second S buffer of the same tile: the tensor pipe runs
  // P V(j-1) and Q K(j+1)^T while the softmax works on block j (per key block that tile has twice the tensor-core
  // work of a D = 128 tile under the same softmax, so one warpgroup keeps up).
  static constexpr int kTiles = D == 256 ? 1 : 2;
  static constexpr int kSoftmaxWarps = 4 * kTiles;
  static constexpr int kHalves = D / 64;
  static constexpr int kTileBytes = kHalves * kHalfBytes;  // one Q tile / one K block / one V block
  // the masked variant gives 32 KB of the K/V ring to the second mask staging buffers (D = 256: two 64 KB slots,
  // one K and one V block in flight, and the mask buffers fit beside them)
  static constexpr int kSlots = D == 256 ? 2 : (D == 128 ? 4 : 8) - (kMask ? 32 * 1024 / kTileBytes : 0);
  static constexpr int kMaskBytes = kMask ? kSoftmaxWarps * 32 * 128 : 0;  // per softmax warp: 32 rows x 64 keys x 16-bit (one half block)
  static constexpr int kStageBytes = kSoftmaxWarps * 32 * 128;  // per softmax warp: 32 rows x 64 x 16-bit of O for the TMA store
  static constexpr int kQBufs = D == 64 ? 2 : 1;        // Q buffers: with D = 64 there is room to load the next item's Q early
  static constexpr int kQBytes = kQBufs * kTiles * kTileBytes;
  static constexpr int kRingBytes = kSlots * kTileBytes;
  static constexpr int kBarBytes = 512;
  static constexpr int kSmemBytes = kQBytes + kRingBytes + kStageBytes + kMaskBytes + kBarBytes + 1024;
  static constexpr uint32_t kTmemCols = 512;
  static constexpr uint32_t kColS0 = 0, kColS1 = 128, kColO0 = 256, kColO1 = 256 + D;  // (tile 1's columns: only with kTiles == 2)
};
static_assert(Cfg<256, true>::kSmemBytes <= 227 * 1024, "shared memory of the widest variant");

struct PrefillArgs {
  void* o;
  float* lse;
#ifdef DT_BRINGUP
  float* dbg;   // optional [2][128][128] fp32 dump of the first S block of CTA (0,0,0), or timeline stamps
  int options;  // bit 1: timeline probe of CTA 0 into dbg
#endif
  int64_t o_sb, o_ss, o_sh;
  unsigned int* status;
  int Sq, Sk, Hq, Hkv;
  float scale_log2;
  int is_causal;
  int window;         // sliding window W (0 = off): row i sees keys j > i + (Sk - Sq) - W
  const void* sinks;  // [Hq] attention sinks in the tensors' type, or null
  // additive mask [B or 1, Hq or 1, Sq, Sk] in the tensors' type (kernel variant kMask only): element strides,
  // 0 on a broadcast axis; rows are 16-byte aligned (base and strides multiples of 8 elements)
  const void* mask;
  int64_t m_sb, m_sh, m_sq;
  // one byte per (32 query rows x 64 keys) patch of the mask: non-zero when the patch holds a non-zero entry;
  // [mask batches][mask heads][n_rg row groups][n_kh key halves, padded to an even count]
  const unsigned char* mask_flags;
  int n_rg, n_kh;
  float scale;  // the plain scale (scale_log2 = scale * log2(e)); the masked variant adds the mask in this domain
  int n_qpairs, n_items;  // work items = (batch, head, pair of query tiles)
  int n_slots;            // n_items rounded up to whole rounds over the grid (the causal order leaves some slots empty)
  // variable-length batch (both null otherwise): packed rows, sequence s owns query rows [off_q[s], off_q[s+1])
  // and key rows [off_k[s], off_k[s+1]); the item's batch index is then the sequence
  const int32_t* off_q;
  const int32_t* off_k;
  // head-sharded mode: the same O tile is also stored into these views (other GPUs' output buffers, same
  // strides as o) with ordinary 16-byte stores
  void* extra_o[kMaxExtraOutputs];
  int n_extra;
  int d_real;  // the tensors' head dim (<= the kernel's D): TMA zero-fills the columns beyond it on load and clips them on store
};

struct Barriers {
  uint64_t q_full[2];
  uint64_t q_empty[2];
  uint64_t s_full[2];
  uint64_t o_full[2];  // all P*V of an item done: O may be read (separate from s_full so no barrier runs two phases ahead)
  uint64_t p_half[2][2];  // [tile][first / second 64 keys of P written]
  uint64_t kv_full[8];
  uint64_t kv_empty[8];
  uint64_t pv_done;  // one tile per item: completes once per P V, so that an O rescale can wait for the previous block's
  uint32_t tmem_base;
  int abort_flag;
};

template <typename T>
__device__ __forceinline__ uint32_t pack_pair(float lo, float hi) {
  if constexpr (std::is_same<T, __half>::value) {
    __half2 t = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&t);
  } else {
    __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&t);
  }
}

// S = Q K^T for one 128-row tile: both operands K-major with 128-byte swizzle, D/16 steps of k = 16.
// Descriptor start addresses advance by 32 B per step inside a 64-element half and by 16 KB to the next half.
template <int D>
__device__ __forceinline__ void issue_qk(uint32_t s_tmem, uint64_t q_desc, uint64_t k_desc, uint32_t idesc) {
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    const uint64_t o = (uint64_t)(((ks >> 2) * kHalfBytes + (ks & 3) * 32) >> 4);
    ptx::mma_ss(s_tmem, q_desc + o, k_desc + o, idesc, ks > 0 ? 1u : 0u);
  }
}

// O (+)= P V for one tile: P from TMEM (two 16-bit keys per 32-bit column, 8 columns per step), V is
// [key][d] = MN-major; one step consumes 16 keys = 2 KB of each 64-wide half.
__device__ __forceinline__ void issue_pv(uint32_t o_tmem, uint32_t p_tmem, uint64_t v_desc, uint32_t idesc,
                                         uint32_t accumulate, int k_begin, int k_end) {
  if (k_end - k_begin == 4) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int kk = k_begin + i;
      ptx::mma_ts(o_tmem, p_tmem + kk * 8, v_desc + (uint64_t)(kk * (2048 >> 4)), idesc, (kk > 0) ? 1u : accumulate);
    }
  } else {
#pragma unroll 1
    for (int kk = k_begin; kk < k_end; ++kk)
      ptx::mma_ts(o_tmem, p_tmem + kk * 8, v_desc + (uint64_t)(kk * (2048 >> 4)), idesc, (kk > 0) ? 1u : accumulate);
  }
}

// Experiment builds (-DDT_PREFILL_OPTIONS=bits, never the product): bit 3 = the softmax warps skip the exponentials;
// bit 4 = nobody waits for S or P (free-running softmax and MMA: garbage results, the pure throughput of each
// side); bit 5 = the softmax warps skip the row maximum; bit 6 (with bit 4) = the softmax warps do nothing per block.  Bring-up builds: a.options bit 1 = timeline probe of CTA 0.
#ifndef DT_PREFILL_OPTIONS
#define DT_PREFILL_OPTIONS 0
#endif
#define DT_OPT(bit) ((DT_PREFILL_OPTIONS & (bit)) != 0)
#ifdef DT_BRINGUP
__device__ __forceinline__ void stamp(const PrefillArgs& a, int slot) {
  if ((a.options & 2) && a.dbg != nullptr && blockIdx.x == 0 && slot < 4096)
    reinterpret_cast<unsigned long long*>(a.dbg)[slot] = ptx::globaltimer_ns();
}
#else
__device__ __forceinline__ void stamp(const PrefillArgs&, int) {}
#endif

// Pre-pass of the masked variant: which (32 rows x 64 keys) patches of the additive mask hold anything but zeros.
// A padding mask is zero almost everywhere, and the attention kernel skips the patches flagged zero altogether.
// One warp per patch, 8 lanes on a row's 128 contiguous bytes; entries beyond Sq / Sk are never read.
__global__ void __launch_bounds__(256) mask_flags_kernel(const unsigned short* __restrict__ mask, int64_t m_sb, int64_t m_sh,
                                                         int64_t m_sq, int Hm, int Sq, int Sk, int n_rg, int n_kh,
                                                         int is_causal, unsigned char* __restrict__ flags) {
  const int lane = threadIdx.x & 31;
  const int kh = blockIdx.x * 8 + (threadIdx.x >> 5), rg = blockIdx.y, bh = blockIdx.z;
  if (kh >= n_kh) return;
  const int mb = bh / Hm, mh = bh - mb * Hm;
  const unsigned short* base = mask + mb * m_sb + mh * m_sh;
  const int key = kh * 64 + (lane & 7) * 8;
  uint32_t any = 0u;
  // under the causal rule the attention kernel never visits a patch that lies wholly beyond its rows' last visible key
  const bool visited = !is_causal || (long long)kh * 64 <= (long long)rg * 32 + 31 + (Sk - Sq);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int row = rg * 32 + i * 4 + (lane >> 3);
    if (!visited || row >= Sq || key >= Sk) continue;
    const unsigned short* src = base + (int64_t)row * m_sq + key;
    if (key + 8 <= Sk) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(src));
      any |= v.x | v.y | v.z | v.w;
    } else {
      for (int e = 0; key + e < Sk; ++e) any |= src[e];
    }
  }
  const bool nz = __any_sync(0xffffffffu, any != 0u);
  if (lane == 0) flags[((int64_t)bh * n_rg + rg) * n_kh + kh] = nz ? 1 : 0;
}

// 16-bit pair -> two floats (the mask is stored in the tensors' type)
template <typename T>
__device__ __forceinline__ float2 unpack_pair(uint32_t x) {
  if constexpr (std::is_same<T, __half>::value) return __half22float2(*reinterpret_cast<const __half2*>(&x));
  else return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&x));
}

template <typename T, int D, bool kMask>
__global__ void __launch_bounds__(kThreads, 1)
prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_o,
                       const PrefillArgs a) {
  using C = Cfg<D, kMask>;
  constexpr int kBf16 = std::is_same<T, __half>::value ? 0 : 1;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw);
  const uint32_t q_smem = base;
  const uint32_t ring_smem = base + C::kQBytes;
  const uint32_t stage_smem = base + C::kQBytes + C::kRingBytes;
  // masked variant: [second mask staging buffers] between the O staging rows and the barriers
  const uint32_t mask_smem = stage_smem + C::kStageBytes;
  Barriers* bars = reinterpret_cast<Barriers*>(base_ptr + C::kQBytes + C::kRingBytes + C::kStageBytes + C::kMaskBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = a.Hq / a.Hkv;

  // Work items (batch, head, pair of query tiles), q-tile pair fastest so that CTAs running at the same
  // time share one head's K/V in L2.  The CTA is persistent: it takes items blockIdx.x, + gridDim.x, ...
  struct Item {
    int b, h, kvh, q0, nkv, j0;  // K/V blocks j0 .. j0 + nkv - 1; nkv == 0: nothing to do (q0 beyond the sequence)
    int sq, sk, off;             // rows of this (batch item | sequence); causal: key j visible to query i iff j <= i + off
    int qrow, krow;              // first packed row of the sequence (0 unless variable-length)
    bool two;
  };
  auto decode_item = [&](int item) {
    Item it;
    int qt = item % a.n_qpairs;
    int bh = item / a.n_qpairs;
    if (a.is_causal) {
      // Under the causal rule an item's work grows with its query position.  The items are dealt out heaviest
      // first (all heads' last tile pair, then the one before, ...), forwards in even rounds over the CTAs and
      // backwards in odd rounds, so that every CTA's items add up to about the same number of K/V blocks.
      const int round = item / (int)gridDim.x;
      int pos = item - round * (int)gridDim.x;
      if (round & 1) pos = (int)gridDim.x - 1 - pos;
      const int order = round * (int)gridDim.x + pos;
      const int nbh = a.n_items / a.n_qpairs;
      const int level = order / nbh;
      bh = order - level * nbh;
      qt = a.n_qpairs - 1 - level;
      if (order >= a.n_items) {  // a slot of the last, incomplete round without an item
        it = Item{};
        it.nkv = 0;
        return it;
      }
    }
    it.h = bh % a.Hq;
    it.b = bh / a.Hq;
    it.kvh = it.h / G;
    it.q0 = qt * (C::kTiles * kBM);
    it.sq = a.Sq;
    it.sk = a.Sk;
    it.qrow = it.krow = 0;
    if (a.off_q) {
      it.qrow = a.off_q[it.b];
      it.krow = a.off_k[it.b];
      it.sq = a.off_q[it.b + 1] - it.qrow;
      it.sk = a.off_k[it.b + 1] - it.krow;
      it.b = 0;
    }
    it.off = it.sk - it.sq;
    it.two = C::kTiles == 2 && it.q0 + kBM < it.sq;
    it.j0 = 0;
    if (it.q0 >= it.sq) {  // only with variable lengths: this sequence is shorter than the longest one
      it.nkv = 0;
      return it;
    }
    int nkv = max(1, (it.sk + kBN - 1) / kBN);  // a sequence without keys still runs one (fully masked) block
    if (a.is_causal) {
      const int last_row = min(it.sq, it.q0 + C::kTiles * kBM) - 1;
      const long long lim = (long long)last_row + it.off + 1;  // keys [0, lim) can be visible
      const int need = (int)((max(0LL, min((long long)it.sk, lim)) + kBN - 1) / kBN);
      nkv = max(1, min(nkv, need));
    }
    if (a.window > 0) {  // blocks entirely below the first row's window are never visited
      const long long lo = (long long)it.q0 + it.off - a.window + 1;
      it.j0 = (int)min((long long)(nkv - 1), max(0LL, lo) / kBN);
    }
    it.nkv = nkv - it.j0;
    return it;
  };

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(&bars->q_full[i], 1);
      ptx::mbar_init(&bars->q_empty[i], 1);
    }
    for (int t = 0; t < 2; ++t) {
      ptx::mbar_init(&bars->s_full[t], 1);
      ptx::mbar_init(&bars->o_full[t], 1);
      ptx::mbar_init(&bars->p_half[t][0], 4);  // one arrival per softmax warp
      ptx::mbar_init(&bars->p_half[t][1], 4);
    }
    for (int i = 0; i < C::kSlots; ++i) {
      ptx::mbar_init(&bars->kv_full[i], 1);
      ptx::mbar_init(&bars->kv_empty[i], 1);
    }
    ptx::mbar_init(&bars->pv_done, 1);
    bars->abort_flag = 0;
    ptx::fence_mbar_init();
  }
  if (warp == 2) {
    ptx::tmem_alloc(&bars->tmem_base, C::kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = bars->tmem_base;
  volatile int* abort_flag = &bars->abort_flag;

  // Register budget: the data-movement warpgroup gives registers back, the softmax warpgroups take them.
  // (Each setmaxnreg must dominate the code it governs, hence the nesting.)
  if (warp < 4) {
    ptx::setmaxnreg_dec<kRegsLow>();
    if (warp == 0) {
      // =========================== TMA producer ===========================
      if (lane == 0) {
        ptx::prefetch_tensormap(&map_q);
        ptx::prefetch_tensormap(&map_k);
        ptx::prefetch_tensormap(&map_v);
        ptx::prefetch_tensormap(&map_o);
        int ring_it = 0;  // K/V ring position, continues across items
        int n_item = 0;
        bool ok = true;
        auto load_kv = [&](const Item& w, int j, bool is_v) {
          const int slot = ring_it % C::kSlots, use = ring_it / C::kSlots;
          if (use > 0 && !ptx::mbar_wait(&bars->kv_empty[slot], (use - 1) & 1, abort_flag)) {
            atomicCAS(a.status, 0u, 2u);
            *abort_flag = 1;
            return false;
          }
          ptx::mbar_arrive_expect_tx(&bars->kv_full[slot], (uint32_t)C::kTileBytes);
#pragma unroll
          for (int hf = 0; hf < C::kHalves; ++hf)
            ptx::tma_load_4d(base_ptr + C::kQBytes + slot * C::kTileBytes + hf * kHalfBytes, is_v ? &map_v : &map_k,
                             &bars->kv_full[slot], hf * 64, w.kvh, w.krow + (w.j0 + j) * kBN, w.b);
          ++ring_it;
          return true;
        };
        for (int item = blockIdx.x; item < a.n_slots && ok; item += gridDim.x, ++n_item) {
          const Item w = decode_item(item);
          if (w.nkv == 0) {  // empty item: not counted (the loop header increments n_item)
            --n_item;
            continue;
          }
          // The Q tiles of the NEXT item are pulled into L2 now: their rows are 256-byte pieces a whole
          // token stride apart (slow to gather from HBM), and the real load sits on the critical path
          // between two items.
          if (item + (int)gridDim.x < a.n_slots) {
            const Item nx = decode_item(item + gridDim.x);
            for (int t = 0; t < (nx.two ? 2 : 1); ++t)
#pragma unroll
              for (int hf = 0; hf < C::kHalves; ++hf)
                if (nx.nkv > 0) ptx::tma_prefetch_l2_4d(&map_q, hf * 64, nx.h, nx.qrow + nx.q0 + t * kBM, nx.b);
          }
          // first K/V block of this item may be fetched while the previous item still owns the Q buffers
          // (one tile per item: the MMA warp consumes K(0), K(1), V(0), K(2), V(1), ..., and the ring follows that order)
          if constexpr (C::kTiles == 1) ok = load_kv(w, 0, false) && (w.nkv == 1 || load_kv(w, 1, false));
          else ok = load_kv(w, 0, false) && load_kv(w, 0, true);
          if (!ok) break;
          const int qb = n_item % C::kQBufs, quse = n_item / C::kQBufs;
          if (quse > 0 && !ptx::mbar_wait(&bars->q_empty[qb], (quse - 1) & 1, abort_flag)) {
            atomicCAS(a.status, 0u, 2u);
            *abort_flag = 1;
            break;
          }
          stamp(a, 16 * n_item + 0);
          ptx::mbar_arrive_expect_tx(&bars->q_full[qb], (uint32_t)((w.two ? 2 : 1) * C::kTileBytes));
          for (int t = 0; t < (w.two ? 2 : 1); ++t)
#pragma unroll
            for (int hf = 0; hf < C::kHalves; ++hf)
              ptx::tma_load_4d(base_ptr + (qb * C::kTiles + t) * C::kTileBytes + hf * kHalfBytes, &map_q, &bars->q_full[qb], hf * 64,
                               w.h, w.qrow + w.q0 + t * kBM, w.b);
          if constexpr (C::kTiles == 1) {
            for (int j = 0; j < w.nkv && ok; ++j) ok = load_kv(w, j, true) && (j + 2 >= w.nkv || load_kv(w, j + 2, false));
          } else {
            for (int j = 1; j < w.nkv && ok; ++j) ok = load_kv(w, j, false) && load_kv(w, j, true);
          }
        }
      }
    } else if (warp == 1) {
      // =========================== MMA issuer ===========================
      if (lane == 0) {
        constexpr uint32_t idesc_qk = ptx::make_idesc_f16(kBf16, kBM, kBN, 0, 0);
        constexpr uint32_t idesc_pv = ptx::make_idesc_f16(kBf16, kBM, D, 0, 1);
        // Descriptors differ only in the 14-bit start-address field, so stepping through a tile is one add.
        const uint64_t desc_k_major = ptx::make_smem_desc_sw128(0, 16, 1024);            // Q, K
        const uint64_t desc_mn_major = ptx::make_smem_desc_sw128(0, kHalfBytes, 1024);   // V
        const uint64_t qd_base = desc_k_major | (uint64_t)((q_smem & 0x3FFFFu) >> 4);
        const uint64_t ring_k = desc_k_major | (uint64_t)((ring_smem & 0x3FFFFu) >> 4);
        const uint64_t ring_v = desc_mn_major | (uint64_t)((ring_smem & 0x3FFFFu) >> 4);
        const uint32_t s0 = tmem + C::kColS0, s1 = tmem + C::kColS1, o0 = tmem + C::kColO0, o1 = tmem + C::kColO1;
        int slot = 0, par = 0;     // ring position of the next K/V block to consume
        uint32_t pph0 = 0, pph1 = 0;  // phases of the P hand-off barriers, per tile
        int n_item = 0;
        bool ok = true;
        auto fail = [&](unsigned code) {
          atomicCAS(a.status, 0u, code);
          *abort_flag = 1;
          ok = false;
        };
        auto advance = [&]() {
          if (++slot == C::kSlots) { slot = 0; par ^= 1; }
        };
        for (int item = blockIdx.x; item < a.n_slots && ok; item += gridDim.x, ++n_item) {
          const Item w = decode_item(item);
          if (w.nkv == 0) {  // empty item: not counted (the loop header increments n_item)
            --n_item;
            continue;
          }
          const int ntile = w.two ? 2 : 1;
          const int qb = n_item % C::kQBufs;
          const uint64_t qd0 = qd_base + (uint64_t)(qb * C::kTiles * (C::kTileBytes >> 4));
          const uint64_t qd1 = qd0 + (uint64_t)(C::kTileBytes >> 4);
          if constexpr (C::kTiles == 1) {
            // One tile per item (D = 256): S is double-buffered in TMEM (the columns a second tile would use), so that
            // Q K(j+1)^T and P V(j-1) run while the softmax works on block j.  Order on the tensor pipe:
            // QK(0) QK(1) | PV(0) QK(2) | PV(1) QK(3) | ...
            if (!ptx::mbar_wait(&bars->q_full[qb], (n_item / C::kQBufs) & 1, abort_flag)) {
              fail(1u);
              break;
            }
            auto qk = [&](int i) -> bool {  // S[i & 1] = Q K(i)^T from the ring's next slot
              if (!ptx::mbar_wait(&bars->kv_full[slot], par, abort_flag)) {
                fail(1u);
                return false;
              }
              ptx::tc_fence_after();
              issue_qk<D>((i & 1) ? s1 : s0, qd0, ring_k + (uint64_t)(slot * (C::kTileBytes >> 4)), idesc_qk);
              ptx::tc_commit(&bars->s_full[i & 1]);
              ptx::tc_commit(&bars->kv_empty[slot]);
              if (i == w.nkv - 1) ptx::tc_commit(&bars->q_empty[qb]);  // Q is no longer needed: the next item may load its own
              advance();
              return true;
            };
            if (!qk(0) || (w.nkv > 1 && !qk(1))) break;
            for (int j = 0; j < w.nkv && ok; ++j) {
              const int b = j & 1;
              const uint32_t sb = b ? s1 : s0;
              uint32_t& pph = b ? pph1 : pph0;
              const int valid = max(16, min(kBN, w.sk - (w.j0 + j) * kBN));
              const int ksteps = (valid + 15) >> 4;
              const int k_mid = min(ksteps, 4);
              if (!ptx::mbar_wait(&bars->kv_full[slot], par, abort_flag)) {  // V(j)
                fail(1u);
                break;
              }
              const int slot_v = slot;
              const uint64_t vd = ring_v + (uint64_t)(slot_v * (C::kTileBytes >> 4));
              advance();
              if (!ptx::mbar_wait(&bars->p_half[b][0], pph, abort_flag)) { fail(4u); break; }
              ptx::tc_fence_after();
              issue_pv(o0, sb, vd, idesc_pv, j > 0 ? 1u : 0u, 0, k_mid);
              if (!ptx::mbar_wait(&bars->p_half[b][1], pph, abort_flag)) { fail(4u); break; }
              pph ^= 1;
              ptx::tc_fence_after();
              issue_pv(o0, sb, vd, idesc_pv, 1u, k_mid, ksteps);
              ptx::tc_commit(&bars->kv_empty[slot_v]);
              ptx::tc_commit(&bars->pv_done);
              if (j + 2 < w.nkv && !qk(j + 2)) break;  // overwrites the S / P columns the P V above has just read
              if (j + 1 == w.nkv) ptx::tc_commit(&bars->o_full[0]);
            }
            continue;
          }
          // ---- S_t(0) = Q_t K(0)^T ----
          stamp(a, 16 * n_item + 5);
          if (!ptx::mbar_wait(&bars->q_full[qb], (n_item / C::kQBufs) & 1, abort_flag)) {
            fail(1u);
            break;
          }
          stamp(a, 16 * n_item + 6);
          if (!ptx::mbar_wait(&bars->kv_full[slot], par, abort_flag)) {
            fail(1u);
            break;
          }
          stamp(a, 16 * n_item + 1);
          ptx::tc_fence_after();
          {
            const uint64_t kd = ring_k + (uint64_t)(slot * (C::kTileBytes >> 4));
            issue_qk<D>(s0, qd0, kd, idesc_qk);
            ptx::tc_commit(&bars->s_full[0]);
            if (ntile == 2) {
              issue_qk<D>(s1, qd1, kd, idesc_qk);
              ptx::tc_commit(&bars->s_full[1]);
            }
            ptx::tc_commit(&bars->kv_empty[slot]);
            if (w.nkv == 1) ptx::tc_commit(&bars->q_empty[qb]);  // Q is no longer needed: the next item may load its own
            advance();
          }
          for (int j = 0; j < w.nkv && ok; ++j) {
            const int slot_v = slot, par_v = par;
            advance();
            const int slot_k = slot, par_k = par;
            const bool more = j + 1 < w.nkv;
            if (more) advance();
            const int valid = max(16, min(kBN, w.sk - (w.j0 + j) * kBN));  // at least one 16-key step (P = 0 there if sk = 0)
            const int ksteps = (valid + 15) >> 4;
            const int k_mid = min(ksteps, 4);
            if (!ptx::mbar_wait(&bars->kv_full[slot_v], par_v, abort_flag) ||
                (more && !ptx::mbar_wait(&bars->kv_full[slot_k], par_k, abort_flag))) {
              fail(1u);
              break;
            }
            const uint64_t vd = ring_v + (uint64_t)(slot_v * (C::kTileBytes >> 4));
            const uint64_t kd = ring_k + (uint64_t)(slot_k * (C::kTileBytes >> 4));
            const bool last_qk = more && (j + 2 == w.nkv);  // the QK issued in this iteration is the item's last
            // ---- tile 0 ----  (P arrives in two halves of 64 keys so P*V starts while the softmax still runs)
            if (!DT_OPT(16) && !ptx::mbar_wait(&bars->p_half[0][0], pph0, abort_flag)) { fail(4u); break; }
            if (j == 0) stamp(a, 16 * n_item + 2);
            ptx::tc_fence_after();
            issue_pv(o0, s0, vd, idesc_pv, j > 0 ? 1u : 0u, 0, k_mid);
            if (!DT_OPT(16) && !ptx::mbar_wait(&bars->p_half[0][1], pph0, abort_flag)) { fail(4u); break; }
            pph0 ^= 1;
            ptx::tc_fence_after();
            issue_pv(o0, s0, vd, idesc_pv, 1u, k_mid, ksteps);
            if (ntile == 1) ptx::tc_commit(&bars->kv_empty[slot_v]);
            if (more) issue_qk<D>(s0, qd0, kd, idesc_qk);
            ptx::tc_commit(more ? &bars->s_full[0] : &bars->o_full[0]);  // next S ready, or (last block) O complete
            if (!more) stamp(a, 16 * n_item + 3);
            if (more && ntile == 1) {
              ptx::tc_commit(&bars->kv_empty[slot_k]);
              if (last_qk) ptx::tc_commit(&bars->q_empty[qb]);
            }
            // ---- tile 1 ----
            if (ntile == 2) {
              if (!DT_OPT(16) && !ptx::mbar_wait(&bars->p_half[1][0], pph1, abort_flag)) { fail(4u); break; }
              ptx::tc_fence_after();
              issue_pv(o1, s1, vd, idesc_pv, j > 0 ? 1u : 0u, 0, k_mid);
              if (!DT_OPT(16) && !ptx::mbar_wait(&bars->p_half[1][1], pph1, abort_flag)) { fail(4u); break; }
              pph1 ^= 1;
              ptx::tc_fence_after();
              issue_pv(o1, s1, vd, idesc_pv, 1u, k_mid, ksteps);
              ptx::tc_commit(&bars->kv_empty[slot_v]);
              if (more) issue_qk<D>(s1, qd1, kd, idesc_qk);
              ptx::tc_commit(more ? &bars->s_full[1] : &bars->o_full[1]);
              if (more) {
                ptx::tc_commit(&bars->kv_empty[slot_k]);
                if (last_qk) ptx::tc_commit(&bars->q_empty[qb]);
              }
            }
          }
        }
      }
    }
  } else {
    ptx::setmaxnreg_inc<kRegsHigh>();
    // =========================== softmax / correction / epilogue ===========================
    const int t = (warp - 4) >> 2;  // tile
    const int row_in_tile = ((warp & 3) << 5) + lane;
    const uint32_t lane_addr = (uint32_t)((warp & 3) << 5) << 16;
    uint32_t t_s = tmem + (t ? C::kColS1 : C::kColS0) + lane_addr;  // (one tile per item: S alternates between the two)
    const uint32_t t_o = tmem + (t ? C::kColO1 : C::kColO0) + lane_addr;
    uint32_t sph = 0, sph_b = 0, oph = 0;  // phases of s_full[] / o_full[t], continue across items
    bool ok = true;
#ifdef DT_BRINGUP
    bool first_dump = true;
#endif
    int n_item = 0;
    uint32_t n_blocks = 0;  // K/V blocks this warpgroup has handed over so far, over all items (one tile per item)
    const bool probe = (warp == 4 && lane == 0);

    for (int item = blockIdx.x; item < a.n_slots && ok; item += gridDim.x) {
      const Item w = decode_item(item);
      if (w.nkv == 0) continue;
      if (t == 1 && !w.two) continue;  // this item has no second tile: neither side touches tile 1's barriers
      const int row = w.q0 + t * kBM + row_in_tile;
      const long long vis = a.is_causal ? (long long)row + w.off : (long long)w.sk;  // last visible key
      const long long lo = a.window > 0 ? (long long)row + w.off - a.window + 1 : 0;  // first visible key
      float m_used = -INFINITY, l = 0.f;
      // masked variant: this warp's row of patch flags (null when its 32 rows lie beyond Sq: nothing to add there)
      const unsigned char* patch_flags = nullptr;
      if constexpr (kMask) {
        const int rg = (w.q0 + t * kBM + ((warp & 3) << 5)) >> 5;
        if (rg < a.n_rg) {
          const int64_t mb = a.m_sb ? w.b : 0, mh = a.m_sh ? w.h : 0;
          const int64_t hm = a.m_sh ? a.Hq : 1;
          patch_flags = a.mask_flags + ((mb * hm + mh) * a.n_rg + rg) * a.n_kh;
        }
      }
      // flags of block jj: bit 0 = its first 64 keys carry mask values, bit 1 = its second 64 keys
      auto block_flags = [&](int jj) -> uint32_t {
        if (!kMask || patch_flags == nullptr || jj >= w.nkv) return 0u;
        const uint32_t f = __ldg(reinterpret_cast<const unsigned short*>(patch_flags + 2 * (w.j0 + jj)));
        return ((f & 0xffu) ? 1u : 0u) | ((f >> 8) ? 2u : 0u);
      };
      uint32_t flags_cur = block_flags(0);

      for (int j = 0; j < (DT_OPT(64) ? 0 : w.nkv); ++j) {  // (experiment bit 6: no softmax work at all)
        const uint32_t flags_next = block_flags(j + 1);  // asked for early, used when the next block's mask is requested
        // Masked variant: the warp's 32 rows x 128 mask values of a block travel global -> shared memory with
        // asynchronous 16-byte copies, 8 lanes on one row's 128 contiguous bytes (whole cache lines; a lane fetching its
        // own row's 256 bytes would touch 32 lines per instruction and that made the L1 the bottleneck), in two halves
        // of 64 keys with a staging buffer each: the first one in this warp's O staging rows (idle until the epilogue), the
        // second one in the area taken from the K/V ring.  A block's halves are requested one block ahead; rows beyond Sq
        // and keys beyond Sk are zero-filled, never read.
        auto mask_prefetch = [&](int jj, int half, uint32_t flags) {
          if constexpr (kMask) {
            if (jj < w.nkv && ((flags >> half) & 1u)) {  // patches without mask values are not even fetched
              const int keyh = (w.j0 + jj) * kBN + half * 64;
              const uint32_t buf = (half ? mask_smem : stage_smem) + (uint32_t)(warp - 4) * (32 * 128);
              const T* mbase = reinterpret_cast<const T*>(a.mask) + (int64_t)w.b * a.m_sb + (int64_t)w.h * a.m_sh + keyh;
              const int ch = lane & 7;
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const int r = i * 4 + (lane >> 3);  // row within the warp's 32
                const int grow = w.q0 + t * kBM + ((warp & 3) << 5) + r;
                const int left = grow < w.sq ? w.sk - (keyh + ch * 8) : 0;  // mask entries from this chunk's first key on
                const int nbytes = left >= 8 ? 16 : (left > 0 ? left * 2 : 0);
                ptx::cp_async_16(buf + (uint32_t)r * 128 + (((uint32_t)ch ^ ((uint32_t)r & 7u)) << 4),
                                 nbytes ? (const void*)(mbase + (int64_t)grow * a.m_sq + ch * 8) : (const void*)a.mask, nbytes);
              }
            }
            ptx::cp_async_commit();  // always a group, possibly empty, so that the wait counts stay regular
          }
        };
        if constexpr (kMask) {
          if (j == 0) {
            // the O staging rows double as the first mask buffer: the previous item's TMA store must have read them
            if (lane == 0) ptx::bulk_wait_read_all();
            __syncwarp();
            mask_prefetch(0, 0, flags_cur);
            mask_prefetch(0, 1, flags_cur);
          }
        }
        // S buffer of this block: the tile's own, or (one tile per item) the two buffers in turn
        const int sb = C::kTiles == 1 ? (j & 1) : t;
        if constexpr (C::kTiles == 1) t_s = tmem + (sb ? C::kColS1 : C::kColS0) + lane_addr;
        uint32_t& sph_cur = (C::kTiles == 1 && sb) ? sph_b : sph;
        if (!DT_OPT(16) && !__all_sync(0xffffffffu, ptx::mbar_wait(&bars->s_full[sb], sph_cur, abort_flag))) {
          atomicCAS(a.status, 0u, 3u);
          *abort_flag = 1;
          ok = false;
          break;
        }
        sph_cur ^= 1;
        if (probe && j == 0) stamp(a, 16 * n_item + 8);
        ptx::tc_fence_after();
        uint32_t s[4][32];
        if constexpr (kMask) {
          // scores in two halves of 64 keys; each half gets mask / scale added once its mask values have landed (the
          // scores stay in the unscaled domain of the unmasked kernel).  A half whose mask values are all zero for the
          // whole warp -- most of a padding mask -- is left as it is.
          const uint64_t inv2 = ptx::pack_f32x2(1.f / a.scale, 1.f / a.scale);
          auto add_mask_half = [&](int half) {
            if (!((flags_cur >> half) & 1u)) return;  // the same answer for the whole warp
            const uint32_t buf = (half ? mask_smem : stage_smem) + (uint32_t)(warp - 4) * (32 * 128) + (uint32_t)lane * 128;
            uint4 mk[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) mk[q] = ptx::ld_shared_v4(buf + ((((uint32_t)q) ^ ((uint32_t)lane & 7u)) << 4));
            uint32_t any = 0u;
#pragma unroll
            for (int q = 0; q < 8; ++q) any |= mk[q].x | mk[q].y | mk[q].z | mk[q].w;
            if (__any_sync(0xffffffffu, any != 0u)) {
#pragma unroll
              for (int q = 0; q < 8; ++q) {
                const uint32_t mw[4] = {mk[q].x, mk[q].y, mk[q].z, mk[q].w};
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                  const float2 mf = unpack_pair<T>(mw[u]);
                  const int c = half * 2 + (q >> 2), i = (q & 3) * 8 + u * 2;
                  const uint64_t r2 = ptx::fma_f32x2(ptx::pack_f32x2(mf.x, mf.y), inv2,
                                                     ptx::pack_f32x2(__uint_as_float(s[c][i]), __uint_as_float(s[c][i + 1])));
                  float r0, r1;
                  ptx::unpack_f32x2(r2, r0, r1);
                  s[c][i] = __float_as_uint(r0);
                  s[c][i + 1] = __float_as_uint(r1);
                }
              }
            }
            __syncwarp();  // every lane has read its row: the buffer may be refilled
          };
          ptx::tmem_ld32(t_s + 0, s[0]);
          ptx::tmem_ld32(t_s + 32, s[1]);
          ptx::cp_async_wait<1>();  // this block's first half has landed (its second half may still be on its way)
          __syncwarp();
          ptx::tc_wait_ld();
          add_mask_half(0);
          mask_prefetch(j + 1, 0, flags_next);
          ptx::tmem_ld32(t_s + 64, s[2]);
          ptx::tmem_ld32(t_s + 96, s[3]);
          ptx::cp_async_wait<1>();  // this block's second half (the group behind it is the next block's first half)
          __syncwarp();
          ptx::tc_wait_ld();
          add_mask_half(1);
          mask_prefetch(j + 1, 1, flags_next);
          flags_cur = flags_next;
        } else {
          ptx::tmem_ld32(t_s + 0, s[0]);
          ptx::tmem_ld32(t_s + 32, s[1]);
          ptx::tmem_ld32(t_s + 64, s[2]);
          ptx::tmem_ld32(t_s + 96, s[3]);
          ptx::tc_wait_ld();
        }
        const float sl2 = a.scale_log2;
        if (probe && j == 0) stamp(a, 16 * n_item + 4);

#ifdef DT_BRINGUP
        if (a.dbg != nullptr && !(a.options & 2) && first_dump && j == 0 && blockIdx.x == 0) {
          float* dst = a.dbg + ((size_t)t * kBM + row_in_tile) * kBN;
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int i = 0; i < 32; ++i) dst[c * 32 + i] = __uint_as_float(s[c][i]);
        }
        first_dump = false;
#endif

        const int key0 = (w.j0 + j) * kBN;
        const bool need_mask = (key0 + kBN > w.sk) || (a.is_causal && (long long)(key0 + kBN - 1) > vis) || (long long)key0 < lo;
        // chunks of 32 keys that lie entirely beyond Sk are skipped (short K/V such as 77 text tokens)
        const int nch = max(1, (min(kBN, w.sk - key0) + 31) >> 5);  // at least the chunk the MMA warp always reads
        if (need_mask) {
          // bounds relative to this block as 32-bit values, so that each element costs one compare against a
          // constant: columns hi_rel+1 .. 127 and 0 .. lo_rel-1 are hidden
          const long long lim = min((long long)w.sk - 1, vis);  // keys <= lim visible
          const int hi_rel = (int)max(-1LL, min(lim - key0, (long long)(kBN - 1)));
          const int lo_rel = (int)max(0LL, min(lo - key0, (long long)kBN));
          if (lo_rel == 0) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              if (c >= nch || (c + 1) * 32 - 1 <= hi_rel) continue;  // chunk never read, or entirely visible
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (c * 32 + i > hi_rel) s[c][i] = 0xff800000u;  // -inf
            }
          } else {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              if (c >= nch) continue;
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (c * 32 + i > hi_rel || c * 32 + i < lo_rel) s[c][i] = 0xff800000u;  // -inf
            }
          }
        }
        if (probe && j == 0) stamp(a, 16 * n_item + 12);
        // row max: four independent chains of 3-input max (one per 32-column chunk)
        float mxc[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          if (c >= nch) {
            mxc[c] = -INFINITY;
            continue;
          }
          mxc[c] = ptx::max3(__uint_as_float(s[c][0]), __uint_as_float(s[c][1]), __uint_as_float(s[c][2]));
#pragma unroll
          for (int i = 3; i < 31; i += 2) mxc[c] = ptx::max3(mxc[c], __uint_as_float(s[c][i]), __uint_as_float(s[c][i + 1]));
          mxc[c] = fmaxf(mxc[c], __uint_as_float(s[c][31]));
        }
        float mx = fmaxf(fmaxf(mxc[0], mxc[1]), fmaxf(mxc[2], mxc[3]));
        if (DT_OPT(32)) mx = __uint_as_float(s[0][0]);  // bring-up: no row maximum
        mx *= sl2;  // scale > 0 is a precondition of this kernel
        const float m_cand = fmaxf(m_used, mx);
        // Lazy rescale: keep the old reference max unless the new one is larger by more than the threshold.
        const bool grow = (m_cand - m_used > kRescaleThreshold) || (m_used == -INFINITY && m_cand != -INFINITY);
        if (__any_sync(0xffffffffu, grow)) {
          const float m_new = grow ? m_cand : m_used;
          const float alpha = (m_new == -INFINITY) ? 1.f : fast_exp2(m_used - m_new);
          l *= alpha;
          m_used = m_new;
          if (j > 0) {
            if constexpr (C::kTiles == 1) {
              // With S double-buffered this block's scores arrive before the previous block's P V has run: O may only
              // be touched once that one has retired.  (It cannot be more than one phase behind: the P V of this block
              // waits for the P written below.)
              if (!__all_sync(0xffffffffu, ptx::mbar_wait(&bars->pv_done, (n_blocks - 1) & 1u, abort_flag))) {
                atomicCAS(a.status, 0u, 7u);
                *abort_flag = 1;
                ok = false;
                break;
              }
              ptx::tc_fence_after();
            }
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
              uint32_t ov[32];
              ptx::tmem_ld32(t_o + c * 32, ov);
              ptx::tc_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
              ptx::tmem_st32(t_o + c * 32, ov);
            }
          }
        }
        // p = exp2(s * scale_log2 - m): packed fp32x2 multiply-add, packed row sums in four independent
        // accumulators, packed conversion to the 16-bit P the second MMA reads from TMEM
        if (probe && j == 0) stamp(a, 16 * n_item + 13);
        const float neg_m = (m_used == -INFINITY) ? 0.f : -m_used;
        const uint64_t neg_m2 = ptx::pack_f32x2(neg_m, neg_m);
        const uint64_t scale2 = ptx::pack_f32x2(sl2, sl2);
        uint64_t lsum[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          lsum[c] = 0ull;
          if (c < nch) {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const uint64_t x2 = ptx::fma_f32x2(ptx::pack_f32x2(__uint_as_float(s[c][2 * i]), __uint_as_float(s[c][2 * i + 1])),
                                               scale2, neg_m2);
            float p0, p1;
            if (DT_OPT(8)) {  // bring-up: no exponentials
              ptx::unpack_f32x2(x2, p0, p1);
            } else if ((i % kPolyPeriod) == kPolyPeriod - 1) {  // a share of the exponentials runs on the FMA pipes
              ptx::exp2_poly_x2(x2, p0, p1);
            } else {
              float x0, x1;
              ptx::unpack_f32x2(x2, x0, x1);
              p0 = fast_exp2(x0);
              p1 = fast_exp2(x1);
            }
            lsum[c] = ptx::add_f32x2(lsum[c], ptx::pack_f32x2(p0, p1));
            // the packed pair goes into the register score i of this chunk came in (scores 2i and 2i+1 are used up)
            if constexpr (kBf16 != 0) ptx::cvt_pack_bf16_into(s[c][i], p0, p1);
            else ptx::cvt_pack_f16_into(s[c][i], p0, p1);
          }
          ptx::tmem_st16(t_s + c * 16, s[c]);
          }
          if (c == 1 || c == 3) {  // 64 keys of P are in TMEM: let the MMA warp start on them
            ptx::tc_wait_st();
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&bars->p_half[sb][c >> 1]);
            if (probe && j == 0) stamp(a, 16 * n_item + 14 + (c >> 1));
          }
        }
        {
          float a0, a1, b0, b1;
          ptx::unpack_f32x2(ptx::add_f32x2(lsum[0], lsum[1]), a0, a1);
          ptx::unpack_f32x2(ptx::add_f32x2(lsum[2], lsum[3]), b0, b1);
          l += (a0 + a1) + (b0 + b1);
        }
        ++n_blocks;
      }
      if (!ok) break;
      if (probe) stamp(a, 16 * n_item + 9);

      // ---- epilogue: O / l -> global (the MMA warp already works on the next item's first S meanwhile) ----
      if (!DT_OPT(16) && !__all_sync(0xffffffffu, ptx::mbar_wait(&bars->o_full[t], oph, abort_flag))) {
        atomicCAS(a.status, 0u, 5u);
        *abort_flag = 1;
        ok = false;
        break;
      }
      oph ^= 1;
      if (probe) stamp(a, 16 * n_item + 10);
      ptx::tc_fence_after();
      if (a.sinks && row < w.sq) {
        // attention sink: one more score without a value row joins the denominator (l and O are relative to m_used)
        const float sl = to_float(reinterpret_cast<const T*>(a.sinks)[w.h]) * kLog2e;
        if (m_used == -INFINITY) {
          m_used = sl;
          l = 1.f;
        } else {
          l += fast_exp2(sl - m_used);
        }
      }
      // a row that never saw a visible key (m_used still -inf) yields zeros, whatever the masked entries summed to
      const float inv = (l > 0.f && m_used != -INFINITY) ? 1.f / l : 0.f;
      // O goes out through shared memory and a TMA store per warp (32 rows x 64 columns): whole 128-byte
      // row pieces reach L2, instead of 16-byte pieces scattered over 32 rows per instruction.
      {
        const uint32_t my_stage = stage_smem + (uint32_t)(warp - 4) * (32 * 128);
        const int wrow0 = w.q0 + t * kBM + ((warp & 3) << 5);
        // The tensor map clips at the end of the tensor, not at the end of a packed sequence: with variable
        // lengths a warp whose 32 rows reach past its sequence stores row by row instead.
        const bool tma_ok = a.off_q ? (wrow0 + 32 <= w.sq) : (wrow0 < w.sq);
        const bool guarded_main = a.off_q != nullptr && wrow0 < w.sq && !tma_ok;
#pragma unroll
        for (int hf = 0; hf < D / 64; ++hf) {
          // the previous TMA store of this warp (last half, or the previous item) must have read the staging rows
          // before they are overwritten: waited for here, as late as possible, not right after issuing it
          if (lane == 0) ptx::bulk_wait_read_all();
          __syncwarp();
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            uint32_t ov[32];
            ptx::tmem_ld32(t_o + hf * 64 + c * 32, ov);
            ptx::tc_wait_ld();
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint4 pk;
              pk.x = pack_pair<T>(__uint_as_float(ov[v * 8 + 0]) * inv, __uint_as_float(ov[v * 8 + 1]) * inv);
              pk.y = pack_pair<T>(__uint_as_float(ov[v * 8 + 2]) * inv, __uint_as_float(ov[v * 8 + 3]) * inv);
              pk.z = pack_pair<T>(__uint_as_float(ov[v * 8 + 4]) * inv, __uint_as_float(ov[v * 8 + 5]) * inv);
              pk.w = pack_pair<T>(__uint_as_float(ov[v * 8 + 6]) * inv, __uint_as_float(ov[v * 8 + 7]) * inv);
              // 128-byte swizzle: 16-byte chunk q of row r lives at chunk q ^ (r & 7)
              const uint32_t q = (uint32_t)(c * 4 + v);
              const uint32_t addr = my_stage + (uint32_t)lane * 128 + ((q ^ ((uint32_t)lane & 7u)) << 4);
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(pk.x), "r"(pk.y), "r"(pk.z), "r"(pk.w)
                           : "memory");
            }
          }
          ptx::fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0 && tma_ok && hf * 64 < a.d_real) {  // (a half made of padding columns only is not stored)
            ptx::tma_store_4d(&map_o, my_stage, hf * 64, w.h, w.qrow + wrow0, w.b);
            ptx::bulk_commit_group();
          }
          if (a.n_extra > 0 || guarded_main) {
            // copies of the tile for the other GPUs (and the row-guarded store of a sequence's last rows):
            // 8 lanes write one row's 128 bytes, 4 rows per instruction
            const int64_t row_off = (int64_t)w.b * a.o_sb + (int64_t)w.h * a.o_sh + hf * 64 + (int64_t)w.qrow * a.o_ss;
#pragma unroll 1
            for (int e = guarded_main ? -1 : 0; e < a.n_extra; ++e) {
              T* dst = reinterpret_cast<T*>(e < 0 ? a.o : a.extra_o[e]) + row_off;
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const int r = i * 4 + (lane >> 3), ch = lane & 7;
                uint4 val;
                const uint32_t addr = my_stage + (uint32_t)r * 128 + (((uint32_t)ch ^ ((uint32_t)r & 7u)) << 4);
                asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(val.x), "=r"(val.y), "=r"(val.z), "=r"(val.w) : "r"(addr));
                if (wrow0 + r < w.sq && hf * 64 + ch * 8 < a.d_real) *reinterpret_cast<uint4*>(dst + (int64_t)(wrow0 + r) * a.o_ss + ch * 8) = val;
              }
            }
          }
          __syncwarp();
        }
      }
      if (a.lse && row < w.sq)
        a.lse[((int64_t)w.b * a.Hq + w.h) * a.Sq + w.qrow + row] =
            (l > 0.f && m_used != -INFINITY) ? m_used * kLn2 + logf(l) : -INFINITY;
      // the next item's first P*V overwrites O: order this thread's TMEM reads before its later arrivals
      ptx::tc_fence_before();
      if (probe) stamp(a, 16 * n_item + 11);
      ++n_item;
    }
  }

  // =========================== teardown ===========================
  if (warp >= 4 && lane == 0) ptx::bulk_wait_read_all();  // staging rows read; the global writes complete with the kernel
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, C::kTmemCols);
  }
}

#ifdef DT_BRINGUP
int g_options = 0;
float* g_dbg = nullptr;
#endif

template <typename T, int D, bool kMask>
int launch_t(const dt_sdpa_params& p, cudaStream_t stream, void* const* extra, int n_extra, void* workspace,
             size_t workspace_bytes) {
  using C = Cfg<D, kMask>;
  CUtensorMap mq, mk, mv, mo;
  if (!make_bshd_tensor_map(&mq, p.q, p.B, p.Sq, p.Hq, p.D, p.dtype, kBM)) return DT_UNSUPPORTED;
  if (!make_bshd_tensor_map(&mk, p.k, p.B, p.Sk, p.Hkv, p.D, p.dtype, kBN)) return DT_UNSUPPORTED;
  if (!make_bshd_tensor_map(&mv, p.v, p.B, p.Sk, p.Hkv, p.D, p.dtype, kBN)) return DT_UNSUPPORTED;
  if (!make_bshd_tensor_map(&mo, p.o, p.B, p.Sq, p.Hq, p.D, p.dtype, 32)) return DT_UNSUPPORTED;
  PrefillArgs a{};
  a.o = p.o.ptr;
  a.lse = p.lse;
#ifdef DT_BRINGUP
  a.dbg = g_dbg;
  a.options = g_options;
#endif
  a.o_sb = p.o.stride_b; a.o_ss = p.o.stride_s; a.o_sh = p.o.stride_h;
  a.status = device_status_word();
  if (!a.status) return DT_CUDA;
  a.Sq = p.Sq; a.Sk = p.Sk; a.Hq = p.Hq; a.Hkv = p.Hkv;
  a.scale_log2 = p.scale * kLog2e;
  a.scale = p.scale;
  a.mask = p.mask;
  a.m_sb = p.mask_stride_b; a.m_sh = p.mask_stride_h; a.m_sq = p.mask_stride_q;
  if (kMask) {
    if (!workspace || workspace_bytes < prefill_workspace_bytes(p)) return DT_WORKSPACE;
    const int Bm = p.mask_stride_b ? p.B : 1, Hm = p.mask_stride_h ? p.Hq : 1;
    a.n_rg = (p.Sq + 31) / 32;
    a.n_kh = ((p.Sk + 63) / 64 + 1) & ~1;
    a.mask_flags = static_cast<const unsigned char*>(workspace);
    dim3 fgrid((a.n_kh + 7) / 8, a.n_rg, Bm * Hm);
    if (fgrid.y > 65535 || fgrid.z > 65535) return DT_UNSUPPORTED;
    mask_flags_kernel<<<fgrid, 256, 0, stream>>>(static_cast<const unsigned short*>(p.mask), p.mask_stride_b, p.mask_stride_h,
                                                p.mask_stride_q, Hm, p.Sq, p.Sk, a.n_rg, a.n_kh, p.is_causal,
                                                static_cast<unsigned char*>(workspace));
    DT_CUDA_TRY(cudaGetLastError());
  }
  a.is_causal = p.is_causal;
  a.window = p.sliding_window;
  a.sinks = p.sinks;
  if (n_extra < 0 || n_extra > kMaxExtraOutputs) return DT_BAD_ARG;
  a.n_extra = n_extra;
  a.d_real = p.D;
  for (int i = 0; i < n_extra; ++i) a.extra_o[i] = extra[i];
  const bool varlen = p.seq_offsets_q != nullptr;
  a.off_q = p.seq_offsets_q;
  a.off_k = p.seq_offsets_k;
  a.n_qpairs = ((varlen ? p.max_seq_q : p.Sq) + C::kTiles * kBM - 1) / (C::kTiles * kBM);
  a.n_items = a.n_qpairs * p.Hq * (varlen ? p.n_seq : p.B);
  auto kern = prefill_tcgen05_kernel<T, D, kMask>;
  DT_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
  const int n_sm = device_sm_count();
  dim3 grid(a.n_items < n_sm ? a.n_items : n_sm);  // one persistent CTA per SM
  a.n_slots = (a.n_items + (int)grid.x - 1) / (int)grid.x * (int)grid.x;
  kern<<<grid, kThreads, C::kSmemBytes, stream>>>(mq, mk, mv, mo, a);
  DT_CUDA_TRY(cudaGetLastError());
  return DT_OK;
}

}  // namespace

bool prefill_supported(const dt_sdpa_params& p) {
  // variable-length batches: the plain operator only (per-sequence lengths are on the device, so the causal and
  // window cases, which need sq <= sk per sequence, stay on the generic kernel)
  if (p.seq_offsets_q && (p.is_causal || p.sliding_window > 0 || p.n_seq > 65535)) return false;
  if (p.sliding_window > 0 && p.Sq > p.Sk) return false;  // rows that may see no key: generic kernel
  if (p.dtype != DT_F16 && p.dtype != DT_BF16) return false;
  if (p.D < 8 || p.D > 256 || p.D % 8) return false;  // head dims below 64 / 128 / 256 run zero-padded (SD1.5: 40, 80, 160)
  // additive mask: each row's entries are read with 16-byte loads
  if (p.mask && (reinterpret_cast<uintptr_t>(p.mask) % 16 || p.mask_stride_b % 8 || p.mask_stride_h % 8 || p.mask_stride_q % 8))
    return false;
  if (!(p.scale > 0.f)) return false;
  if (p.Hq % p.Hkv) return false;
  if (p.Hq > 65535 || p.B > 65535) return false;
  if (p.is_causal && p.Sq > p.Sk) return false;  // rows without any visible key: left to the generic kernel
  auto ok = [](const dt_tensor4& t) {
    return (reinterpret_cast<uintptr_t>(t.ptr) % 16 == 0) && t.stride_b % 8 == 0 && t.stride_s % 8 == 0 &&
           t.stride_h % 8 == 0;
  };
  return ok(p.q) && ok(p.k) && ok(p.v) && ok(p.o);
}

size_t prefill_workspace_bytes(const dt_sdpa_params& p) {
  if (!p.mask) return 0;
  const size_t Bm = p.mask_stride_b ? p.B : 1, Hm = p.mask_stride_h ? p.Hq : 1;
  const size_t n_rg = (p.Sq + 31) / 32, n_kh = ((p.Sk + 63) / 64 + 1) & ~(size_t)1;
  return (Bm * Hm * n_rg * n_kh + 255) / 256 * 256;
}

int launch_prefill(const dt_sdpa_params& p, cudaStream_t stream, void* const* extra_outputs, int n_extra, void* workspace,
                   size_t workspace_bytes) {
#define DT_PREFILL_GO(T, DD, M) launch_t<T, DD, M>(p, stream, extra_outputs, n_extra, workspace, workspace_bytes)
#define DT_PREFILL_BY_D(T, M) (p.D > 128 ? DT_PREFILL_GO(T, 256, M) : p.D > 64 ? DT_PREFILL_GO(T, 128, M) : DT_PREFILL_GO(T, 64, M))
  if (p.mask) return p.dtype == DT_F16 ? DT_PREFILL_BY_D(__half, true) : DT_PREFILL_BY_D(__nv_bfloat16, true);
  return p.dtype == DT_F16 ? DT_PREFILL_BY_D(__half, false) : DT_PREFILL_BY_D(__nv_bfloat16, false);
#undef DT_PREFILL_BY_D
#undef DT_PREFILL_GO
}

}  // namespace dt

#ifdef DT_BRINGUP
// Bring-up builds only: kernel probe bits and the buffer the probes write to.
extern "C" int dt_internal_set_prefill_options(int options) {
  dt::g_options = options;
  return 0;
}
extern "C" int dt_internal_set_prefill_dump(float* device_buffer) {
  dt::g_dbg = device_buffer;
  return 0;
}
#endif
