// Cross-attention over a SHORT key/value sequence for sm_100a: the text-conditioning attention of the UNet models
// (Libraries/SwiftDiffusion/Sources/Models/UNetXL.swift:57-185, UNet.swift:269-504: thousands of image queries
// against the 77 tokens of a text prompt).  All keys fit one block, so there is no online-softmax loop: a 128-row
// query tile is  S = Q K^T  ->  row softmax  ->  O = P V  ->  store.  The path is bound by streaming Q in and O out
// of HBM once, and what costs is the latency of that chain, so the CTA runs THREE independent chains:
//
//   warps 0-2     one issuer thread per pipeline: its TMA loads (Q tiles double-buffered one tile ahead, K/V once
//                 per head) and its tcgen05.mma instructions; warp 3 allocates and releases TMEM
//   warps 4-15    three softmax warpgroups, each working through its own run of query tiles, one query row per
//                 thread: wait S -> S row from TMEM -> hide keys >= Sk -> max, exp2, sum -> P (16-bit) back to TMEM
//                 over S -> tell the issuer -> wait O -> O / l -> swizzled staging -> TMA store.  While one
//                 warpgroup waits for its MMA or its loads the other two compute.
//   issuer per tile: O = P V as soon as the four warps have stored P, then S' = Q' K^T of the next tile behind it
//                 in the tensor pipe (which runs them in order, so S' may overwrite P).
//   TMEM: warpgroup g owns columns [160 g, 160 g + 160): S / P in the first 96 (up to 96 keys), O in the last 64.
//
// (Measured on B200, SDXL shape: with thread 0 of each softmax warpgroup issuing its own MMAs the pipelines run in
// lockstep, their MMAs queue up behind each other and the issuing warp falls 0.6 - 0.9 us per tile behind the
// other three: 15.6 us per call.  One issuer thread for all three pipelines cannot keep up: 20.3 us.  This form:
// 14.0 us; starting the pipelines 0.3 - 0.9 us apart to take them out of lockstep, or all exponentials on the
// special-function unit, changed nothing.)
//
// fp16 / bf16, head dim <= 64 (zero-padded by TMA), Sk <= 96, no causal rule / window / mask / sinks (those take
// the general kernel).  Every wait is bounded and reports through the device status word; no thread waits at a
// barrier that another thread could fail to reach, and TMEM is released on every path.
#include <type_traits>

#include "sm100_ptx.cuh"

namespace dt {
namespace {

#ifndef DT_SHORT_POLY
#define DT_SHORT_POLY 1
#endif
constexpr int kRows = 128;            // query rows per tile
constexpr int kGroups = 3;            // softmax warpgroups = independent pipelines per CTA
constexpr int kThreadsShort = 128 + kGroups * 128;  // issuer warpgroup (one active warp) + the softmax warpgroups
constexpr int kQBytes = 128 * 128;    // one Q tile: 128 rows x 64 x 16-bit, one TMA box
constexpr int kStageBytesShort = 4 * 32 * 128;  // O staging of one warpgroup: 4 warps x 32 rows x 128 B
constexpr uint32_t kColsPerGroup = 160, kColO = 96;
// 128 * kRegsIssuer + 384 * kRegsSoftmax must not exceed the 512 * 128 registers the CTA is launched with
constexpr int kRegsIssuer = 80, kRegsSoftmax = 144;

template <int NU>  // NU = 16-key units of the key block (5: up to 80 keys, 6: up to 96)
struct ShortCfg {
  static constexpr int kKeys = NU * 16;
  static constexpr int kKVBytes = kKeys * 128;  // K (or V) block: kKeys rows x 64 x 16-bit
  static constexpr int kGroupBytes = 2 * kQBytes + 2 * kKVBytes + kStageBytesShort;
  static constexpr int kSmemBytes = kGroups * kGroupBytes + 1024 /*alignment*/ + 256 /*barriers*/;
};

struct ShortArgs {
  float* lse;
  unsigned int* status;
  int Sq, Sk, Hq, Hkv;
  int n_qtiles, n_tiles;  // tiles = (batch, head, 128-row query tile), query tile fastest
  float scale_log2;
#ifdef DT_BRINGUP
  unsigned long long* dbg;  // timeline probe: [warpgroup run][tile of the run][8] globaltimer stamps
#endif
};

#ifdef DT_BRINGUP
unsigned long long* g_short_dbg = nullptr;
#define DT_SSTAMP(k) do { if (a.dbg && (threadIdx.x & 127) == 0 && (t - t_begin) < 8) a.dbg[(gi * 8 + (t - t_begin)) * 8 + (k)] = ptx::globaltimer_ns(); } while (0)
#else
#define DT_SSTAMP(k) do { } while (0)
#endif

struct GroupBars {
  uint64_t q_full[2];  // TMA: a Q tile has landed
  uint64_t kv_full;    // TMA: K and V of a head have landed
  uint64_t s_full;     // tensor pipe: S of the current tile is complete
  uint64_t p_full;     // the four softmax warps: P of the current tile is in TMEM (and O of the previous tile was read)
  uint64_t o_full;     // tensor pipe: O of the current tile is complete
};

template <typename T>
__device__ __forceinline__ uint32_t pack16(float lo, float hi) {
  if constexpr (std::is_same<T, __half>::value) return ptx::cvt_pack_f16(lo, hi);
  else return ptx::cvt_pack_bf16(lo, hi);
}

struct ShortTile { int b, h, kvh, q0; };
__device__ __forceinline__ ShortTile decode_short_tile(const ShortArgs& a, int t) {
  ShortTile w;
  const int bh = t / a.n_qtiles;
  w.q0 = (t - bh * a.n_qtiles) * kRows;
  w.b = bh / a.Hq;
  w.h = bh - w.b * a.Hq;
  w.kvh = w.h / (a.Hq / a.Hkv);
  return w;
}

template <typename T, int NU>
__global__ void __launch_bounds__(kThreadsShort, 1)
crossattn_short_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_o,
                       const ShortArgs a) {
  using C = ShortCfg<NU>;
  constexpr int kBf16 = std::is_same<T, __half>::value ? 0 : 1;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw);
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s[kGroups];
  // pipeline g: shared memory [Q buffer 0][Q buffer 1][K][V][O staging] at g * kGroupBytes, barriers behind all three
  GroupBars* bars_all = reinterpret_cast<GroupBars*>(base_ptr + kGroups * C::kGroupBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#ifdef DT_BRINGUP
  if (a.dbg && threadIdx.x == 0) a.dbg[((long long)blockIdx.x * kGroups * 8 + 6) * 8 + 7] = ptx::globaltimer_ns();  // CTA entry
#endif
  // pipeline g's run of tiles: an even share of all (batch, head, query tile) triples, consecutive, so that most
  // of a run reads one head's K/V
  const long long n_runs = (long long)gridDim.x * kGroups;
  auto run_begin = [&](int g) { return (int)(((long long)blockIdx.x * kGroups + g) * a.n_tiles / n_runs); };
  auto run_end = [&](int g) { return (int)(((long long)blockIdx.x * kGroups + g + 1) * a.n_tiles / n_runs); };

  auto load_q = [&](int g, int buf, const ShortTile& w) {
    uint64_t* bar = &bars_all[g].q_full[buf];
    ptx::mbar_arrive_expect_tx(bar, (uint32_t)kQBytes);
    ptx::tma_load_4d(base_ptr + g * C::kGroupBytes + buf * kQBytes, &map_q, bar, 0, w.h, w.q0, w.b);
  };
  auto load_kv = [&](int g, const ShortTile& w) {
    uint64_t* bar = &bars_all[g].kv_full;
    uint8_t* dst = base_ptr + g * C::kGroupBytes + 2 * kQBytes;
    ptx::mbar_arrive_expect_tx(bar, (uint32_t)(2 * C::kKVBytes));
    ptx::tma_load_4d(dst, &map_k, bar, 0, w.kvh, 0, w.b);
    ptx::tma_load_4d(dst + C::kKVBytes, &map_v, bar, 0, w.kvh, 0, w.b);
  };

  const bool issuer = warp < kGroups && lane == 0;  // warp g, lane 0: the issuer of pipeline g
  if (issuer) {
    const int g = warp;
    ptx::prefetch_tensormap(&map_q);
    ptx::prefetch_tensormap(&map_k);
    ptx::prefetch_tensormap(&map_v);
    ptx::mbar_init(&bars_all[g].q_full[0], 1);
    ptx::mbar_init(&bars_all[g].q_full[1], 1);
    ptx::mbar_init(&bars_all[g].kv_full, 1);
    ptx::mbar_init(&bars_all[g].s_full, 1);
    ptx::mbar_init(&bars_all[g].p_full, 4);  // one arrival per softmax warp
    ptx::mbar_init(&bars_all[g].o_full, 1);
    abort_s[g] = 0;
    ptx::fence_mbar_init();
    // first loads of the pipeline (K/V of its first head, its first two Q tiles): they need only the barriers
    // above and run while TMEM is being allocated
    const int tb = run_begin(g), te = run_end(g);
    if (tb < te) {
      const ShortTile w0 = decode_short_tile(a, tb);
      load_kv(g, w0);
      load_q(g, 0, w0);
      if (tb + 1 < te) load_q(g, 1, decode_short_tile(a, tb + 1));
    }
  }
  if (warp == 3) {
    ptx::prefetch_tensormap(&map_o);
    ptx::tmem_alloc(&tmem_base_s, 512);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_all = tmem_base_s;

  if (warp < 4) {
    ptx::setmaxnreg_dec<kRegsIssuer>();
    if (issuer) {
      // =========================== issuer of pipeline g ===========================
      const int g = warp;
      GroupBars& bar = bars_all[g];
      volatile int* abort_flag = &abort_s[g];
      constexpr uint32_t idesc_qk = ptx::make_idesc_f16(kBf16, kRows, C::kKeys, 0, 0);
      constexpr uint32_t idesc_pv = ptx::make_idesc_f16(kBf16, kRows, 64, 0, 1);
      const uint32_t g_smem = base + (uint32_t)(g * C::kGroupBytes);
      const uint32_t s_tmem = tmem_all + (uint32_t)g * kColsPerGroup;
      const uint64_t dq0 = ptx::make_smem_desc_sw128(g_smem, 16, 1024);                   // K-major: Q buffers, K
      const uint64_t dk = ptx::make_smem_desc_sw128(g_smem + 2 * kQBytes, 16, 1024);
      const uint64_t dv = ptx::make_smem_desc_sw128(g_smem + 2 * kQBytes + C::kKVBytes, (uint32_t)C::kKVBytes, 1024);  // MN-major: V
      auto issue_qk = [&](int buf) {  // S = Q[buf] K^T: four steps of 16 head dims, 32 B apart in the 128-byte rows
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          ptx::mma_ss(s_tmem, dq0 + (uint64_t)((buf * kQBytes + ks * 32) >> 4), dk + (uint64_t)((ks * 32) >> 4), idesc_qk,
                      ks > 0 ? 1u : 0u);
        ptx::tc_commit(&bar.s_full);
      };
      const int t_begin = run_begin(g), t_end = run_end(g);
      bool ok = t_begin < t_end;
      auto fail = [&]() {
        atomicCAS(a.status, 0u, 1u);
        *abort_flag = 1;
        ok = false;
      };
      uint32_t n_kv = 0;  // K/V loads consumed so far: the parity of the next one
      if (ok) {
        if (ptx::mbar_wait(&bar.kv_full, 0, abort_flag) && ptx::mbar_wait(&bar.q_full[0], 0, abort_flag)) {
          n_kv = 1;
          ptx::tc_fence_after();
          issue_qk(0);
        } else {
          fail();
        }
      }
      ShortTile w = decode_short_tile(a, ok ? t_begin : 0);
      for (int t = t_begin; t < t_end && ok; ++t) {
        const int i = t - t_begin;  // ordinal of the tile within the run: barrier parities follow from it
        const bool more = t + 1 < t_end;
        const ShortTile nx = decode_short_tile(a, more ? t + 1 : t);
        // O = P V as soon as the four warps have stored P (8 TMEM columns per 16 keys), V [key][dim] in shared memory
        if (!ptx::mbar_wait(&bar.p_full, (uint32_t)(i & 1), abort_flag)) { fail(); break; }
        ptx::tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < NU; ++kk)
          ptx::mma_ts(s_tmem + kColO, s_tmem + kk * 8, dv + (uint64_t)(kk * (2048 >> 4)), idesc_pv, kk > 0 ? 1u : 0u);
        ptx::tc_commit(&bar.o_full);
        // P(t) in TMEM means S(t) was read, so Q(t)'s buffer is free: fetch the tile after next into it
        if (t + 2 < t_end) load_q(g, i & 1, decode_short_tile(a, t + 2));
        if (!more) break;
        if (nx.b != w.b || nx.kvh != w.kvh) {
          // another head: its K/V replace the current ones once the P V above has read V (S read K long ago)
          if (!ptx::mbar_wait(&bar.o_full, (uint32_t)(i & 1), abort_flag)) { fail(); break; }
          load_kv(g, nx);
          if (!ptx::mbar_wait(&bar.kv_full, n_kv & 1u, abort_flag)) { fail(); break; }
          ++n_kv;
        }
        // the next tile sits in the other Q buffer; its S goes behind the P V in the tensor pipe
        if (!ptx::mbar_wait(&bar.q_full[(i + 1) & 1], (uint32_t)(((i + 1) >> 1) & 1), abort_flag)) { fail(); break; }
        ptx::tc_fence_after();
        issue_qk((i + 1) & 1);
        w = nx;
      }
    }
  } else {
    ptx::setmaxnreg_inc<kRegsSoftmax>();
    // =========================== softmax / epilogue warpgroups ===========================
    const int group = (warp >> 2) - 1, wig = warp & 3;  // pipeline, warp within it
    GroupBars* bars = &bars_all[group];
    volatile int* abort_flag = &abort_s[group];
    const uint32_t t_s = tmem_all + (uint32_t)group * kColsPerGroup + ((uint32_t)(wig << 5) << 16);
    const uint32_t t_o = t_s + kColO;
    const uint32_t stage_smem = base + (uint32_t)(group * C::kGroupBytes) + 2 * kQBytes + 2 * C::kKVBytes + (uint32_t)wig * (32 * 128);
    const int t_begin = run_begin(group), t_end = run_end(group);
#ifdef DT_BRINGUP
    const long long gi = (long long)blockIdx.x * kGroups + group;
    if (a.dbg && (threadIdx.x & 127) == 0) a.dbg[(gi * 8 + 7) * 8 + 7] = ptx::globaltimer_ns();  // start of the run
#endif
    auto give_up = [&](unsigned code) {
      atomicCAS(a.status, 0u, code);
      *abort_flag = 1;
    };

    for (int t = t_begin; t < t_end; ++t) {
      const uint32_t par = (uint32_t)((t - t_begin) & 1);
      const ShortTile w = decode_short_tile(a, t);
      const int row = w.q0 + (wig << 5) + lane;
      // ---- S row -> P row ----
      DT_SSTAMP(0);
      if (!__all_sync(0xffffffffu, ptx::mbar_wait(&bars->s_full, par, abort_flag))) {
        give_up(3u);
        break;
      }
      DT_SSTAMP(1);
      ptx::tc_fence_after();
      uint32_t s[NU][16];
#pragma unroll
      for (int u = 0; u < NU; ++u) ptx::tmem_ld16(t_s + u * 16, s[u]);
      ptx::tc_wait_ld();
      // keys >= Sk are TMA zero fill (score 0, not -inf): hide them
#pragma unroll
      for (int u = 0; u < NU; ++u) {
        if (u * 16 + 15 < a.Sk) continue;
#pragma unroll
        for (int i = 0; i < 16; ++i)
          if (u * 16 + i >= a.Sk) s[u][i] = 0xff800000u;
      }
      float mx[NU];
#pragma unroll
      for (int u = 0; u < NU; ++u) {
        mx[u] = ptx::max3(__uint_as_float(s[u][0]), __uint_as_float(s[u][1]), __uint_as_float(s[u][2]));
#pragma unroll
        for (int i = 3; i < 15; i += 2) mx[u] = ptx::max3(mx[u], __uint_as_float(s[u][i]), __uint_as_float(s[u][i + 1]));
        mx[u] = fmaxf(mx[u], __uint_as_float(s[u][15]));
      }
      float mall = mx[0];
#pragma unroll
      for (int u = 1; u < NU; ++u) mall = fmaxf(mall, mx[u]);
      const float m = mall * a.scale_log2;  // scale > 0 is a precondition of this kernel
      const float neg_m = (m == -INFINITY) ? 0.f : -m;
      const uint64_t neg_m2 = ptx::pack_f32x2(neg_m, neg_m);
      const uint64_t scale2 = ptx::pack_f32x2(a.scale_log2, a.scale_log2);
      uint64_t lsum[2] = {0ull, 0ull};
      // P as 16-bit pairs, 8 TMEM columns per 16 keys, stored unit by unit so that the score registers free up
#pragma unroll
      for (int u = 0; u < NU; ++u) {
        uint32_t pk[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const uint64_t x2 = ptx::fma_f32x2(ptx::pack_f32x2(__uint_as_float(s[u][2 * i]), __uint_as_float(s[u][2 * i + 1])),
                                             scale2, neg_m2);
          float p0, p1;
          if (DT_SHORT_POLY && (i % 3) == 2) {  // a share of the exponentials runs on the FMA pipes
            ptx::exp2_poly_x2(x2, p0, p1);
          } else {
            float x0, x1;
            ptx::unpack_f32x2(x2, x0, x1);
            p0 = fast_exp2(x0);
            p1 = fast_exp2(x1);
          }
          lsum[i & 1] = ptx::add_f32x2(lsum[i & 1], ptx::pack_f32x2(p0, p1));
          pk[i] = pack16<T>(p0, p1);
        }
        ptx::tmem_st8(t_s + u * 8, pk);
      }
      ptx::tc_wait_st();
      float a0, a1;
      ptx::unpack_f32x2(ptx::add_f32x2(lsum[0], lsum[1]), a0, a1);
      const float l = a0 + a1;
      // this warp's 32 rows of P are in TMEM (and its reads of the previous tile's O are done): tell the issuer
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&bars->p_full);
      DT_SSTAMP(2);

      // ---- epilogue: O / l -> swizzled staging rows -> one TMA store per warp ----
      if (!__all_sync(0xffffffffu, ptx::mbar_wait(&bars->o_full, par, abort_flag))) {
        give_up(5u);
        break;
      }
      DT_SSTAMP(4);
      ptx::tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      if (lane == 0) ptx::bulk_wait_read_all();  // the previous store of this warp has read the staging rows
      __syncwarp();
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t ov[32];
        ptx::tmem_ld32(t_o + c * 32, ov);
        ptx::tc_wait_ld();
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          const uint32_t x = pack16<T>(__uint_as_float(ov[v * 8 + 0]) * inv, __uint_as_float(ov[v * 8 + 1]) * inv);
          const uint32_t y = pack16<T>(__uint_as_float(ov[v * 8 + 2]) * inv, __uint_as_float(ov[v * 8 + 3]) * inv);
          const uint32_t z = pack16<T>(__uint_as_float(ov[v * 8 + 4]) * inv, __uint_as_float(ov[v * 8 + 5]) * inv);
          const uint32_t ww = pack16<T>(__uint_as_float(ov[v * 8 + 6]) * inv, __uint_as_float(ov[v * 8 + 7]) * inv);
          // 128-byte swizzle: 16-byte chunk q of row r lives at chunk q ^ (r & 7)
          const uint32_t q = (uint32_t)(c * 4 + v);
          const uint32_t addr = stage_smem + (uint32_t)lane * 128 + ((q ^ ((uint32_t)lane & 7u)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(x), "r"(y), "r"(z), "r"(ww) : "memory");
        }
      }
      ptx::fence_proxy_async_smem();
      __syncwarp();
      const int wrow0 = w.q0 + (wig << 5);
      if (lane == 0 && wrow0 < a.Sq) {  // rows beyond Sq are clipped by the tensor map
        ptx::tma_store_4d(&map_o, stage_smem, 0, w.h, wrow0, w.b);
        ptx::bulk_commit_group();
      }
      if (a.lse && row < a.Sq) a.lse[((int64_t)w.b * a.Hq + w.h) * a.Sq + row] = l > 0.f ? m * kLn2 + logf(l) : -INFINITY;
      DT_SSTAMP(5);
    }
    if (lane == 0) ptx::bulk_wait_read_all();  // the staging rows have been read; the global writes complete with the kernel
  }

  // =========================== teardown ===========================
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 3) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_all, 512);
  }
#ifdef DT_BRINGUP
  if (a.dbg && threadIdx.x == 96) a.dbg[((long long)blockIdx.x * kGroups * 8 + 6) * 8 + 6] = ptx::globaltimer_ns();  // CTA exit
#endif
}

template <typename T, int NU>
int launch_short_t(const dt_sdpa_params& p, cudaStream_t stream) {
  using C = ShortCfg<NU>;
  CUtensorMap mq, mk, mv, mo;
  if (!make_bshd_tensor_map(&mq, p.q, p.B, p.Sq, p.Hq, p.D, p.dtype, kRows)) return DT_UNSUPPORTED;
  if (!make_bshd_tensor_map(&mk, p.k, p.B, p.Sk, p.Hkv, p.D, p.dtype, C::kKeys)) return DT_UNSUPPORTED;
  if (!make_bshd_tensor_map(&mv, p.v, p.B, p.Sk, p.Hkv, p.D, p.dtype, C::kKeys)) return DT_UNSUPPORTED;
  if (!make_bshd_tensor_map(&mo, p.o, p.B, p.Sq, p.Hq, p.D, p.dtype, 32)) return DT_UNSUPPORTED;
  ShortArgs a{};
  a.lse = p.lse;
  a.status = device_status_word();
  if (!a.status) return DT_CUDA;
  a.Sq = p.Sq; a.Sk = p.Sk; a.Hq = p.Hq; a.Hkv = p.Hkv;
  a.n_qtiles = (p.Sq + kRows - 1) / kRows;
  const long long tiles = (long long)a.n_qtiles * p.Hq * p.B;
  if (tiles > 0x7fffffffLL) return DT_UNSUPPORTED;
  a.n_tiles = (int)tiles;
  a.scale_log2 = p.scale * kLog2e;
#ifdef DT_BRINGUP
  a.dbg = g_short_dbg;
#endif
  auto kern = crossattn_short_kernel<T, NU>;
  DT_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
  const int n_sm = device_sm_count();
  const int want = (a.n_tiles + kGroups - 1) / kGroups;  // at least one tile per warpgroup
  dim3 grid(want < n_sm ? want : n_sm);                   // one persistent CTA per SM
  kern<<<grid, kThreadsShort, C::kSmemBytes, stream>>>(mq, mk, mv, mo, a);
  DT_CUDA_TRY(cudaGetLastError());
  return DT_OK;
}

}  // namespace

bool short_kv_supported(const dt_sdpa_params& p) {
  if (p.dtype != DT_F16 && p.dtype != DT_BF16) return false;
  if (p.D < 8 || p.D > 64 || p.D % 8) return false;
  if (p.Sk > 96) return false;
  if (p.is_causal || p.sliding_window > 0 || p.mask || p.sinks || p.seq_offsets_q) return false;
  if (!(p.scale > 0.f)) return false;
  if (p.Hq % p.Hkv || p.Hq > 65535 || p.B > 65535) return false;
  auto ok = [](const dt_tensor4& t) {
    return (reinterpret_cast<uintptr_t>(t.ptr) % 16 == 0) && t.stride_b % 8 == 0 && t.stride_s % 8 == 0 &&
           t.stride_h % 8 == 0;
  };
  return ok(p.q) && ok(p.k) && ok(p.v) && ok(p.o);
}

int launch_short_kv(const dt_sdpa_params& p, cudaStream_t stream) {
  const bool five = p.Sk <= 80;
  if (p.dtype == DT_F16) return five ? launch_short_t<__half, 5>(p, stream) : launch_short_t<__half, 6>(p, stream);
  return five ? launch_short_t<__nv_bfloat16, 5>(p, stream) : launch_short_t<__nv_bfloat16, 6>(p, stream);
}

}  // namespace dt

#ifdef DT_BRINGUP
// Bring-up builds only: timeline buffer of the short key/value kernel.
extern "C" int dt_internal_set_short_dump(unsigned long long* device_buffer) {
  dt::g_short_dbg = device_buffer;
  return 0;
}
#endif
