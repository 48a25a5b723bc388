// The step immediately after the attention node when the reference builds it with
// multiHeadOutputProjectionFused: true (Libraries/SwiftDiffusion/Sources/Models/UNet.swift:122-130, weights loaded
// at UNet.swift:865-874): out[b, s, :] = concat_h(O[b, s, h, :]) . W^T + bias, i.e. the "unify heads" Dense folded
// into the operator.  Here it is a TMA + tcgen05 GEMM that runs right behind the attention kernel on the same
// stream, reading the attention output from the workspace while it is still in L2.
//
//   C[M, N] = A[M, K] . B[N, K]^T + bias[N]      A = attention output rows (K = Hq * D, contiguous),
//                                                B = Dense weight, [out, in] row-major, both K-major operands
//   CTA   = persistent, one per SM, looping over 128 x 256 tiles of C, column tile fastest (CTAs that run together
//           share A row blocks and W column blocks in L2; N = 256 halves the A traffic per FLOP: the loop is bound by
//           L2 -> shared memory bandwidth, not by the tensor pipe); 8 warps: TMA producer, MMA issuer, TMEM allocator, (idle), 4 epilogue warps.
//   loop  = K in steps of 64 (one 128-byte swizzle atom): an A box of 128 rows and a B box of 256 rows land in a
//           4-stage ring; one thread issues four tcgen05.mma (M128 N256 K16) per stage into one of two 256-column fp32
//           accumulators in TMEM (the epilogue of tile i overlaps the main loop of tile i + 1) and commits the stage
//           back to the producer; the ring keeps running across tiles.
//   tail  = the tiles left over after the last full round over the SMs are cut into 2 or 4 column slices (N = 128 or
//           64 per MMA) when that many slices still fit one round, so the last round costs a half or a quarter of a
//           tile time instead of a whole one (SDXL's 320 tiles on 148 SMs: 2 rounds + 96 quarter tiles); a problem
//           with fewer tiles than SMs is sliced the same way to use more of them.
//   out   = accumulator rows -> + bias -> 16-bit -> swizzled staging rows -> one TMA store per warp and half
//           (clipped by the tensor map at the edges of M and N).
// Every wait is bounded and reports through the device status word (code 6).
#include "sm100_ptx.cuh"

namespace dt {
namespace {

constexpr int kTile = 128;           // rows of A per tile (M)
constexpr int kTileN = 256;          // rows of B per tile (N)
constexpr int kKStep = 64;           // K elements per stage: 128 bytes
constexpr int kStages = 4;
constexpr int kBoxBytesP = kTile * 128;  // the A box: 128 rows x 128 bytes
constexpr int kStageBytesP = kBoxBytesP + kTileN * 128;
constexpr int kStagingBytes = 4 * 32 * 128;  // four epilogue warps x 32 rows x 128 bytes
constexpr int kProjThreads = 256;
constexpr int kProjSmem = kStages * kStageBytesP + kStagingBytes + 1024 + 256;

struct ProjBarriers {
  uint64_t full[kStages], empty[kStages], acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

struct ProjArgs {
  const void* bias;  // [N] or null
  unsigned int* status;
  int S, N, K, tiles_per_batch;
  int n_tiles_n, n_tiles;  // column tiles, all tiles (column tile fastest)
  int full_rounds;         // rounds in which CTA x works on whole tile x + round * gridDim.x
  int tail_split, tail_units;  // then CTA x < tail_units takes slice x % tail_split of tile full_rounds * gridDim.x + x / tail_split
  // Row-parallel mode (head-sharded ranks each hold a K-slice): the fp32 partial tile goes to the rank that owns
  // its rows, into slab [this rank] of that rank's receive buffer [world][rows_per_rank][N] (ordinary stores, peer
  // memory over NVLink for other ranks); the owner sums the slabs afterwards.  slab[0] == nullptr: plain mode.
  float* slab[8];
  int rank, rows_per_rank;
};

template <typename T>
__device__ __forceinline__ uint32_t pack_pair_t(float a, float b) {
  if constexpr (std::is_same<T, __half>::value) return ptx::cvt_pack_f16(a, b);
  else return ptx::cvt_pack_bf16(a, b);
}

template <typename T>
__global__ void __launch_bounds__(kProjThreads)
out_proj_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                const __grid_constant__ CUtensorMap map_b_tail, const __grid_constant__ CUtensorMap map_c, const ProjArgs a) {
  constexpr bool kBf16 = !std::is_same<T, __half>::value;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw);
  const uint32_t staging = base + kStages * kStageBytesP;
  ProjBarriers* bars = reinterpret_cast<ProjBarriers*>(base_ptr + kStages * kStageBytesP + kStagingBytes);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nk = (a.K + kKStep - 1) / kKStep;
  // tile -> (column offset, batch item, row offset)
  auto tile_n0 = [&](int t) { return (t % a.n_tiles_n) * kTileN; };
  auto tile_b = [&](int t) { return (t / a.n_tiles_n) / a.tiles_per_batch; };
  auto tile_s0 = [&](int t) { return ((t / a.n_tiles_n) % a.tiles_per_batch) * kTile; };
  // i-th unit of work of this CTA: a whole tile, or (last) one column slice of a left-over tile
  struct Unit { int n0, b, s0, width; };
  auto unit_at = [&](int i, Unit& u) -> bool {
    int t;
    if (i < a.full_rounds) {
      t = (int)blockIdx.x + i * (int)gridDim.x;
      u.width = kTileN;
      u.n0 = tile_n0(t);
    } else if (i == a.full_rounds && (int)blockIdx.x < a.tail_units) {
      t = a.full_rounds * (int)gridDim.x + (int)blockIdx.x / a.tail_split;
      u.width = kTileN / a.tail_split;
      u.n0 = tile_n0(t) + ((int)blockIdx.x % a.tail_split) * u.width;
    } else {
      return false;
    }
    u.b = tile_b(t);
    u.s0 = tile_s0(t);
    return true;
  };

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      ptx::mbar_init(&bars->full[i], 1);
      ptx::mbar_init(&bars->empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(&bars->acc_full[i], 1);
      ptx::mbar_init(&bars->acc_empty[i], 4);  // one arrival per epilogue warp
    }
    bars->abort_flag = 0;
    ptx::fence_mbar_init();
  }
  if (warp == 2) {
    ptx::tmem_alloc(&bars->tmem_base, 2 * kTileN);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = bars->tmem_base;

  if (warp == 0) {
    // =========================== TMA producer ===========================
    if (lane == 0) {
      ptx::prefetch_tensormap(&map_a);
      ptx::prefetch_tensormap(&map_b);
      ptx::prefetch_tensormap(&map_c);
      if (a.tail_split > 1) ptx::prefetch_tensormap(&map_b_tail);
      int it = 0;  // ring position, continues across tiles
      bool ok = true;
      Unit u;
      for (int i = 0; ok && unit_at(i, u); ++i) {
        const int n0 = u.n0, b = u.b, s0 = u.s0;
        const CUtensorMap* mb = u.width == kTileN ? &map_b : &map_b_tail;
        const uint32_t stage_tx = (uint32_t)(kBoxBytesP + u.width * 128);
        for (int kb = 0; kb < nk; ++kb, ++it) {
          const int st = it % kStages, use = it / kStages;
          if (use > 0 && !ptx::mbar_wait(&bars->empty[st], (use - 1) & 1, abort_flag)) {
            atomicCAS(a.status, 0u, 6u);
            *abort_flag = 1;
            ok = false;
            break;
          }
          ptx::mbar_arrive_expect_tx(&bars->full[st], stage_tx);
          uint8_t* dst = base_ptr + st * kStageBytesP;
          ptx::tma_load_4d(dst, &map_a, &bars->full[st], kb * kKStep, 0, s0, b);
          ptx::tma_load_4d(dst + kBoxBytesP, mb, &bars->full[st], kb * kKStep, 0, n0, 0);
        }
      }
    }
  } else if (warp == 1) {
    // =========================== MMA issuer ===========================
    if (lane == 0) {
      const uint64_t desc = ptx::make_smem_desc_sw128(0, 16, 1024);
      bool ok = true;
      int it = 0, n_tile = 0;
      Unit u;
      for (; ok && unit_at(n_tile, u); ++n_tile) {
        const uint32_t idesc = ptx::make_idesc_f16(kBf16, kTile, u.width, 0, 0);
        const int buf = n_tile & 1, use = n_tile >> 1;
        // the epilogue must have drained this accumulator (two tiles ago)
        if (use > 0 && !ptx::mbar_wait(&bars->acc_empty[buf], (use - 1) & 1, abort_flag)) {
          atomicCAS(a.status, 0u, 6u);
          *abort_flag = 1;
          break;
        }
        ptx::tc_fence_after();
        const uint32_t acc = tmem + (uint32_t)(buf * kTileN);
        for (int kb = 0; kb < nk; ++kb, ++it) {
          const int st = it % kStages;
          if (!ptx::mbar_wait(&bars->full[st], (it / kStages) & 1, abort_flag)) {
            atomicCAS(a.status, 0u, 6u);
            *abort_flag = 1;
            ok = false;
            break;
          }
          ptx::tc_fence_after();
          const uint32_t sa = base + st * kStageBytesP, sb = sa + kBoxBytesP;
          const uint64_t da = desc | (uint64_t)((sa & 0x3FFFFu) >> 4), db = desc | (uint64_t)((sb & 0x3FFFFu) >> 4);
#pragma unroll
          for (int kk = 0; kk < kKStep / 16; ++kk)
            ptx::mma_ss(acc, da + (uint64_t)(kk * 2), db + (uint64_t)(kk * 2), idesc, (kb > 0 || kk > 0) ? 1u : 0u);
          ptx::tc_commit(&bars->empty[st]);  // the stage may be refilled once these MMAs have read it
        }
        if (ok) ptx::tc_commit(&bars->acc_full[buf]);
      }
    }
  } else if (warp >= 4) {
    // =========================== epilogue ===========================
    const int ew = warp - 4;  // TMEM lanes 32*ew .. 32*ew + 31 = tile rows
    int n_tile = 0;
    Unit u;
    for (; unit_at(n_tile, u); ++n_tile) {
      const int buf = n_tile & 1;
      const int n0 = u.n0, b = u.b, s0 = u.s0;
      if (!__all_sync(0xffffffffu, ptx::mbar_wait(&bars->acc_full[buf], (n_tile >> 1) & 1, abort_flag))) {
        atomicCAS(a.status, 0u, 6u);
        *abort_flag = 1;
        break;
      }
      ptx::tc_fence_after();
      const uint32_t t_acc = tmem + (uint32_t)(buf * kTileN) + ((uint32_t)(ew * 32) << 16);
      const uint32_t my_stage = staging + (uint32_t)ew * (32 * 128);
      const T* bias = reinterpret_cast<const T*>(a.bias);
      const int row0 = s0 + ew * 32;
      if (a.slab[0] != nullptr) {
        // ---- row-parallel mode: fp32 partials to the owner of these rows ----
        const int owner = s0 / a.rows_per_rank;  // a tile never straddles two owners (rows_per_rank % 128 == 0)
        float* slab = a.slab[0];  // selected without indexing the parameter array dynamically
#pragma unroll
        for (int i = 1; i < 8; ++i)
          if (owner == i) slab = a.slab[i];
        float* dst = slab + ((size_t)a.rank * a.rows_per_rank + (size_t)(row0 - owner * a.rows_per_rank)) * a.N;
#pragma unroll 1
        for (int c = 0; c < u.width / 32; ++c) {
          uint32_t acc[32];
          ptx::tmem_ld32(t_acc + c * 32, acc);
          ptx::tc_wait_ld();
          // stage 32 rows x 128 bytes (16-byte chunk q of row r at q ^ (r & 7)), then 8 lanes write one row
#pragma unroll
          for (int v = 0; v < 8; ++v) {
            const uint32_t addr = my_stage + (uint32_t)lane * 128 + (((uint32_t)v ^ ((uint32_t)lane & 7u)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(acc[v * 4 + 0]), "r"(acc[v * 4 + 1]),
                         "r"(acc[v * 4 + 2]), "r"(acc[v * 4 + 3])
                         : "memory");
          }
          __syncwarp();
          const int col = n0 + c * 32 + (lane & 7) * 4;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int r = i * 4 + (lane >> 3), ch = lane & 7;
            uint4 val;
            const uint32_t addr = my_stage + (uint32_t)r * 128 + (((uint32_t)ch ^ ((uint32_t)r & 7u)) << 4);
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(val.x), "=r"(val.y), "=r"(val.z), "=r"(val.w) : "r"(addr));
            if (row0 + r < a.S && col < a.N) *reinterpret_cast<uint4*>(dst + (size_t)r * a.N + col) = val;
          }
          __syncwarp();
        }
      } else {
#pragma unroll 1
      for (int hf = 0; hf < u.width / 64; ++hf) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t acc[32];
          ptx::tmem_ld32(t_acc + hf * 64 + c * 32, acc);
          ptx::tc_wait_ld();
          const int col0 = n0 + hf * 64 + c * 32;
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            float f[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int col = col0 + v * 8 + i;
              f[i] = __uint_as_float(acc[v * 8 + i]) + ((bias && col < a.N) ? to_float(bias[col]) : 0.f);
            }
            uint4 pk;
            pk.x = pack_pair_t<T>(f[0], f[1]);
            pk.y = pack_pair_t<T>(f[2], f[3]);
            pk.z = pack_pair_t<T>(f[4], f[5]);
            pk.w = pack_pair_t<T>(f[6], f[7]);
            // 128-byte swizzle: 16-byte chunk q of row r lives at chunk q ^ (r & 7)
            const uint32_t q = (uint32_t)(c * 4 + v);
            const uint32_t addr = my_stage + (uint32_t)lane * 128 + ((q ^ ((uint32_t)lane & 7u)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(pk.x), "r"(pk.y), "r"(pk.z), "r"(pk.w)
                         : "memory");
          }
        }
        ptx::fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0 && row0 < a.S && n0 + hf * 64 < a.N) {
          ptx::tma_store_4d(&map_c, my_stage, n0 + hf * 64, 0, row0, b);
          ptx::bulk_commit_group();
          ptx::bulk_wait_read_all();  // the staging rows are rewritten for the second half
        }
        __syncwarp();
      }
      }
      // every TMEM load of this tile has completed: hand the accumulator back to the MMA warp
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&bars->acc_empty[buf]);
    }
    if (lane == 0) ptx::bulk_wait_read_all();  // the staging rows have been read; the global writes complete with the kernel
  }

  // =========================== teardown ===========================
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, 2 * kTileN);
  }
}

template <typename T>
int launch_proj_t(const dt_tensor4& a_view, int B, int S, int K, const void* weight, const void* bias, int N,
                  const dt_tensor4& out, int dtype, cudaStream_t stream, float* const* slabs = nullptr, int world = 0,
                  int rank = 0, int rows_per_rank = 0) {
  CUtensorMap ma, mb, mb_tail, mc;
  dt_tensor4 w_view{const_cast<void*>(weight), (int64_t)N * K, (int64_t)K, (int64_t)K};
  if (!make_bshd_tensor_map(&ma, a_view, B, S, 1, K, dtype, kTile)) return DT_UNSUPPORTED;
  if (!make_bshd_tensor_map(&mb, w_view, 1, N, 1, K, dtype, kTileN)) return DT_UNSUPPORTED;
  if (!make_bshd_tensor_map(&mc, out, B, S, 1, N, dtype, 32)) return DT_UNSUPPORTED;
  ProjArgs a{};
  a.bias = bias;
  a.status = device_status_word();
  if (!a.status) return DT_CUDA;
  a.S = S; a.N = N; a.K = K;
  a.tiles_per_batch = (S + kTile - 1) / kTile;
  if (slabs) {
    if (world < 1 || world > 8 || rows_per_rank % kTile || B != 1) return DT_BAD_ARG;
    for (int i = 0; i < world; ++i) a.slab[i] = slabs[i];
    a.rank = rank;
    a.rows_per_rank = rows_per_rank;
  }
  auto kern = out_proj_kernel<T>;
  DT_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kProjSmem));
  a.n_tiles_n = (N + kTileN - 1) / kTileN;
  const int64_t tiles = (int64_t)a.n_tiles_n * a.tiles_per_batch * B;
  if (tiles > (1 << 30)) return DT_UNSUPPORTED;
  a.n_tiles = (int)tiles;
  const int sms = device_sm_count();
  // whole rounds of one tile per SM, then the left-over tiles in column slices while the slices fit one round
  a.full_rounds = (int)(tiles / sms);
  const int rem = (int)(tiles % sms);
  a.tail_split = rem == 0 ? 1 : (4 * rem <= sms ? 4 : (2 * rem <= sms ? 2 : 1));
  a.tail_units = rem * a.tail_split;
  mb_tail = mb;
  if (a.tail_split > 1 && !make_bshd_tensor_map(&mb_tail, w_view, 1, N, 1, K, dtype, kTileN / a.tail_split)) return DT_UNSUPPORTED;
  dim3 grid((unsigned)(a.full_rounds > 0 ? sms : a.tail_units));  // one persistent CTA per SM
  kern<<<grid, kProjThreads, kProjSmem, stream>>>(ma, mb, mb_tail, mc, a);
  DT_CUDA_TRY(cudaGetLastError());
  return DT_OK;
}

}  // namespace

// a_view: [B, S, 1, K] rows of the attention output; out: [B, S, 1, N]
int launch_out_proj(const dt_tensor4& a_view, int B, int S, int K, const void* weight, const void* bias, int N,
                    const dt_tensor4& out, int dtype, cudaStream_t stream) {
  if (dtype == DT_F16) return launch_proj_t<__half>(a_view, B, S, K, weight, bias, N, out, dtype, stream);
  if (dtype == DT_BF16) return launch_proj_t<__nv_bfloat16>(a_view, B, S, K, weight, bias, N, out, dtype, stream);
  return DT_UNSUPPORTED;
}

// Row-parallel form: A [M, K_local] (this rank's heads), W_local [N, K_local]; fp32 partial tiles are stored into
// slab `rank` of the receive buffer of the rank that owns the tile's rows.  `scratch_out` is a valid [M, N] 16-bit
// view only used to build the (unused) store map.
int launch_out_proj_rowparallel(const dt_tensor4& a_view, int M, int K, const void* weight, int N, const dt_tensor4& scratch_out,
                                int dtype, float* const* slabs, int world, int rank, int rows_per_rank, cudaStream_t stream) {
  if (dtype == DT_F16)
    return launch_proj_t<__half>(a_view, 1, M, K, weight, nullptr, N, scratch_out, dtype, stream, slabs, world, rank, rows_per_rank);
  if (dtype == DT_BF16)
    return launch_proj_t<__nv_bfloat16>(a_view, 1, M, K, weight, nullptr, N, scratch_out, dtype, stream, slabs, world, rank,
                                        rows_per_rank);
  return DT_UNSUPPORTED;
}

namespace {
// out[i, :] = bias + sum over ranks of slab[r][i, :], rounded to T: the owner's half of the reduce-scatter.
template <typename T>
__global__ void __launch_bounds__(256) slab_reduce_kernel(const float* __restrict__ recv, const T* __restrict__ bias,
                                                          T* __restrict__ out, int64_t out_stride, int world, int rows,
                                                          int rows_per_rank, int N) {
  const int vec_per_row = N / 4;
  const int64_t total = (int64_t)rows * vec_per_row;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int row = (int)(i / vec_per_row), c4 = (int)(i - (int64_t)row * vec_per_row);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (bias) {
      acc.x = to_float(bias[c4 * 4 + 0]); acc.y = to_float(bias[c4 * 4 + 1]);
      acc.z = to_float(bias[c4 * 4 + 2]); acc.w = to_float(bias[c4 * 4 + 3]);
    }
    for (int r = 0; r < world; ++r) {  // fixed order: the sum does not depend on arrival order
      const float4 v = *reinterpret_cast<const float4*>(recv + ((size_t)r * rows_per_rank + row) * N + c4 * 4);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    T* o = out + (int64_t)row * out_stride + c4 * 4;
    o[0] = from_float<T>(acc.x); o[1] = from_float<T>(acc.y); o[2] = from_float<T>(acc.z); o[3] = from_float<T>(acc.w);
  }
}
}  // namespace

int launch_slab_reduce(const float* recv, const void* bias, void* out, int64_t out_stride, int world, int rows,
                       int rows_per_rank, int N, int dtype, cudaStream_t stream) {
  if (rows <= 0) return DT_OK;
  const int64_t total = (int64_t)rows * (N / 4);
  int64_t blocks = (total + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (dtype == DT_F16)
    slab_reduce_kernel<__half><<<(int)blocks, 256, 0, stream>>>(recv, (const __half*)bias, (__half*)out, out_stride, world, rows,
                                                                rows_per_rank, N);
  else if (dtype == DT_BF16)
    slab_reduce_kernel<__nv_bfloat16><<<(int)blocks, 256, 0, stream>>>(recv, (const __nv_bfloat16*)bias, (__nv_bfloat16*)out,
                                                                       out_stride, world, rows, rows_per_rank, N);
  else
    return DT_UNSUPPORTED;
  DT_CUDA_TRY(cudaGetLastError());
  return DT_OK;
}

}  // namespace dt
