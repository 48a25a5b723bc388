// Head-sharded attention across the GPUs of one box: each rank runs the local head slice, the output
// slices are exchanged with ncclAllGather over NVLink/NVSwitch on a side stream, and a permute kernel
// lays them out as [B, Sq, H, D].  The query rows are cut into chunks so the gather of chunk c overlaps
// the attention of chunk c+1.  NCCL is loaded with dlopen at first use: the core library has no
// link-time NCCL dependency, and a process that already loaded an NCCL (PyTorch's) shares it.
//
// The reference has no counterpart: it is single-GPU per process (ccv is built with have_nccl = False,
// WORKSPACE.linux:127).  Every TMA load on this path is a plain per-CTA load from this GPU's own memory.
#include <cuda.h>
#include <dlfcn.h>
#include <nccl.h>

#include <stdlib.h>
#include <string.h>

#include <chrono>
#include <thread>

#include "common.cuh"

namespace dt {
namespace {

struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRankConfig)(ncclComm_t*, int, ncclUniqueId, int, ncclConfig_t*) = nullptr;
  ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
  ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  bool ok = false;
};

NcclApi& nccl() {
  static NcclApi api;
  static bool tried = false;
  if (tried) return api;
  tried = true;
  // DTATTN_NCCL_LIB names the NCCL build to load (a deployment with several NCCLs; the failure-path tests point it
  // at a stand-in whose communicator never becomes ready); otherwise the one already in the process or on the path.
  const char* names[] = {getenv("DTATTN_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
  for (const char* n : names) {
    if (!n || !*n) continue;
    api.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
    if (api.handle) break;
  }
  if (!api.handle) return api;
#define LOAD(field, sym) *reinterpret_cast<void**>(&api.field) = dlsym(api.handle, sym)
  LOAD(GetUniqueId, "ncclGetUniqueId");
  LOAD(CommInitRankConfig, "ncclCommInitRankConfig");
  LOAD(CommGetAsyncError, "ncclCommGetAsyncError");
  LOAD(CommAbort, "ncclCommAbort");
  LOAD(CommDestroy, "ncclCommDestroy");
  LOAD(AllGather, "ncclAllGather");
  LOAD(AllReduce, "ncclAllReduce");
#undef LOAD
  api.ok = api.GetUniqueId && api.CommInitRankConfig && api.CommGetAsyncError && api.CommAbort && api.CommDestroy &&
           api.AllGather && api.AllReduce;
  return api;
}

constexpr int kMaxChunks = 64;

struct Comm {
  ncclComm_t comm = nullptr;
  int rank = 0, world = 1;
  int timeout_ms = 30000;
  cudaStream_t side = nullptr;
  cudaEvent_t chunk_done[kMaxChunks];
  cudaEvent_t all_done = nullptr;
  // output buffers registered for the fused mode: every rank's buffer mapped into this process
  static constexpr int kMaxRegs = 8;
  struct Reg {
    void* local = nullptr;
    size_t bytes = 0;
    void* peer[8] = {nullptr};       // peer[r] = rank r's buffer as seen from here (own rank: the local pointer)
    void* opened[8] = {nullptr};     // bases returned by cudaIpcOpenMemHandle, to close later
  } regs[kMaxRegs];
  int n_regs = 0;
  int* flag = nullptr;               // 4 bytes for the in-stream rendezvous after a fused step
  int last_fused_reg = -1;           // registered buffer the previous fused call stored into (-1: none yet)
  unsigned long long proj_calls = 0; // projected head-sharded calls so far: picks the half of the receive buffer
  void* xchg = nullptr;              // small device buffer for exchanging handles
};

struct IpcInfo {
  cudaIpcMemHandle_t handle;
  unsigned long long offset;
  unsigned long long bytes;
};

// Poll the communicator until the pending operation left the in-progress state or the limit ran out.
int wait_nccl(Comm* c, ncclResult_t r, int timeout_ms) {
  NcclApi& api = nccl();
  if (r == ncclSuccess) return DT_OK;
  if (r != ncclInProgress) return DT_NCCL;
  const auto t0 = std::chrono::steady_clock::now();
  for (;;) {
    ncclResult_t st = ncclSuccess;
    if (api.CommGetAsyncError(c->comm, &st) != ncclSuccess) return DT_NCCL;
    if (st == ncclSuccess) return DT_OK;
    if (st != ncclInProgress) return DT_NCCL;
    const auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
    if (ms > timeout_ms) return DT_TIMEOUT;
    std::this_thread::sleep_for(std::chrono::microseconds(50));
  }
}

// src [world][B][Sq][Hl][D] -> dst view [B, Sq, world*Hl, D]; 16-byte vectors.
__global__ void permute_gathered_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst_base, int world, int B,
                                        int Sq, int Hl, int vec_per_head, int64_t d_sb, int64_t d_ss, int64_t d_sh,
                                        int64_t total) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t t = i;
    const int vv = (int)(t % vec_per_head); t /= vec_per_head;
    const int h = (int)(t % Hl); t /= Hl;
    const int s = (int)(t % Sq); t /= Sq;
    const int b = (int)(t % B); t /= B;
    const int w = (int)t;
    // strides are in 16-byte vectors here
    dst_base[b * d_sb + s * d_ss + (int64_t)(w * Hl + h) * d_sh + vv] = src[i];
  }
}

}  // namespace

int launch_permute_gathered(const void* src, dt_tensor4 dst, int world, int B, int Sq, int Hl, int D, int dtype,
                            cudaStream_t stream) {
  const size_t es = dtype_size(dtype);
  const size_t head_bytes = (size_t)D * es;
  if (head_bytes % 16) return DT_UNSUPPORTED;
  const int vec = (int)(16 / es);
  if (dst.stride_b % vec || dst.stride_s % vec || dst.stride_h % vec) return DT_UNSUPPORTED;
  if (reinterpret_cast<uintptr_t>(src) % 16 || reinterpret_cast<uintptr_t>(dst.ptr) % 16) return DT_UNSUPPORTED;
  const int vph = (int)(head_bytes / 16);
  const int64_t total = (int64_t)world * B * Sq * Hl * vph;
  const int threads = 256;
  int64_t blocks = (total + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  permute_gathered_kernel<<<(int)blocks, threads, 0, stream>>>(
      reinterpret_cast<const uint4*>(src), reinterpret_cast<uint4*>(dst.ptr), world, B, Sq, Hl, vph,
      dst.stride_b / vec, dst.stride_s / vec, dst.stride_h / vec, total);
  DT_CUDA_TRY(cudaGetLastError());
  return DT_OK;
}

}  // namespace dt

using namespace dt;

extern "C" {

int dt_comm_unique_id(void* id_out_128) {
  if (!id_out_128) return DT_BAD_ARG;
  NcclApi& api = nccl();
  if (!api.ok) return DT_NCCL;
  ncclUniqueId id;
  if (api.GetUniqueId(&id) != ncclSuccess) return DT_NCCL;
  static_assert(sizeof(ncclUniqueId) == DT_NCCL_UNIQUE_ID_BYTES, "unique id size");
  memcpy(id_out_128, &id, sizeof(id));
  return DT_OK;
}

int dt_comm_init(void** comm_out, int rank, int world, const void* unique_id_128, int timeout_ms) {
  if (!comm_out || !unique_id_128 || world <= 0 || rank < 0 || rank >= world) return DT_BAD_ARG;
  *comm_out = nullptr;
  NcclApi& api = nccl();
  if (!api.ok) return DT_NCCL;
  Comm* c = new Comm();
  c->rank = rank;
  c->world = world;
  c->timeout_ms = timeout_ms > 0 ? timeout_ms : 30000;
  ncclUniqueId id;
  memcpy(&id, unique_id_128, sizeof(id));
  ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
  cfg.blocking = 0;  // so that a rank that never joins ends in DT_TIMEOUT instead of a hang
  ncclResult_t r = api.CommInitRankConfig(&c->comm, world, id, rank, &cfg);
  int st = (r == ncclSuccess || r == ncclInProgress) ? wait_nccl(c, ncclInProgress, c->timeout_ms) : DT_NCCL;
  if (st != DT_OK) {
    if (c->comm) api.CommAbort(c->comm);
    delete c;
    return st;
  }
  if (cudaStreamCreateWithFlags(&c->side, cudaStreamNonBlocking) != cudaSuccess) { delete c; return DT_CUDA; }
  for (int i = 0; i < kMaxChunks; ++i) cudaEventCreateWithFlags(&c->chunk_done[i], cudaEventDisableTiming);
  cudaEventCreateWithFlags(&c->all_done, cudaEventDisableTiming);
  *comm_out = c;
  return DT_OK;
}

int dt_comm_destroy(void* comm) {
  if (!comm) return DT_OK;
  Comm* c = reinterpret_cast<Comm*>(comm);
  NcclApi& api = nccl();
  if (c->side) cudaStreamSynchronize(c->side);
  for (int i = 0; i < c->n_regs; ++i)
    for (int r = 0; r < 8; ++r)
      if (c->regs[i].opened[r]) cudaIpcCloseMemHandle(c->regs[i].opened[r]);
  if (c->flag) cudaFree(c->flag);
  if (c->xchg) cudaFree(c->xchg);
  if (c->comm && api.ok) api.CommDestroy(c->comm);
  for (int i = 0; i < kMaxChunks; ++i) cudaEventDestroy(c->chunk_done[i]);
  if (c->all_done) cudaEventDestroy(c->all_done);
  if (c->side) cudaStreamDestroy(c->side);
  delete c;
  return DT_OK;
}

// Fused mode set-up: every rank hands the others an IPC handle of its output buffer, so that the attention
// epilogue can store O tiles straight into all ranks' [B,Sq,H,D] buffers over NVLink (ordinary peer stores).
int dt_comm_register_output(void* comm, void* o_full, size_t bytes) {
  if (!comm || !o_full || bytes == 0) return DT_BAD_ARG;
  Comm* c = reinterpret_cast<Comm*>(comm);
  NcclApi& api = nccl();
  if (!api.ok) return DT_NCCL;
  if (c->world > 8) return DT_UNSUPPORTED;
  if (c->n_regs >= Comm::kMaxRegs) return DT_UNSUPPORTED;
  if (c->world == 1) {
    Comm::Reg& r = c->regs[c->n_regs++];
    r.local = o_full; r.bytes = bytes; r.peer[0] = o_full;
    return DT_OK;
  }
  // allocation base of the buffer (a framework may hand out pieces of a larger allocation)
  typedef CUresult (*GetRangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);
  static GetRangeFn get_range = nullptr;
  if (!get_range) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &sym, cudaEnableDefault, &q) != cudaSuccess || !sym) return DT_CUDA;
    get_range = reinterpret_cast<GetRangeFn>(sym);
  }
  CUdeviceptr base = 0;
  size_t range = 0;
  if (get_range(&base, &range, (CUdeviceptr)o_full) != CUDA_SUCCESS) return DT_CUDA;
  IpcInfo mine;
  memset(&mine, 0, sizeof(mine));
  DT_CUDA_TRY(cudaIpcGetMemHandle(&mine.handle, reinterpret_cast<void*>(base)));
  mine.offset = (unsigned long long)((CUdeviceptr)o_full - base);
  mine.bytes = bytes;
  if (!c->xchg) DT_CUDA_TRY(cudaMalloc(&c->xchg, sizeof(IpcInfo) * 9));
  if (!c->flag) {
    DT_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&c->flag), 256));
    DT_CUDA_TRY(cudaMemset(c->flag, 0, 256));
  }
  IpcInfo* dev = reinterpret_cast<IpcInfo*>(c->xchg);
  DT_CUDA_TRY(cudaMemcpyAsync(dev + 8, &mine, sizeof(mine), cudaMemcpyHostToDevice, c->side));
  ncclResult_t r = api.AllGather(dev + 8, dev, sizeof(IpcInfo), ncclChar, c->comm, c->side);
  int st = wait_nccl(c, r, c->timeout_ms);
  if (st != DT_OK) return st;
  IpcInfo all[8];
  DT_CUDA_TRY(cudaMemcpyAsync(all, dev, sizeof(IpcInfo) * c->world, cudaMemcpyDeviceToHost, c->side));
  DT_CUDA_TRY(cudaStreamSynchronize(c->side));
  Comm::Reg& reg = c->regs[c->n_regs];
  reg = Comm::Reg();
  reg.local = o_full;
  reg.bytes = bytes;
  for (int q = 0; q < c->world; ++q) {
    if (all[q].bytes != bytes) return DT_BAD_ARG;  // every rank must register the same size
    if (q == c->rank) {
      reg.peer[q] = o_full;
      continue;
    }
    void* pb = nullptr;
    DT_CUDA_TRY(cudaIpcOpenMemHandle(&pb, all[q].handle, cudaIpcMemLazyEnablePeerAccess));
    reg.opened[q] = pb;
    reg.peer[q] = static_cast<char*>(pb) + all[q].offset;
  }
  ++c->n_regs;
  return DT_OK;
}

static size_t al256(size_t x) { return (x + 255) / 256 * 256; }

int dt_sdpa_headsharded_workspace_size(const dt_sdpa_params* local, int world, int chunks, size_t* bytes) {
  if (!local || !bytes || world <= 0 || chunks <= 0 || chunks > kMaxChunks) return DT_BAD_ARG;
  size_t inner = 0;
  int st = dt_sdpa_workspace_size(local, &inner);
  if (st != DT_OK) return st;
  const size_t slice = (size_t)local->B * local->Sq * local->Hq * local->D * dtype_size(local->dtype);
  // every chunk gets its own staging and gather region, so no region is reused while in flight
  *bytes = al256(inner) + al256(slice) + al256(slice * world) + 256 * (size_t)chunks * 2;
  return DT_OK;
}

int dt_sdpa_forward_headsharded(void* comm, const dt_sdpa_params* local, dt_tensor4 o_full, int chunks,
                                void* workspace, size_t workspace_bytes, void* cuda_stream) {
  if (!comm || !local || !o_full.ptr) return DT_BAD_ARG;
  Comm* c = reinterpret_cast<Comm*>(comm);
  NcclApi& api = nccl();
  if (!api.ok) return DT_NCCL;
  if (chunks <= 0 || chunks > kMaxChunks) return DT_BAD_ARG;
  // A row chunk is a call of its own with fewer query rows: that would shift the bottom-right causal diagonal and the
  // sliding window, and packed sequences cannot be cut at arbitrary rows.  Those calls run as one piece.
  if (local->is_causal || local->sliding_window > 0 || local->seq_offsets_q) chunks = 1;
  if (local->mask || local->lse) return DT_UNSUPPORTED;
  // ---- fused mode: o_full was registered on every rank -> the epilogue stores each O tile into all ranks'
  // buffers while the tensor cores work on the next tile; one small in-stream rendezvous ends the step ----
  for (int i = 0; i < c->n_regs; ++i) {
    const Comm::Reg& reg = c->regs[i];
    if (reg.local != o_full.ptr) continue;
    const size_t es = dtype_size(local->dtype);
    dt_sdpa_params p = *local;
    const size_t head_off = (size_t)c->rank * local->Hq * o_full.stride_h * es;
    p.o = o_full;
    p.o.ptr = static_cast<char*>(o_full.ptr) + head_off;
    if (!prefill_supported(p) || (p.flags & DT_FLAG_FORCE_GENERIC)) break;  // only the tensor-core kernel has the extra stores
    void* extra[8];
    int n_extra = 0;
    for (int q = 0; q < c->world; ++q)
      if (q != c->rank) extra[n_extra++] = static_cast<char*>(reg.peer[q]) + head_off;
    cudaStream_t fs = (cudaStream_t)cuda_stream;
    int st2 = DT_OK;
    if (c->world > 1 && c->last_fused_reg == i) {
      // The same buffer as in the previous call: a rank that runs ahead would store this call's tiles into a slower
      // rank's buffer while that rank's stream still reads the previous result.  A rendezvous in front of the kernel
      // holds every rank's stores back until all ranks' streams have got here, i.e. past their readers of the
      // previous result.  Callers that alternate between two registered buffers never pay for it: the rendezvous
      // that ended the call in between already gives that order.
      ncclResult_t r0 = api.AllReduce(c->flag, c->flag, 1, ncclInt, ncclSum, c->comm, fs);
      st2 = wait_nccl(c, r0, c->timeout_ms);
      if (st2 != DT_OK) return st2;
    }
    c->last_fused_reg = i;
    st2 = launch_prefill(p, fs, extra, n_extra);
    if (st2 != DT_OK) return st2;
    if (c->world > 1) {
      // kernel completion makes this rank's peer stores visible; after the rendezvous every rank's have landed
      ncclResult_t r = api.AllReduce(c->flag, c->flag, 1, ncclInt, ncclSum, c->comm, fs);
      st2 = wait_nccl(c, r, c->timeout_ms);
      if (st2 != DT_OK) return st2;
    }
    return DT_OK;
  }
  if (chunks > local->Sq) chunks = local->Sq;
  size_t need = 0, inner = 0;
  int st = dt_sdpa_headsharded_workspace_size(local, c->world, chunks, &need);
  if (st != DT_OK) return st;
  if (!workspace || workspace_bytes < need) return DT_WORKSPACE;
  dt_sdpa_workspace_size(local, &inner);
  cudaStream_t s = (cudaStream_t)cuda_stream;
  const size_t es = dtype_size(local->dtype);
  const int B = local->B, Hl = local->Hq, D = local->D;
  uint8_t* w = reinterpret_cast<uint8_t*>(workspace);
  void* inner_ws = w;
  uint8_t* stage = w + al256(inner);
  const size_t slice = (size_t)B * local->Sq * Hl * D * es;
  uint8_t* gath = stage + al256(slice);

  // Rows per chunk.  The attention kernel is persistent (one CTA per SM, work items of 256 query rows x one
  // head), so a chunk should hold a whole number of rounds over the SMs: round the rows up to a multiple of
  // 256 * sms / gcd(sms, B * heads), which may leave fewer chunks than asked for.
  int rows_per = (local->Sq + chunks - 1) / chunks;
  if (chunks > 1) {
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    long long x = sms, y = (long long)B * Hl;
    while (y) { long long r = x % y; x = y; y = r; }
    const long long unit = 256LL * (sms / x);
    long long rp = ((long long)rows_per + unit - 1) / unit * unit;
    rows_per = rp > local->Sq ? local->Sq : (int)rp;
  }
  size_t stage_off = 0, gath_off = 0;
  int ci = 0;
  for (int r0 = 0; r0 < local->Sq; r0 += rows_per, ++ci) {
    const int rows = local->Sq - r0 < rows_per ? local->Sq - r0 : rows_per;
    dt_sdpa_params p = *local;
    p.Sq = rows;
    p.q.ptr = reinterpret_cast<uint8_t*>(local->q.ptr) + (size_t)r0 * local->q.stride_s * es;
    p.o.ptr = stage + stage_off;
    p.o.stride_h = D;
    p.o.stride_s = (int64_t)Hl * D;
    p.o.stride_b = (int64_t)rows * Hl * D;
    st = dt_sdpa_forward(&p, inner_ws, inner, s);
    if (st != DT_OK) return st;
    DT_CUDA_TRY(cudaEventRecord(c->chunk_done[ci], s));
    DT_CUDA_TRY(cudaStreamWaitEvent(c->side, c->chunk_done[ci], 0));
    const size_t cbytes = (size_t)B * rows * Hl * D * es;
    ncclResult_t r = api.AllGather(stage + stage_off, gath + gath_off, cbytes, ncclChar, c->comm, c->side);
    st = wait_nccl(c, r, c->timeout_ms);
    if (st != DT_OK) return st;
    dt_tensor4 dst = o_full;
    dst.ptr = reinterpret_cast<uint8_t*>(o_full.ptr) + (size_t)r0 * o_full.stride_s * es;
    st = launch_permute_gathered(gath + gath_off, dst, c->world, B, rows, Hl, D, local->dtype, c->side);
    if (st != DT_OK) return st;
    stage_off += cbytes;
    gath_off += cbytes * c->world;
  }
  DT_CUDA_TRY(cudaEventRecord(c->all_done, c->side));
  DT_CUDA_TRY(cudaStreamWaitEvent(s, c->all_done, 0));
  return DT_OK;
}

// ---- head-sharded attention + output projection: row-parallel GEMM + reduce-scatter -----------------------

static int proj_rows_per_rank(int64_t M, int world) {
  const int64_t per = (M + world - 1) / world;
  return (int)((per + 127) / 128 * 128);  // whole 128-row tiles, so that a tile has one owner
}

int dt_sdpa_projected_headsharded_sizes(const dt_sdpa_params* local, int world, int C, size_t* workspace_bytes,
                                        size_t* recv_bytes, int* rows_per_rank) {
  if (!local || world <= 0 || world > 8 || C <= 0) return DT_BAD_ARG;
  if (local->dtype != DT_F16 && local->dtype != DT_BF16) return DT_UNSUPPORTED;
  if (C % 8 || ((int64_t)local->Hq * local->D) % 8) return DT_UNSUPPORTED;
  dt_sdpa_params t = *local;
  t.o = t.q;
  size_t inner = 0;
  int st = dt_sdpa_workspace_size(&t, &inner);
  if (st != DT_OK) return st;
  const int64_t M = (int64_t)local->B * local->Sq;
  const int rpr = proj_rows_per_rank(M, world);
  const size_t o_off = al256(inner) < 4096 ? 4096 : al256(inner);  // the ticket area stays clear
  if (workspace_bytes) *workspace_bytes = o_off + al256((size_t)M * local->Hq * local->D * 2) + al256((size_t)128 * C * 2);
  // two halves used alternately: a fast rank's next call must not overwrite slabs a slower rank is still summing
  if (recv_bytes) *recv_bytes = 2 * (size_t)world * rpr * C * sizeof(float);
  if (rows_per_rank) *rows_per_rank = rpr;
  return DT_OK;
}

int dt_sdpa_forward_projected_headsharded(void* comm, const dt_sdpa_params* local, const void* weight_local,
                                          const void* bias, int C, void* recv, dt_tensor4 out_rows, void* workspace,
                                          size_t workspace_bytes, void* cuda_stream) {
  if (!comm || !local || !weight_local || !recv || !out_rows.ptr) return DT_BAD_ARG;
  Comm* c = reinterpret_cast<Comm*>(comm);
  NcclApi& api = nccl();
  if (!api.ok) return DT_NCCL;
  size_t need = 0, recv_bytes = 0;
  int rpr = 0;
  int st = dt_sdpa_projected_headsharded_sizes(local, c->world, C, &need, &recv_bytes, &rpr);
  if (st != DT_OK) return st;
  if (!workspace || workspace_bytes < need) return DT_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(weight_local) % 16 || reinterpret_cast<uintptr_t>(recv) % 16 ||
      reinterpret_cast<uintptr_t>(out_rows.ptr) % 16 || out_rows.stride_s % 8)
    return DT_UNSUPPORTED;
  const Comm::Reg* reg = nullptr;
  for (int i = 0; i < c->n_regs; ++i)
    if (c->regs[i].local == recv) reg = &c->regs[i];
  if (!reg || reg->bytes < recv_bytes) return DT_BAD_ARG;  // recv must be registered on every rank (dt_comm_register_output)
  cudaStream_t s = (cudaStream_t)cuda_stream;
  // 1. local head slice -> [M, Kl] rows in the workspace
  dt_sdpa_params p = *local;
  dt_sdpa_params t = *local;
  t.o = t.q;
  size_t inner = 0;
  dt_sdpa_workspace_size(&t, &inner);
  const size_t o_off = al256(inner) < 4096 ? 4096 : al256(inner);
  const int64_t Kl = (int64_t)local->Hq * local->D;
  const int64_t M = (int64_t)local->B * local->Sq;
  uint8_t* w = static_cast<uint8_t*>(workspace);
  p.o.ptr = w + o_off;
  p.o.stride_h = local->D;
  p.o.stride_s = Kl;
  p.o.stride_b = Kl * local->Sq;
  st = dt_sdpa_forward(&p, workspace, o_off, s);
  if (st != DT_OK) return st;
  // 2. partial C = O_local . W_local^T, each 128-row tile stored (fp32) into slab [rank] of its owner's buffer
  const size_t half = (size_t)(c->proj_calls++ & 1) * ((size_t)c->world * rpr * C);  // floats
  float* slabs[8];
  for (int q = 0; q < c->world; ++q) slabs[q] = static_cast<float*>(reg->peer[q]) + half;
  dt_tensor4 a_view{p.o.ptr, Kl * M, Kl, Kl};
  dt_tensor4 scratch{w + o_off + al256((size_t)M * Kl * 2), (int64_t)C * 128, (int64_t)C, (int64_t)C};
  st = launch_out_proj_rowparallel(a_view, (int)M, (int)Kl, weight_local, C, scratch, local->dtype, slabs, c->world, c->rank,
                                   rpr, s);
  if (st != DT_OK) return st;
  // 3. rendezvous: kernel completion makes this rank's peer stores visible; after it every rank's have landed
  if (c->world > 1) {
    if (!c->flag) return DT_BAD_ARG;
    ncclResult_t r = api.AllReduce(c->flag, c->flag, 1, ncclInt, ncclSum, c->comm, s);
    st = wait_nccl(c, r, c->timeout_ms);
    if (st != DT_OK) return st;
  }
  // 4. this rank's rows: bias + sum of the slabs, rounded to the 16-bit type
  const int64_t row0 = (int64_t)c->rank * rpr;
  const int rows = (int)(M - row0 < 0 ? 0 : (M - row0 < rpr ? M - row0 : rpr));
  return launch_slab_reduce(static_cast<const float*>(recv) + half, bias, out_rows.ptr, out_rows.stride_s, c->world, rows, rpr, C,
                            local->dtype, s);
}

}  // extern "C"
