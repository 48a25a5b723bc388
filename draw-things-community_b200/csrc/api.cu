// C ABI of the attention library (include/dtattn.h): argument validation, kernel selection, workspace
// sizing, the host-tensor entry point and the gathered-layout permute.  No kernel math lives here.
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <mutex>

#include "sm100_ptx.cuh"

namespace dt {

// ---- error bookkeeping -------------------------------------------------------------------------------

static thread_local int g_last_cuda_error = 0;

int record_cuda_error(cudaError_t e) {
  g_last_cuda_error = (int)e;
  return DT_CUDA;
}

// ---- per-device status word --------------------------------------------------------------------------
// The word lives in the library image (one copy per device that loads the library), so no entry point has to
// allocate it.  In host code the array's name is a host-side stand-in: the device address comes from
// cudaGetSymbolAddress, once per device, with that device current.

static __device__ __align__(256) unsigned int g_status_storage[64];
static std::mutex g_status_mu;
static unsigned int* g_status_words[64] = {nullptr};

unsigned int* device_status_word() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lk(g_status_mu);
  if (!g_status_words[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_storage) != cudaSuccess) return nullptr;
    g_status_words[dev] = reinterpret_cast<unsigned int*>(p);  // zero-initialised when the module is loaded
  }
  return g_status_words[dev];
}

int device_sm_count() {
  static int counts[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    cudaGetLastError();
    return 148;
  }
  std::lock_guard<std::mutex> lk(g_status_mu);
  if (counts[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    counts[dev] = n;
  }
  return counts[dev];
}

// ---- tensor maps -------------------------------------------------------------------------------------

EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  });
  return fn;
}

namespace {
// Encoding a tensor map costs a driver call of about a microsecond; a decode step re-uses the same views
// thousands of times.  Small per-thread direct-mapped cache keyed by everything the encoding depends on.
struct MapKey {
  const void* ptr;
  int64_t sb, ss, sh;
  int B, S, H, D, dtype, box_rows;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && sb == o.sb && ss == o.ss && sh == o.sh && B == o.B && S == o.S && H == o.H && D == o.D &&
           dtype == o.dtype && box_rows == o.box_rows;
  }
};
struct MapEntry {
  MapKey key;
  CUtensorMap map;
  bool valid;
};
constexpr int kMapCacheSize = 64;
thread_local MapEntry g_map_cache[kMapCacheSize];

size_t map_hash(const MapKey& k) {
  size_t h = reinterpret_cast<size_t>(k.ptr) >> 4;
  h = h * 1000003u ^ (size_t)k.S;
  h = h * 1000003u ^ (size_t)k.box_rows;
  h = h * 1000003u ^ (size_t)k.ss;
  h = h * 1000003u ^ (size_t)k.B;
  return h;
}
}  // namespace

bool make_bshd_tensor_map(CUtensorMap* map, const dt_tensor4& t, int B, int S, int H, int D, int dtype,
                          int box_rows) {
  const MapKey key{t.ptr, t.stride_b, t.stride_s, t.stride_h, B, S, H, D, dtype, box_rows};
  MapEntry& slot = g_map_cache[map_hash(key) % kMapCacheSize];
  if (slot.valid && slot.key == key) {
    *map = slot.map;
    return true;
  }
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return false;
  if (dtype != DT_F16 && dtype != DT_BF16) return false;
  if (reinterpret_cast<uintptr_t>(t.ptr) % 16) return false;
  const cuuint64_t es = 2;
  // A dimension of extent 1 may carry any stride in the view; give TMA a legal one.
  auto stride_bytes = [&](int64_t s, int extent, cuuint64_t fallback) -> cuuint64_t {
    return extent == 1 ? fallback : (cuuint64_t)s * es;
  };
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)H, (cuuint64_t)S, (cuuint64_t)B};
  cuuint64_t sh = stride_bytes(t.stride_h, H, (cuuint64_t)D * es);
  cuuint64_t ss = stride_bytes(t.stride_s, S, sh * (cuuint64_t)H);
  cuuint64_t sb = stride_bytes(t.stride_b, B, ss * (cuuint64_t)S);
  cuuint64_t strides[3] = {sh, ss, sb};
  for (int i = 0; i < 3; ++i)
    if (strides[i] % 16 || strides[i] == 0 || strides[i] >= (1ull << 40)) return false;
  cuuint32_t box[4] = {64, 1, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(map, dtype == DT_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4,
                   t.ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  slot.key = key;
  slot.map = *map;
  slot.valid = true;
  return true;
}

// ---- validation and dispatch -------------------------------------------------------------------------

int validate_params(const dt_sdpa_params* p) {
  if (!p) return DT_BAD_ARG;
  if (p->B <= 0 || p->Sq <= 0 || p->Sk <= 0 || p->Hq <= 0 || p->Hkv <= 0 || p->D <= 0) return DT_BAD_ARG;
  if (p->Hq % p->Hkv) return DT_BAD_ARG;
  if (p->dtype != DT_F16 && p->dtype != DT_BF16 && p->dtype != DT_F32) return DT_BAD_ARG;
  if (!p->q.ptr || !p->k.ptr || !p->v.ptr || !p->o.ptr) return DT_BAD_ARG;
  if (!(p->scale == p->scale)) return DT_BAD_ARG;  // NaN
  const size_t es = dtype_size(p->dtype);
  const dt_tensor4* ts[4] = {&p->q, &p->k, &p->v, &p->o};
  for (auto t : ts)
    if (reinterpret_cast<uintptr_t>(t->ptr) % es) return DT_BAD_ARG;
  if (p->D > 256) return DT_UNSUPPORTED;
  if (p->sliding_window < 0) return DT_BAD_ARG;
  if (p->sinks && reinterpret_cast<uintptr_t>(p->sinks) % es) return DT_BAD_ARG;
  if (p->mask && reinterpret_cast<uintptr_t>(p->mask) % es) return DT_BAD_ARG;
  if (p->lse && reinterpret_cast<uintptr_t>(p->lse) % sizeof(float)) return DT_BAD_ARG;
  if ((p->seq_offsets_q != nullptr) != (p->seq_offsets_k != nullptr)) return DT_BAD_ARG;
  if (p->seq_offsets_q) {
    if (p->B != 1 || p->n_seq <= 0 || p->max_seq_q <= 0 || p->max_seq_k <= 0) return DT_BAD_ARG;
    if (p->max_seq_q > p->Sq || p->max_seq_k > p->Sk) return DT_BAD_ARG;
    if (p->mask) return DT_UNSUPPORTED;
  }
  return DT_OK;
}

enum Kernel { kGeneric = 0, kDecode = 1, kPrefill = 2, kShortKV = 3 };

static Kernel choose(const dt_sdpa_params& p) {
  if (p.flags & DT_FLAG_FORCE_GENERIC) return kGeneric;
  if (decode_supported(p) && p.Sk >= 256) return kDecode;
  // a short key/value sequence under many query rows: the dedicated streaming kernel (a handful of rows stays with
  // the kernels below, which need fewer resources per launch)
  if (short_kv_supported(p) && (long long)p.B * p.Hq * p.Sq >= 4096) return kShortKV;
  if (prefill_supported(p)) return kPrefill;
  if (decode_supported(p)) return kDecode;
  return kGeneric;
}

}  // namespace dt

using namespace dt;

extern "C" {

const char* dt_status_string(int status) {
  switch (status) {
    case DT_OK: return "ok";
    case DT_BAD_ARG: return "bad argument";
    case DT_UNSUPPORTED: return "unsupported shape, dtype or layout";
    case DT_WORKSPACE: return "workspace missing or too small";
    case DT_CUDA: return "CUDA call failed";
    case DT_NCCL: return "NCCL unavailable or failed";
    case DT_TIMEOUT: return "bounded wait ran out";
    case DT_NO_DEVICE: return "no usable sm_100 device";
    case DT_SCRATCH_LIMIT: return "request exceeds the built-in scratch of dt_sdpa_decode_noalloc";
  }
  return "unknown status";
}

int dt_last_cuda_error(void) { return g_last_cuda_error; }

int dt_abi_version(void) { return 2; }

int dt_sdpa_kernel_name(const dt_sdpa_params* p, const char** name) {
  int st = validate_params(p);
  if (st != DT_OK) return st;
  if (!name) return DT_BAD_ARG;
  static const char* names[4] = {"generic", "decode_splitkv", "prefill_tcgen05", "crossattn_short"};
  *name = names[choose(*p)];
  return DT_OK;
}

int dt_sdpa_workspace_size(const dt_sdpa_params* p, size_t* bytes) {
  int st = validate_params(p);
  if (st != DT_OK) return st;
  if (!bytes) return DT_BAD_ARG;
  const Kernel k = choose(*p);
  *bytes = k == kDecode ? decode_workspace_bytes(*p) : k == kPrefill ? prefill_workspace_bytes(*p) : 0;
  return DT_OK;
}

int dt_sdpa_workspace_init(void* workspace, size_t bytes, void* cuda_stream) {
  if (!workspace || bytes == 0) return DT_OK;
  DT_CUDA_TRY(cudaMemsetAsync(workspace, 0, bytes, (cudaStream_t)cuda_stream));
  return DT_OK;
}

int dt_sdpa_forward(const dt_sdpa_params* p, void* workspace, size_t workspace_bytes, void* cuda_stream) {
  int st = validate_params(p);
  if (st != DT_OK) return st;
  cudaStream_t stream = (cudaStream_t)cuda_stream;
  switch (choose(*p)) {
    case kDecode: return launch_decode(*p, workspace, workspace_bytes, stream);
    case kPrefill: return launch_prefill(*p, stream, nullptr, 0, workspace, workspace_bytes);
    case kShortKV: return launch_short_kv(*p, stream);
    default: return launch_generic(*p, stream);
  }
}

// ---- attention + output projection (multiHeadOutputProjectionFused) -------------------------------------

// The attention output of the projected call lives in the workspace: p->o may be null.
static dt_sdpa_params with_placeholder_o(const dt_sdpa_params* p) {
  dt_sdpa_params t = *p;
  t.o = t.q;
  return t;
}

static int validate_proj(const dt_sdpa_params* p_in, const dt_out_proj* proj) {
  if (!p_in) return DT_BAD_ARG;
  const dt_sdpa_params t = with_placeholder_o(p_in);
  const dt_sdpa_params* p = &t;
  int st = validate_params(p);
  if (st != DT_OK) return st;
  if (!proj || !proj->weight || !proj->out.ptr || proj->C <= 0) return DT_BAD_ARG;
  if (p->dtype != DT_F16 && p->dtype != DT_BF16) return DT_UNSUPPORTED;
  if (p->seq_offsets_q) return DT_UNSUPPORTED;
  const int64_t K = (int64_t)p->Hq * p->D;
  if (K % 8 || proj->C % 8) return DT_UNSUPPORTED;  // 16-byte rows for TMA
  auto al = [](const void* q) { return reinterpret_cast<uintptr_t>(q) % 16 == 0; };
  if (!al(proj->weight) || !al(proj->out.ptr) || proj->out.stride_b % 8 || proj->out.stride_s % 8) return DT_UNSUPPORTED;
  if (proj->bias && reinterpret_cast<uintptr_t>(proj->bias) % 2) return DT_BAD_ARG;
  return DT_OK;
}

static size_t align256(size_t x) { return (x + 255) / 256 * 256; }
// Where the attention output starts inside the workspace: behind the attention kernel's own scratch, and never
// inside the first 4 KB, which hold the split-KV ticket counters that every call must leave zeroed.
static size_t proj_o_offset(size_t inner) { return align256(inner) < 4096 ? 4096 : align256(inner); }

int dt_sdpa_projected_workspace_size(const dt_sdpa_params* p, const dt_out_proj* proj, size_t* bytes) {
  int st = validate_proj(p, proj);
  if (st != DT_OK) return st;
  if (!bytes) return DT_BAD_ARG;
  size_t inner = 0;
  const dt_sdpa_params t = with_placeholder_o(p);
  st = dt_sdpa_workspace_size(&t, &inner);
  if (st != DT_OK) return st;
  *bytes = proj_o_offset(inner) + align256((size_t)p->B * p->Sq * p->Hq * p->D * 2);
  return DT_OK;
}

int dt_sdpa_forward_projected(const dt_sdpa_params* p, const dt_out_proj* proj, void* workspace, size_t workspace_bytes,
                              void* cuda_stream) {
  int st = validate_proj(p, proj);
  if (st != DT_OK) return st;
  size_t need = 0, inner = 0;
  dt_sdpa_params q = with_placeholder_o(p);
  dt_sdpa_projected_workspace_size(p, proj, &need);
  dt_sdpa_workspace_size(&q, &inner);
  if (!workspace || workspace_bytes < need) return DT_WORKSPACE;
  // attention output, head-major rows [B, Sq, Hq*D], kept in the workspace: the GEMM reads it back from L2
  const int64_t K = (int64_t)p->Hq * p->D;
  q.o.ptr = static_cast<uint8_t*>(workspace) + proj_o_offset(inner);
  q.o.stride_h = p->D;
  q.o.stride_s = K;
  q.o.stride_b = K * p->Sq;
  st = dt_sdpa_forward(&q, workspace, proj_o_offset(inner), cuda_stream);
  if (st != DT_OK) return st;
  dt_tensor4 a_view{q.o.ptr, q.o.stride_b, q.o.stride_s, K};
  dt_tensor4 out = proj->out;
  out.stride_h = proj->C;
  return launch_out_proj(a_view, p->B, p->Sq, (int)K, proj->weight, proj->bias, proj->C, out, p->dtype,
                         (cudaStream_t)cuda_stream);
}

int dt_device_status(void* cuda_stream, int* code) {
  if (!code) return DT_BAD_ARG;
  unsigned int* w = device_status_word();
  if (!w) return DT_CUDA;
  unsigned int h = 0;
  cudaStream_t s = (cudaStream_t)cuda_stream;
  DT_CUDA_TRY(cudaMemcpyAsync(&h, w, sizeof(h), cudaMemcpyDeviceToHost, s));
  DT_CUDA_TRY(cudaStreamSynchronize(s));
  *code = (int)h;
  if (h) {
    DT_CUDA_TRY(cudaMemsetAsync(w, 0, sizeof(h), s));
    DT_CUDA_TRY(cudaStreamSynchronize(s));
    return DT_TIMEOUT;
  }
  return DT_OK;
}

// ---- host-tensor entry point -------------------------------------------------------------------------

namespace {
struct HostScratch {
  void* dev = nullptr;
  size_t dev_bytes = 0;
  void* ws = nullptr;
  size_t ws_bytes = 0;
  cudaStream_t stream = nullptr;
  cudaStream_t s_in = nullptr, s_out = nullptr;  // copy streams of the pipelined path
  cudaEvent_t ev_in[8] = {nullptr}, ev_done[8] = {nullptr};
};
thread_local HostScratch g_hs;

// Extent in elements of the smallest contiguous span that holds a [B,S,H,D] view.
size_t view_span(const dt_tensor4& t, int B, int S, int H, int D) {
  return (size_t)((B - 1) * t.stride_b + (S - 1) * t.stride_s + (H - 1) * t.stride_h + D);
}
}  // namespace

int dt_host_release(void) {
  if (g_hs.dev) cudaFree(g_hs.dev);
  if (g_hs.ws) cudaFree(g_hs.ws);
  if (g_hs.stream) cudaStreamDestroy(g_hs.stream);
  if (g_hs.s_in) cudaStreamDestroy(g_hs.s_in);
  if (g_hs.s_out) cudaStreamDestroy(g_hs.s_out);
  for (int i = 0; i < 8; ++i) {
    if (g_hs.ev_in[i]) cudaEventDestroy(g_hs.ev_in[i]);
    if (g_hs.ev_done[i]) cudaEventDestroy(g_hs.ev_done[i]);
  }
  g_hs = HostScratch();
  return DT_OK;
}

int dt_sdpa_forward_host(const dt_sdpa_params* ph) {
  int st = validate_params(ph);
  if (st != DT_OK) return st;
  // masks and variable-length offsets are served by the device-tensor entry point only
  if (ph->mask || ph->n_seq || ph->seq_offsets_q || ph->seq_offsets_k) return DT_UNSUPPORTED;
  dt_sdpa_params p = *ph;
  const size_t es = dtype_size(p.dtype);
  const size_t nq = view_span(p.q, p.B, p.Sq, p.Hq, p.D) * es, nk = view_span(p.k, p.B, p.Sk, p.Hkv, p.D) * es;
  const size_t nv = view_span(p.v, p.B, p.Sk, p.Hkv, p.D) * es, no = view_span(p.o, p.B, p.Sq, p.Hq, p.D) * es;
  auto al = [](size_t x) { return (x + 255) / 256 * 256; };
  const size_t nl = p.lse ? al((size_t)p.B * p.Hq * p.Sq * 4) : 0;
  const size_t nsink = p.sinks ? (size_t)p.Hq * es : 0;
  const size_t total = al(nq) + al(nk) + al(nv) + al(no) + nl + al(nsink);
  if (!g_hs.stream) DT_CUDA_TRY(cudaStreamCreateWithFlags(&g_hs.stream, cudaStreamNonBlocking));
  if (g_hs.dev_bytes < total) {
    if (g_hs.dev) cudaFree(g_hs.dev);
    g_hs.dev = nullptr;
    g_hs.dev_bytes = 0;
    DT_CUDA_TRY(cudaMalloc(&g_hs.dev, total));
    g_hs.dev_bytes = total;
  }
  uint8_t* d = reinterpret_cast<uint8_t*>(g_hs.dev);
  p.q.ptr = d; d += al(nq);
  p.k.ptr = d; d += al(nk);
  p.v.ptr = d; d += al(nv);
  p.o.ptr = d; d += al(no);
  if (p.lse) p.lse = reinterpret_cast<float*>(d);
  d += nl;
  if (p.sinks) p.sinks = d;
  size_t wsb = 0;
  st = dt_sdpa_workspace_size(&p, &wsb);
  if (st != DT_OK) return st;
  if (wsb > g_hs.ws_bytes) {
    if (g_hs.ws) cudaFree(g_hs.ws);
    g_hs.ws = nullptr;
    g_hs.ws_bytes = 0;
    DT_CUDA_TRY(cudaMalloc(&g_hs.ws, wsb));
    g_hs.ws_bytes = wsb;
    DT_CUDA_TRY(cudaMemsetAsync(g_hs.ws, 0, wsb, g_hs.stream));
  }
  cudaStream_t s = g_hs.stream;
  if (nsink) DT_CUDA_TRY(cudaMemcpyAsync(const_cast<void*>(p.sinks), ph->sinks, nsink, cudaMemcpyHostToDevice, s));
  // Pipelined path for the large tensor-core shapes: heads are independent, so the host->device copy of one
  // group of heads overlaps the attention of the previous group and the device->host copy of the one before
  // (three streams, both copy engines busy).  Needs heads contiguous inside a token row and regular rows.
  {
    const int G = p.Hq / p.Hkv;
    int groups = 0;
    for (int g : {8, 6, 4, 3, 2})
      if (p.Hkv % g == 0) { groups = g; break; }
    auto regular = [&](const dt_tensor4& t, int S, int H) {
      return t.stride_h == p.D && t.stride_s >= (int64_t)H * p.D && (p.B == 1 || t.stride_b == (int64_t)S * t.stride_s);
    };
    const bool big = nq + nk + nv >= (size_t)(16u << 20);
    const bool pipelined = big && !p.lse && choose(p) == kPrefill && regular(p.q, p.Sq, p.Hq) &&
                           regular(p.k, p.Sk, p.Hkv) && regular(p.v, p.Sk, p.Hkv) && regular(p.o, p.Sq, p.Hq);
    if (pipelined && !g_hs.s_in) {
      DT_CUDA_TRY(cudaStreamCreateWithFlags(&g_hs.s_in, cudaStreamNonBlocking));
      DT_CUDA_TRY(cudaStreamCreateWithFlags(&g_hs.s_out, cudaStreamNonBlocking));
      for (int i = 0; i < 8; ++i) {
        DT_CUDA_TRY(cudaEventCreateWithFlags(&g_hs.ev_in[i], cudaEventDisableTiming));
        DT_CUDA_TRY(cudaEventCreateWithFlags(&g_hs.ev_done[i], cudaEventDisableTiming));
      }
    }
    // One image, every query row sees every key (the diffusion shapes): K and V go up whole as two linear copies,
    // then the queries in runs of whole 256-row work items, each run attended and sent back while the next one is
    // on the bus.  Linear copies of full token rows move faster than the per-head-group 2-D copies below, and the
    // runs shrink towards the end so that little work is left once the last query row has arrived.
    constexpr int kItemRows = 256;
    const int items = p.Sq / kItemRows;  // a ragged tail stays with the last run
    if (pipelined && p.B == 1 && !p.is_causal && p.sliding_window == 0 && items >= 4 &&
        p.q.stride_s == (int64_t)p.Hq * p.D && p.o.stride_s == (int64_t)p.Hq * p.D) {
      int dev = 0, sms = 0;
      cudaGetDevice(&dev);
      if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
      int per = std::max(1, sms / p.Hq);  // items of one run: one wave of the persistent kernel
      if ((items + per - 1) / per > 6) per = (items + 5) / 6;
      int runs[8], n_runs = 0, left = items;
      while (left > per + per / 2) { runs[n_runs++] = per; left -= per; }
      if (left >= 3) { runs[n_runs++] = (2 * left + 2) / 3; left -= runs[n_runs - 1]; }
      runs[n_runs++] = left;
      bool same_kernel = true;  // every run must take the tensor-core kernel within the workspace sized for the whole
      for (int c = 0, r = 0; c < n_runs; ++c) {
        dt_sdpa_params pc = p;
        pc.Sq = c + 1 < n_runs ? runs[c] * kItemRows : p.Sq - r;
        r += pc.Sq;
        size_t w = 0;
        same_kernel = same_kernel && choose(pc) == kPrefill && dt_sdpa_workspace_size(&pc, &w) == DT_OK && w <= g_hs.ws_bytes;
      }
      if (same_kernel) {
      DT_CUDA_TRY(cudaMemcpyAsync(p.k.ptr, ph->k.ptr, nk, cudaMemcpyHostToDevice, g_hs.s_in));
      DT_CUDA_TRY(cudaMemcpyAsync(p.v.ptr, ph->v.ptr, nv, cudaMemcpyHostToDevice, g_hs.s_in));
      const size_t row_bytes = (size_t)p.Hq * p.D * es;
      int r0 = 0;
      for (int c = 0; c < n_runs; ++c) {
        const int rows = c + 1 < n_runs ? runs[c] * kItemRows : p.Sq - r0;
        DT_CUDA_TRY(cudaMemcpyAsync(static_cast<char*>(p.q.ptr) + r0 * row_bytes,
                                    static_cast<const char*>(ph->q.ptr) + r0 * row_bytes, rows * row_bytes,
                                    cudaMemcpyHostToDevice, g_hs.s_in));
        DT_CUDA_TRY(cudaEventRecord(g_hs.ev_in[c], g_hs.s_in));
        DT_CUDA_TRY(cudaStreamWaitEvent(s, g_hs.ev_in[c], 0));
        dt_sdpa_params pc = p;
        pc.Sq = rows;
        pc.q.ptr = static_cast<char*>(p.q.ptr) + r0 * row_bytes;
        pc.o.ptr = static_cast<char*>(p.o.ptr) + r0 * row_bytes;
        st = dt_sdpa_forward(&pc, g_hs.ws, g_hs.ws_bytes, s);
        if (st != DT_OK) return st;
        DT_CUDA_TRY(cudaEventRecord(g_hs.ev_done[c], s));
        DT_CUDA_TRY(cudaStreamWaitEvent(g_hs.s_out, g_hs.ev_done[c], 0));
        DT_CUDA_TRY(cudaMemcpyAsync(static_cast<char*>(ph->o.ptr) + r0 * row_bytes,
                                    static_cast<const char*>(p.o.ptr) + r0 * row_bytes, rows * row_bytes,
                                    cudaMemcpyDeviceToHost, g_hs.s_out));
        r0 += rows;
      }
      DT_CUDA_TRY(cudaStreamSynchronize(g_hs.s_out));
      DT_CUDA_TRY(cudaStreamSynchronize(s));
      return DT_OK;
      }
    }
    if (groups >= 2 && pipelined) {
      const int hk = p.Hkv / groups, hq = hk * G;
      auto copy2d = [&](void* dst, const void* src, const dt_tensor4& t, int S, int heads, int h0, cudaMemcpyKind kind,
                        cudaStream_t cs) {
        const size_t off = (size_t)h0 * p.D * es;
        return cudaMemcpy2DAsync(static_cast<char*>(dst) + off, (size_t)t.stride_s * es,
                                 static_cast<const char*>(src) + off, (size_t)t.stride_s * es, (size_t)heads * p.D * es,
                                 (size_t)p.B * S, kind, cs);
      };
      for (int g = 0; g < groups; ++g) {
        DT_CUDA_TRY(copy2d(p.k.ptr, ph->k.ptr, p.k, p.Sk, hk, g * hk, cudaMemcpyHostToDevice, g_hs.s_in));
        DT_CUDA_TRY(copy2d(p.v.ptr, ph->v.ptr, p.v, p.Sk, hk, g * hk, cudaMemcpyHostToDevice, g_hs.s_in));
        DT_CUDA_TRY(copy2d(p.q.ptr, ph->q.ptr, p.q, p.Sq, hq, g * hq, cudaMemcpyHostToDevice, g_hs.s_in));
        DT_CUDA_TRY(cudaEventRecord(g_hs.ev_in[g], g_hs.s_in));
        DT_CUDA_TRY(cudaStreamWaitEvent(s, g_hs.ev_in[g], 0));
        dt_sdpa_params pg = p;
        pg.Hq = hq;
        pg.Hkv = hk;
        pg.q.ptr = static_cast<char*>(p.q.ptr) + (size_t)g * hq * p.D * es;
        pg.k.ptr = static_cast<char*>(p.k.ptr) + (size_t)g * hk * p.D * es;
        pg.v.ptr = static_cast<char*>(p.v.ptr) + (size_t)g * hk * p.D * es;
        pg.o.ptr = static_cast<char*>(p.o.ptr) + (size_t)g * hq * p.D * es;
        if (p.sinks) pg.sinks = static_cast<const char*>(p.sinks) + (size_t)g * hq * es;
        st = dt_sdpa_forward(&pg, g_hs.ws, g_hs.ws_bytes, s);
        if (st != DT_OK) return st;
        DT_CUDA_TRY(cudaEventRecord(g_hs.ev_done[g], s));
        DT_CUDA_TRY(cudaStreamWaitEvent(g_hs.s_out, g_hs.ev_done[g], 0));
        DT_CUDA_TRY(copy2d(ph->o.ptr, p.o.ptr, p.o, p.Sq, hq, g * hq, cudaMemcpyDeviceToHost, g_hs.s_out));
      }
      DT_CUDA_TRY(cudaStreamSynchronize(g_hs.s_out));
      DT_CUDA_TRY(cudaStreamSynchronize(s));
      return DT_OK;
    }
  }
  DT_CUDA_TRY(cudaMemcpyAsync(p.q.ptr, ph->q.ptr, nq, cudaMemcpyHostToDevice, s));
  DT_CUDA_TRY(cudaMemcpyAsync(p.k.ptr, ph->k.ptr, nk, cudaMemcpyHostToDevice, s));
  DT_CUDA_TRY(cudaMemcpyAsync(p.v.ptr, ph->v.ptr, nv, cudaMemcpyHostToDevice, s));
  // A strided output view has gaps the kernel never writes: carry the host's bytes through them.
  if (no != (size_t)p.B * p.Sq * p.Hq * p.D * es) DT_CUDA_TRY(cudaMemcpyAsync(p.o.ptr, ph->o.ptr, no, cudaMemcpyHostToDevice, s));
  st = dt_sdpa_forward(&p, g_hs.ws, g_hs.ws_bytes, s);
  if (st != DT_OK) return st;
  DT_CUDA_TRY(cudaMemcpyAsync(ph->o.ptr, p.o.ptr, no, cudaMemcpyDeviceToHost, s));
  if (p.lse) DT_CUDA_TRY(cudaMemcpyAsync(ph->lse, p.lse, (size_t)p.B * p.Hq * p.Sq * 4, cudaMemcpyDeviceToHost, s));
  DT_CUDA_TRY(cudaStreamSynchronize(s));
  return DT_OK;
}

int dt_permute_gathered(const void* src, dt_tensor4 dst, int world, int B, int Sq, int Hl, int D, int dtype,
                        void* cuda_stream) {
  if (!src || !dst.ptr || world <= 0 || B <= 0 || Sq <= 0 || Hl <= 0 || D <= 0) return DT_BAD_ARG;
  return launch_permute_gathered(src, dst, world, B, Sq, Hl, D, dtype, (cudaStream_t)cuda_stream);
}

}  // extern "C"
