// Shared declarations of the attention library: kernel launch prototypes and small device helpers.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/dtattn.h"

namespace dt {

// Per-device status word written by kernels whose bounded waits ran out (0 = healthy).
// Codes: 1 = TMA/full barrier wait, 2 = empty-slot wait, 3 = S-ready wait, 4 = P-ready wait,
//        5 = final-O wait.  The word keeps the first code stored.
unsigned int* device_status_word();  // device pointer for the current device (allocated once)

// Multiprocessor count of the current device (looked up once per device; 148 when there is no usable device).
int device_sm_count();

// Remember a failing cudaError_t for dt_last_cuda_error().
int record_cuda_error(cudaError_t e);

#define DT_CUDA_TRY(expr)                                   \
  do {                                                      \
    cudaError_t _e = (expr);                                \
    if (_e != cudaSuccess) return dt::record_cuda_error(_e); \
  } while (0)

inline size_t dtype_size(int dtype) { return dtype == DT_F32 ? 4 : 2; }

// ---- kernel entry points (each in its own .cu) --------------------------------------------------

// CUDA-core flash kernel: any D <= 256, any dtype, mask, causal, GQA.  Fallback and second opinion.
int launch_generic(const dt_sdpa_params& p, cudaStream_t stream);

// Argument rules every attention entry point shares (null or misaligned pointers, extents, NaN scale, negative
// window, variable-length bookkeeping): DT_OK, DT_BAD_ARG or DT_UNSUPPORTED.  Nothing is launched.
int validate_params(const dt_sdpa_params* p);

// Split-KV decode: Sq * (Hq/Hkv) <= 16 query rows per KV head, fp16/bf16, D in {64,128,256}.
bool decode_supported(const dt_sdpa_params& p);
size_t decode_workspace_bytes(const dt_sdpa_params& p);
int launch_decode(const dt_sdpa_params& p, void* workspace, size_t bytes, cudaStream_t stream);

// TMA + tcgen05 flash attention: fp16/bf16, D <= 128 (a multiple of 8), optional 16-byte aligned additive mask.
bool prefill_supported(const dt_sdpa_params& p);
// extra_outputs: up to 7 more [B,Sq,Hq,D] views with the same strides as p.o (other GPUs' buffers in the
// head-sharded mode) that receive a copy of every O tile.
int launch_prefill(const dt_sdpa_params& p, cudaStream_t stream, void* const* extra_outputs = nullptr, int n_extra = 0,
                   void* workspace = nullptr, size_t workspace_bytes = 0);
// Scratch of the masked variant: one byte per (32 query rows x 64 keys) patch of the mask, "has a non-zero entry".
size_t prefill_workspace_bytes(const dt_sdpa_params& p);

// Cross-attention over a short key/value sequence (Sk <= 96, head dim <= 64, the plain operator): three independent
// warpgroup pipelines per CTA, TMA + tcgen05.
bool short_kv_supported(const dt_sdpa_params& p);
int launch_short_kv(const dt_sdpa_params& p, cudaStream_t stream);

// C[B,S,N] = A[B,S,K] . W[N,K]^T + bias: the output projection behind the attention kernel (TMA + tcgen05 GEMM).
int launch_out_proj(const dt_tensor4& a_view, int B, int S, int K, const void* weight, const void* bias, int N,
                    const dt_tensor4& out, int dtype, cudaStream_t stream);

int launch_out_proj_rowparallel(const dt_tensor4& a_view, int M, int K, const void* weight, int N, const dt_tensor4& scratch_out,
                                int dtype, float* const* slabs, int world, int rank, int rows_per_rank, cudaStream_t stream);
int launch_slab_reduce(const float* recv, const void* bias, void* out, int64_t out_stride, int world, int rows,
                       int rows_per_rank, int N, int dtype, cudaStream_t stream);

// [world][rows][Hl][D] -> [B,Sq,world*Hl,D]
int launch_permute_gathered(const void* src, dt_tensor4 dst, int world, int B, int Sq, int Hl, int D,
                            int dtype, cudaStream_t stream);

// ---- device helpers -----------------------------------------------------------------------------

template <typename T>
__device__ __forceinline__ float to_float(T x);
template <>
__device__ __forceinline__ float to_float<float>(float x) { return x; }
template <>
__device__ __forceinline__ float to_float<__half>(__half x) { return __half2float(x); }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T>
__device__ __forceinline__ T from_float(float x);
template <>
__device__ __forceinline__ float from_float<float>(float x) { return x; }
template <>
__device__ __forceinline__ __half from_float<__half>(float x) { return __float2half_rn(x); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

}  // namespace dt
