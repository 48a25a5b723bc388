/*
 * dtattn.h -- C ABI of the B200 (sm_100a) scaled-dot-product-attention forward.
 *
 * This is the boundary a binding of the Draw Things operator
 *     NNC.ScaledDotProductAttention(scale:isCausal:hasAttentionMask:flags:...)
 * calls into.  The reference reaches its own arithmetic through s4nnc -> ccv (neither is vendored in
 * the reference tree), so each entry point below cites the reference call site whose behaviour it
 * replaces rather than a C prototype.
 *
 * Conventions
 *   - plain C types only; no exceptions; every function returns a dt_status (0 = OK, <0 = error).
 *   - all tensors are caller-owned DEVICE memory (except dt_sdpa_forward_host, which takes host
 *     memory); the library never takes ownership.  dt_sdpa_forward, dt_sdpa_decode_step, dt_qk_prologue and
 *     dt_sdpa_forward_projected allocate no device memory: scratch is the caller's workspace and the
 *     device status word is part of the library image.  (dt_sdpa_forward_host and the communicator
 *     set-up calls do allocate.)
 *   - tensors are 4-D views [B, S, H, D] ("BSHD", the layout every reference call site passes, e.g.
 *     Libraries/SwiftDiffusion/Sources/Models/UNet.swift:139-155) described by element strides; the
 *     innermost (D) stride is 1.  Strided views (row-offset views, batch strides larger than S*H*D)
 *     are honoured without a copy (Flux1.swift:236-243, UNet.swift:334-344).
 *   - work is enqueued on the given CUDA stream; no call synchronises the stream.
 *   - re-entrant across host threads and streams as long as each concurrent call has its own
 *     workspace.
 */
#ifndef DTATTN_H_
#define DTATTN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  DT_OK = 0,
  DT_BAD_ARG = -1,      /* null pointer, non-positive extent, Hq % Hkv != 0, misaligned base ...        */
  DT_UNSUPPORTED = -2,  /* valid request that no kernel of this build covers                            */
  DT_WORKSPACE = -3,    /* workspace missing or smaller than dt_sdpa_workspace_size reports             */
  DT_CUDA = -4,         /* a CUDA runtime/driver call failed (dt_last_cuda_error gives the code)        */
  DT_NCCL = -5,         /* NCCL missing or a collective failed                                          */
  DT_TIMEOUT = -6,      /* a bounded wait ran out (device status word or communicator set-up)           */
  DT_NO_DEVICE = -7,    /* no sm_100 device / library built without the kernel                          */
  DT_SCRATCH_LIMIT = -8 /* dt_sdpa_decode_noalloc: the request needs more than DT_NOALLOC_SCRATCH_BYTES  */
} dt_status;

typedef enum { DT_F16 = 0, DT_BF16 = 1, DT_F32 = 2 } dt_dtype;

/* A [B, S, H, D] view: element strides, D contiguous. */
typedef struct {
  void* ptr;
  int64_t stride_b, stride_s, stride_h;
} dt_tensor4;

/* dt_sdpa_params.flags */
#define DT_FLAG_FP16_ACCUM_HINT 1u /* reference flags:[.Float16] (UNet.swift:124); accepted, ignored: accumulation is always fp32 */
#define DT_FLAG_FORCE_GENERIC 2u   /* route to the CUDA-core kernel (second GPU opinion in tests)        */
#define DT_FLAG_KV_PREFIX_STABLE 4u /* decode over a KV cache: the kernel that precedes this call in the stream does
                                      not write the K/V rows this call streams (rows [0, Sk), or the cached prefix
                                      [0, Sk - T_new) of dt_sdpa_decode_step).  The decode kernel is then launched with
                                      programmatic stream serialization: its producer warp starts filling shared
                                      memory from the cache while the preceding kernel drains, and everything else
                                      (Q, new rows, workspace, outputs) waits for that kernel to complete.  Ignored by
                                      the other kernels. */
/* Split-KV decode tuning: fix the number of splits of every (batch, KV head) to n (1..256; 0 = the library's own
   choice, which fills the SMs once).  The value is part of what dt_sdpa_workspace_size depends on: pass the same
   flags to both calls.  Ignored by the other kernels. */
#define DT_FLAG_DECODE_SPLITS(n) ((((uint32_t)(n)) & 0xFFFu) << 16)

typedef struct {
  int32_t B, Sq, Sk, Hq, Hkv, D; /* Hq % Hkv == 0; query head h reads KV head h / (Hq/Hkv)
                                    (Libraries/SwiftDiffusion/Sources/Models/Llama.swift:74-96)          */
  int32_t dtype;                 /* dt_dtype of q, k, v, o and mask                                      */
  float scale;                   /* multiplies Q.K^T: 1 for FlashAttentionLevel.scale1, 1/sqrt(D) for
                                    .scaleMerged (Flux1.swift:224-232)                                   */
  int32_t is_causal;             /* bottom-right aligned: key j is visible to query i iff
                                    j <= i + (Sk - Sq) (Qwen3_5.swift:193-196: Sq new tokens over a
                                    cache prefix of Sk rows)                                             */
  uint32_t flags;
  dt_tensor4 q, k, v, o;
  /* optional additive mask, same dtype as q, logical shape [B or 1, Hq or 1, Sq, Sk]; a broadcast
     axis has stride 0 (CLIPTextModel.swift:46-51).  NULL = none.                                        */
  const void* mask;
  int64_t mask_stride_b, mask_stride_h, mask_stride_q;
  /* optional fp32 log-sum-exp output [B, Hq, Sq] (natural log of sum_j exp(scale*s_ij)), NULL = none   */
  float* lse;
  /* Operator variants (ScaledDotProductAttention(... hasAttentionSinks:, slidingWindow:, isVariableLength:,
     maxSequenceLength:)); all zero / NULL = the plain operator.
     sinks: one logit per query head, [Hq] in the tensors' dtype (the reference passes a [1,1,Hq,1] tensor cast to
       the queries' type, SwiftLLM/Sources/Models/DeepSeek4.swift:482-493): an extra score column without a value
       row, so row i's weights are exp(s_ij - m) / (sum_j exp(s_ij - m) + exp(sink_h - m)).  The scale is not
       applied to it.  lse, when asked for, includes the sink term.
     sliding_window W > 0: key j is visible to query i only if j > i + (Sk - Sq) - W (the last W keys up to and
       including the query's own position), on top of the causal rule when is_causal is set.
     seq_offsets_q / seq_offsets_k (device, int32, n_seq + 1 entries, first 0, non-decreasing): variable-length
       batches (SwiftLLM/Sources/Models/Qwen3_5VL.swift:428-437).  B must be 1; q and o hold sum(Sq_s) rows and
       k, v sum(Sk_s) rows; sequence s attends rows [off_q[s], off_q[s+1]) to rows [off_k[s], off_k[s+1]).  Sq and
       Sk are the packed row counts, max_seq_q / max_seq_k upper bounds of one sequence's rows.               */
  const void* sinks;
  int32_t sliding_window;
  int32_t n_seq, max_seq_q, max_seq_k;
  const int32_t* seq_offsets_q;
  const int32_t* seq_offsets_k;
} dt_sdpa_params;

/* Library / device ------------------------------------------------------------------------------ */

/* Human-readable name of a status code. */
const char* dt_status_string(int status);
/* cudaError_t value recorded by the last failing CUDA call on this host thread (0 if none). */
int dt_last_cuda_error(void);
/* Version of this ABI (bumped on incompatible change). */
int dt_abi_version(void);

/* Forward ----------------------------------------------------------------------------------------
 * Replaces the graph node the reference builds with
 *   ScaledDotProductAttention(scale:, isCausal:, hasAttentionMask:, flags:)(queries, keys, values[, mask])
 * at UNet.swift:139-155 (SD1.5 self-attention), UNetXL.swift:67-185 (SDXL cross-attention),
 * Flux1.swift:224-232 (MMDiT joint attention), Wan.swift:95-131 (video DiT) and
 * SwiftLLM/Sources/Models/Qwen3_5.swift:193-196 (GQA decode over the KV cache).
 */

/* Bytes of scratch dt_sdpa_forward needs for these params (0 is a valid answer). */
int dt_sdpa_workspace_size(const dt_sdpa_params* p, size_t* bytes);
/* Zero the workspace's ticket counters.  Call once after allocating a workspace (and again after any
   call that returned an error); dt_sdpa_forward leaves them zero on success. */
int dt_sdpa_workspace_init(void* workspace, size_t bytes, void* cuda_stream);
/* O = softmax(scale * Q K^T [+ mask] [causal]) V on `cuda_stream` of the current device. */
int dt_sdpa_forward(const dt_sdpa_params* p, void* workspace, size_t workspace_bytes, void* cuda_stream);
/* Which kernel dt_sdpa_forward would pick: writes a short static name ("prefill_tcgen05",
   "decode_splitkv", "generic") to *name. */
int dt_sdpa_kernel_name(const dt_sdpa_params* p, const char** name);

/* Same operator with HOST tensors: copies q, k, v (and sinks) to device scratch it owns, runs
 * dt_sdpa_forward, copies o (and lse) back and synchronises.  Masks and variable-length offsets
 * are refused with DT_UNSUPPORTED: they are served by the device-tensor entry point.  This is the call a host program makes
 * when its tensors live in host memory; it is the end-to-end path the benchmark times.  The scratch
 * is cached per host thread and released by dt_host_release().
 */
int dt_sdpa_forward_host(const dt_sdpa_params* p_host);
int dt_host_release(void);

/* Fused decode step ---------------------------------------------------------------------------------
 * One launch for what the reference's attention block does around the node in a KV-cache step
 * (Libraries/SwiftLLM/Sources/Models/Qwen3_5.swift:167-196):
 *     queries = Functional.cmul(queries, rotary rows of the last Sq tokens)          (:167-181)
 *     keys    = Functional.cmul(keys, rotary)                                        (:182)
 *     keys.moved(to: kIn[.., cachedTokenLength.., ..]); values.moved(to: vIn[...])   (:183-192)
 *     out = ScaledDotProductAttention(scale:, isCausal: true)(queries, kIn, vIn)     (:193-196)
 * attn.k / attn.v are the CACHE views [B, Sk, Hkv, D] with Sk = cached rows + T_new (the rows
 * [Sk - T_new, Sk) are written by this call); attn.q holds the un-rotated queries of the last Sq <= T_new
 * tokens; k_new / v_new are the un-rotated new rows [B, T_new, Hkv, D], T_new <= 16.  rotary is the
 * reference's table for the new tokens, [B or 1, T_new, D] in the tensors' dtype with (cos, sin) interleaved
 * on adjacent head dims (cmul multiplies (x[2i] + i x[2i+1]) by (cos_i + i sin_i)); NULL skips the rotation.
 * attn.is_causal must be 1 when Sq < T_new.  The rotated keys are rounded to the tensors' dtype before
 * they are attended to and stored, as the reference's separate cmul node does.  Same dtypes, head dims and
 * alignment rules as the "decode_splitkv" kernel; anything else returns DT_UNSUPPORTED.
 */
typedef struct {
  dt_sdpa_params attn;
  dt_tensor4 k_new, v_new;
  int32_t T_new;
  const void* rotary;
  int64_t rotary_stride_b, rotary_stride_s; /* stride_b 0 = one table for the whole batch */
  /* optional per-head RMSNorm of the queries and of the new keys before the rotation (qNorm / kNorm,
     Qwen3_5.swift:164-167): weights [D] in the tensors' dtype, y = x / sqrt(mean(x^2) + norm_eps) * weight, rounded to
     the dtype before the rotation as the separate node does.  NULL = that tensor is not normalised. */
  const void* q_norm_weight;
  const void* k_norm_weight;
  float norm_eps;
} dt_decode_step_params;
int dt_sdpa_decode_step_workspace_size(const dt_decode_step_params* s, size_t* bytes);
int dt_sdpa_decode_step(const dt_decode_step_params* s, void* workspace, size_t workspace_bytes,
                        void* cuda_stream);

/* Attention with the output projection folded in ---------------------------------------------------------
 * ScaledDotProductAttention(..., multiHeadOutputProjectionFused: true) (Libraries/SwiftDiffusion/Sources/Models/
 * UNet.swift:122-130; the operator then owns the "unify heads" Dense whose weight and bias are loaded at
 * UNet.swift:865-874): out[b, s, :] = concat_h(O[b, s, h, :]) . weight^T + bias.  weight is [C, Hq*D] row-major
 * (a Dense weight: outputs x inputs) and bias [C] (or NULL), both in the tensors' 16-bit dtype; out is a
 * [B, Sq, C] view given as dt_tensor4 (stride_b, stride_s; stride_h unused).  p->o is not written: the attention
 * output stays in the workspace (rounded to the 16-bit dtype, as the unfused graph's tensor would be) and the
 * projection, a TMA + tcgen05 GEMM on the same stream, reads it from there.  Hq*D and C must be multiples of 8.
 */
typedef struct {
  const void* weight;
  const void* bias;
  int32_t C;
  dt_tensor4 out;
} dt_out_proj;
int dt_sdpa_projected_workspace_size(const dt_sdpa_params* p, const dt_out_proj* proj, size_t* bytes);
int dt_sdpa_forward_projected(const dt_sdpa_params* p, const dt_out_proj* proj, void* workspace,
                              size_t workspace_bytes, void* cuda_stream);

/* Q/K prologue -----------------------------------------------------------------------------------------
 * The steps the reference runs on queries and keys immediately before the attention node, as one pass over HBM
 * instead of one graph node (a full read and write of the tensor) per step:
 *   RMSNorm(epsilon:, axis: [3]) per head row      Flux1.swift:164-181, Qwen3_5.swift:164-167
 *   RMSNorm(epsilon:, axis: [2]) over all h*k channels of a token    Wan.swift:86-91   (norm_per_token = 1)
 *   Functional.cmul(left:, right: rotary)          Flux1.swift:187-188, Wan.swift:92-93, Qwen3_5.swift:168-182
 *   multiplication by D^(-1/4)                     Wan.swift:94-97                      (post_scale)
 * y = post_scale * cmul(rmsnorm(x) * norm_weight, rotary); each step is skipped when its operand is NULL / 1 and
 * each step's result is rounded to `dtype` (DT_F16 or DT_BF16) before the next one, as separate 16-bit graph nodes
 * do.  x and y are [B, S, H, D] views (y may alias x, or be a row-offset view of a larger buffer, which fuses the
 * reference's concat of text and image tokens, Flux1.swift:184-186); D % 8 == 0, D <= 256, 16-byte aligned bases,
 * strides multiples of 8 elements.  rotary: [B or 1, S, H or 1, D] in `dtype`, (cos, sin) interleaved on adjacent
 * channels; a broadcast axis has stride 0.  norm_weight: [D], or [H*D] with norm_per_token.
 * dt_qk_prologue(q, k, stream) processes both tensors in one launch (k may be NULL).
 */
typedef struct {
  int32_t B, S, H, D;
  int32_t dtype;
  dt_tensor4 x, y;
  const void* norm_weight;
  int32_t norm_per_token;
  float eps;
  const void* rotary;
  int64_t rotary_stride_b, rotary_stride_s, rotary_stride_h;
  float post_scale; /* 0 is read as 1 */
} dt_qk_prologue_params;
int dt_qk_prologue(const dt_qk_prologue_params* q, const dt_qk_prologue_params* k, void* cuda_stream);

/* Sparse indexed attention --------------------------------------------------------------------------
 * SparseIndexedAttention(scale:, isCausal: true, hasAttentionSinks: true, slidingWindow:)(queries, rawKeys, rawValues,
 * compressedKeys, compressedValues, selectedRows, sinks) (Libraries/SwiftLLM/Sources/Models/DeepSeek4.swift:521-545,
 * called at :1080 and :1127): every query attends, in ONE softmax, to its sliding causal window of the raw key/value
 * rows and to the rows of a second, compressed key/value tensor that its list of selected rows names, plus the sink of
 * its head.  q, o: [B, Sq, Hq, D]; k_raw, v_raw: [B, Sr, Hkv, D] (query i sees raw rows j with j <= i + (Sr - Sq) when
 * is_causal, and j > i + (Sr - Sq) - sliding_window when sliding_window > 0); k_comp, v_comp: [B, Sc, Hkv, D] (may be
 * NULL when Sc == 0); selected: int32 [B or 1, Sq, n_selected] (strides in elements; stride_b 0 = one list for the
 * whole batch): an entry outside [0, Sc) means "no row", a row listed twice counts twice; sinks: [Hq] in the tensors'
 * dtype or NULL; lse: optional fp32 [B, Hq, Sq].  The reference's model uses one shared KV head for 64 query heads of
 * dim 512 with the same tensor as keys and values; here keys and values are separate views (pass the same pointer
 * twice for that layout: the gathered rows then serve as both), D <= 512, fp16 / bf16 / fp32.  16-bit tensors with D a
 * multiple of 64 and 16-byte aligned rows run on the tensor cores (a token's keys are shared out over a cluster of CTAs
 * when there are few tokens, i.e. in the decode step); everything else on a CUDA-core kernel.  The arithmetic of the
 * reference's operator is in its absent back end: "no row" for out-of-range entries and duplicates counting twice are
 * this library's definition.
 */
typedef struct {
  int32_t B, Sq, Hq, Hkv, D;
  int32_t Sr, Sc, n_selected;
  int32_t dtype;
  float scale;
  int32_t is_causal;
  int32_t sliding_window;
  dt_tensor4 q, o, k_raw, v_raw, k_comp, v_comp;
  const int32_t* selected;
  int64_t selected_stride_b, selected_stride_q;
  const void* sinks;
  float* lse;
  uint32_t flags; /* DT_FLAG_FORCE_GENERIC: the CUDA-core kernel instead of the tensor-core one */
} dt_sparse_indexed_params;
int dt_sparse_indexed_attention(const dt_sparse_indexed_params* p, void* cuda_stream);

/* Decode without any allocation ---------------------------------------------------------------------
 * No counterpart in the reference.  Some hosts of this library cannot obtain device memory at the moment
 * they call: a runtime that handed the whole device to its own allocator at start-up (the reference's graph
 * executor owns device memory this way) has nothing left for a late cudaMalloc, and inside a latency-bound
 * token loop a device allocation would also stall every stream while it runs.  For them this entry point
 * runs the split-KV decode kernel (the same shapes dt_sdpa_forward routes to "decode_splitkv": fp16/bf16,
 * D 64, 128 or 256, Sq * Hq/Hkv <= 16, no mask) with its partial results kept in a fixed array of
 * DT_NOALLOC_SCRATCH_BYTES that is part of the library image; each GPU that loads the library holds that
 * array until the process ends.  It calls no cudaMalloc, cudaFree or allocating library routine; the caller
 * still owns q, k, v, o (and lse).
 *   - A request whose partials do not fit returns DT_SCRATCH_LIMIT and launches nothing.
 *   - The first call on a device looks the array's address up (once per device, with that device current);
 *     make that first call outside of any stream capture.
 *   - All calls on a device share the one array and it keeps what the last call wrote.  The call clears the
 *     few words that must start at zero, on `cuda_stream`.  Two calls that overlap on the GPU (different
 *     streams, or different host threads without ordering) race on it: serialise them.
 *   - Arguments are checked exactly as dt_sdpa_forward checks them (null or misaligned pointers, NaN scale,
 *     negative window ...) before anything is launched.
 *   - A device-side wait that runs out is recorded in a status word of this entry point's own (inside the
 *     library image, not the one dt_device_status reads).  dt_sdpa_decode_noalloc_status copies it into *code
 *     and clears it (synchronises `cuda_stream`; allocates nothing): DT_OK with *code == 0 when every launch
 *     so far ran to its end, DT_TIMEOUT with the code otherwise, in which case the outputs of the calls since
 *     the last check are not to be trusted.
 */
#define DT_NOALLOC_SCRATCH_BYTES (8u << 20)
int dt_sdpa_decode_noalloc(const dt_sdpa_params* p, void* cuda_stream);
int dt_sdpa_decode_noalloc_status(void* cuda_stream, int* code);

/* Device status word ------------------------------------------------------------------------------
 * Kernels never spin without a bound: a wait that runs out stores a non-zero code into a per-device
 * status word and the kernel returns.  dt_device_status reads and clears it (synchronises `stream`).
 */
int dt_device_status(void* cuda_stream, int* code);

/* Head-sharded multi-GPU ---------------------------------------------------------------------------
 * No counterpart in the reference (it is single-GPU per process: Apps/gRPCServerCLI/
 * gRPCServerCLI.swift:291-292, ccv built with have_nccl = False at WORKSPACE.linux:127).  Rank r of
 * `world` owns query heads [r*Hq/world, (r+1)*Hq/world) and the KV heads they read.
 */
#define DT_NCCL_UNIQUE_ID_BYTES 128
/* Fill 128 bytes with an NCCL unique id (rank 0 calls this, then ships the bytes to every rank). */
int dt_comm_unique_id(void* id_out_128);
/* Create a communicator on the current device.  Returns DT_TIMEOUT when the other ranks do not join
   within timeout_ms. */
int dt_comm_init(void** comm, int rank, int world, const void* unique_id_128, int timeout_ms);
int dt_comm_destroy(void* comm);
/* Fused mode (optional): register this rank's full output buffer.  Collective: every rank calls it with a
 * buffer of the same size; the buffers are exchanged as CUDA IPC handles and mapped into every process.  A later
 * dt_sdpa_forward_headsharded whose o_full.ptr is a registered buffer stores each output tile straight into
 * all ranks' buffers from the attention kernel's epilogue (ordinary peer stores over NVLink, overlapped with
 * the tensor-core work) and ends with one small in-stream rendezvous, instead of all-gather + permute.
 * Up to 8 buffers per communicator, up to 8 ranks.
 * Ordering rule of the fused mode: a rank's stores land in the OTHER ranks' buffers, so whatever reads a buffer on
 * a rank must be ordered before the other ranks' next stores into it.  Readers enqueued on the stream that is passed
 * to dt_sdpa_forward_headsharded are: register two buffers and alternate between them, and the rendezvous that ends
 * the call in between gives that order for free; when two consecutive calls name the same buffer the library puts
 * one more rendezvous in front of the second call's kernel.  A reader on another stream must be joined to that
 * stream (an event) before the next call that stores into the buffer it reads. */
int dt_comm_register_output(void* comm, void* o_full, size_t bytes);
/* Run the local head slice (`local`: Hq and Hkv are the per-rank counts, o is ignored) and gather the
 * full output into o_full ([B, Sq, Hq*world, D], contiguous rows) on every rank.  `chunks` >= 1 splits
 * the query rows into that many pieces so the gather of one piece overlaps the attention of the next (causal,
 * sliding-window and variable-length calls always run as one piece; masks and lse are refused).
 * `workspace_bytes` must be at least dt_sdpa_headsharded_workspace_size.
 */
int dt_sdpa_headsharded_workspace_size(const dt_sdpa_params* local, int world, int chunks, size_t* bytes);
int dt_sdpa_forward_headsharded(void* comm, const dt_sdpa_params* local, dt_tensor4 o_full, int chunks,
                                void* workspace, size_t workspace_bytes, void* cuda_stream);

/* Head-sharded attention + output projection: row-parallel GEMM + reduce-scatter in one call (no counterpart in
 * the reference; this is what multiHeadOutputProjectionFused becomes when the heads are spread over GPUs).  Rank r
 * holds its head slice of q, k, v and the matching K-slice of the Dense weight, weight_local [C, Hq_local*D]
 * row-major.  The flattened output rows [B*Sq, C] are dealt out in blocks of *rows_per_rank (a multiple of 128):
 * rank r ends with rows [r*rows_per_rank, (r+1)*rows_per_rank) in out_rows ([rows, C], row stride
 * out_rows.stride_s), bias included.  recv is an fp32 buffer of *recv_bytes that every rank registered with
 * dt_comm_register_output: the GEMM epilogue stores each fp32 partial tile straight into slab [rank] of the owning
 * rank's recv buffer (ordinary stores, over NVLink for other ranks), one small in-stream rendezvous follows, and
 * the owner sums the slabs in rank order (the result does not depend on arrival order).  recv holds two sets of
 * slabs used by alternate calls, so a rank that runs ahead never overwrites what a slower rank is still summing;
 * all ranks must make the same sequence of calls. */
int dt_sdpa_projected_headsharded_sizes(const dt_sdpa_params* local, int world, int C, size_t* workspace_bytes,
                                        size_t* recv_bytes, int* rows_per_rank);
int dt_sdpa_forward_projected_headsharded(void* comm, const dt_sdpa_params* local, const void* weight_local,
                                          const void* bias, int C, void* recv, dt_tensor4 out_rows, void* workspace,
                                          size_t workspace_bytes, void* cuda_stream);

/* Layout helper used by the head-sharded path: src [world][B*Sq][Hl][D] (rank-major gather order)
 * -> dst view [B, Sq, world*Hl, D].  Exposed because a caller that gathers by other means needs it. */
int dt_permute_gathered(const void* src, dt_tensor4 dst, int world, int B, int Sq, int Hl, int D,
                        int dtype, void* cuda_stream);

#ifdef __cplusplus
}
#endif
#endif /* DTATTN_H_ */
