/*
 * sdpa_oracle.c -- plain-C fp32 restatement of the reference's CPU attention semantics.
 *
 * TEST INFRASTRUCTURE ONLY: used by tests/ as a second checker beside oracle/sdpa_oracle.py, and by
 * bench.py as the timed CPU baseline.  The shipped library never links or loads it.
 *
 * PARITY UNPINNED: the reference (drawthingsai/draw-things-community) holds no attention kernel; its CPU
 * back end lives in the un-vendored liuliu/ccv @ 023a9a894445493d8475711c0160be0bac8e6620.  This file
 * follows the explicit graphs the reference itself writes down:
 *   scores = (scale*Q) K^T, softmax over keys, P V      Libraries/SwiftDiffusion/Sources/Models/UNet.swift:217-265
 *   grouped KV heads (kv = h / (Hq/Hkv))                Llama.swift:74-96
 *   additive mask                                       CLIPTextModel.swift:57-70
 *   causal over a cache prefix (bottom-right aligned)   Libraries/SwiftLLM/Sources/Models/Qwen3_5.swift:183-196
 * The reference's CPU build threads with libdispatch (WORKSPACE.linux:128-129); this one uses pthreads
 * over (batch, head, row-block) work items.
 *
 * Build: see oracle/build_oracle.py (gcc -O3 -march=native -fopenmp-simd -shared -fPIC -pthread).
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

typedef struct {
  const float *q, *k, *v, *mask;
  float *o, *lse;
  int64_t q_sb, q_ss, q_sh, k_sb, k_ss, k_sh, v_sb, v_ss, v_sh, o_sb, o_ss, o_sh;
  int64_t m_sb, m_sh, m_sq;
  int B, Sq, Sk, Hq, Hkv, D;
  float scale;
  int is_causal;
  int row_block;
  int n_items;
  int next_item; /* atomic */
} job_t;

static void do_item(const job_t* J, int item, float* S, float* acc) {
  const int rb_per = (J->Sq + J->row_block - 1) / J->row_block;
  const int rb = item % rb_per;
  const int h = (item / rb_per) % J->Hq;
  const int b = item / (rb_per * J->Hq);
  const int G = J->Hq / J->Hkv;
  const int kvh = h / G;
  const int D = J->D, Sk = J->Sk;
  const int i0 = rb * J->row_block;
  const int i1 = i0 + J->row_block < J->Sq ? i0 + J->row_block : J->Sq;
  const float* Kb = J->k + b * J->k_sb + kvh * J->k_sh;
  const float* Vb = J->v + b * J->v_sb + kvh * J->v_sh;
  for (int i = i0; i < i1; ++i) {
    const float* qi = J->q + b * J->q_sb + (int64_t)i * J->q_ss + h * J->q_sh;
    float* Si = S;
    /* visible keys: j <= i + (Sk - Sq) when causal */
    int jmax = Sk;
    if (J->is_causal) {
      int64_t lim = (int64_t)i + (Sk - J->Sq) + 1;
      jmax = lim < 0 ? 0 : (lim > Sk ? Sk : (int)lim);
    }
    const float* mrow = J->mask ? J->mask + b * J->m_sb + h * J->m_sh + (int64_t)i * J->m_sq : NULL;
    float mx = -INFINITY;
    for (int j = 0; j < jmax; ++j) {
      const float* kj = Kb + (int64_t)j * J->k_ss;
      float dot = 0.f;
#pragma omp simd reduction(+ : dot)
      for (int d = 0; d < D; ++d) dot += (qi[d] * J->scale) * kj[d];
      if (mrow) dot += mrow[j];
      Si[j] = dot;
      mx = dot > mx ? dot : mx;
    }
    float* oi = J->o + b * J->o_sb + (int64_t)i * J->o_ss + h * J->o_sh;
    if (jmax == 0 || !(mx > -INFINITY)) { /* no visible key: zeros */
      for (int d = 0; d < D; ++d) oi[d] = 0.f;
      if (J->lse) J->lse[((int64_t)b * J->Hq + h) * J->Sq + i] = -INFINITY;
      continue;
    }
    float l = 0.f;
    for (int j = 0; j < jmax; ++j) {
      float e = expf(Si[j] - mx);
      Si[j] = e;
      l += e;
    }
    const float inv = 1.f / l;
    for (int d = 0; d < D; ++d) acc[d] = 0.f;
    for (int j = 0; j < jmax; ++j) {
      const float p = Si[j] * inv;
      const float* vj = Vb + (int64_t)j * J->v_ss;
#pragma omp simd
      for (int d = 0; d < D; ++d) acc[d] += p * vj[d];
    }
    for (int d = 0; d < D; ++d) oi[d] = acc[d];
    if (J->lse) J->lse[((int64_t)b * J->Hq + h) * J->Sq + i] = mx + logf(l);
  }
}

static void* worker(void* arg) {
  job_t* J = (job_t*)arg;
  float* S = (float*)malloc(sizeof(float) * (size_t)(J->Sk + 16));
  float* acc = (float*)malloc(sizeof(float) * (size_t)(J->D + 16));
  for (;;) {
    int item = __atomic_fetch_add(&J->next_item, 1, __ATOMIC_RELAXED);
    if (item >= J->n_items) break;
    do_item(J, item, S, acc);
  }
  free(S);
  free(acc);
  return NULL;
}

int sdpa_oracle_host_cores(void) { return (int)sysconf(_SC_NPROCESSORS_ONLN); }

/* All tensors fp32, element strides, D contiguous.  Query rows [row_begin, row_end) only (a sample of
 * the rows is how the largest shapes are checked and timed); pass 0, Sq for everything.  Returns the
 * number of threads used, or a negative value on a bad argument. */
int sdpa_oracle_f32(const float* q, const float* k, const float* v, float* o, float* lse, const float* mask,
                    const int64_t* strides /* q_sb,q_ss,q_sh,k_*,v_*,o_*,m_sb,m_sh,m_sq : 15 */,
                    int B, int Sq, int Sk, int Hq, int Hkv, int D, float scale, int is_causal,
                    int nthreads) {
  if (!q || !k || !v || !o || B <= 0 || Sq <= 0 || Sk <= 0 || Hq <= 0 || Hkv <= 0 || D <= 0 || Hq % Hkv) return -1;
  job_t J;
  memset(&J, 0, sizeof(J));
  J.q = q; J.k = k; J.v = v; J.o = o; J.lse = lse; J.mask = mask;
  J.q_sb = strides[0]; J.q_ss = strides[1]; J.q_sh = strides[2];
  J.k_sb = strides[3]; J.k_ss = strides[4]; J.k_sh = strides[5];
  J.v_sb = strides[6]; J.v_ss = strides[7]; J.v_sh = strides[8];
  J.o_sb = strides[9]; J.o_ss = strides[10]; J.o_sh = strides[11];
  J.m_sb = strides[12]; J.m_sh = strides[13]; J.m_sq = strides[14];
  J.B = B; J.Sq = Sq; J.Sk = Sk; J.Hq = Hq; J.Hkv = Hkv; J.D = D;
  J.scale = scale; J.is_causal = is_causal;
  J.row_block = 16;
  J.n_items = B * Hq * ((Sq + J.row_block - 1) / J.row_block);
  J.next_item = 0;
  if (nthreads <= 0) nthreads = sdpa_oracle_host_cores();
  if (nthreads > 256) nthreads = 256;
  if (nthreads > J.n_items) nthreads = J.n_items;
  pthread_t th[256];
  for (int t = 1; t < nthreads; ++t) pthread_create(&th[t], NULL, worker, &J);
  worker(&J);
  for (int t = 1; t < nthreads; ++t) pthread_join(th[t], NULL);
  return nthreads;
}
