/*
 * CPU oracle for paged attention over a block-table KV cache.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the shipped library links, loads or
 * calls this file; only the test-suite, the smoke check and the benchmark's
 * CPU-baseline leg do, and there only as the checker / the reported baseline.
 *
 * PARITY UNPINNED at the kernel boundary: the reference holds no golden vector,
 * known-answer test or fixture for the numerical result of reshape_and_cache,
 * paged_attention or copy_blocks (its kernel tests build parameter structs
 * only), and none of its implementations can be built or run outside macOS /
 * MLX.  The integer index arithmetic below is a line-by-line restatement of
 * the reference kernels; the attention arithmetic restates the reference's
 * software path at the semantic level (exact softmax) in higher precision.
 *
 * Pool layouts (crates/mlx-paged-attn/src/cache_engine.rs:58-106,
 * crates/mlx-sys/src/mlx.cpp:3838-3863):
 *   key   cache [num_blocks, num_kv_heads, head_size/x, block_size, x]
 *   value cache [num_blocks, num_kv_heads, head_size, block_size]
 * Elements are 16-bit (bf16 / f16 bit patterns); x = 8 for 16-bit types.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* bf16 helpers, matching crates/mlx-paged-attn/metal/utils.metal:14-33
 * (NaN -> 0x7FC0; round to nearest even by adding 0x7FFF + lsb). */
static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
static inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7FC0;
  u += ((u >> 16) & 1u) + 0x7FFFu;
  return (uint16_t)(u >> 16);
}

/* f16 bit pattern -> float (cache dtype 0); exact. */
static inline float f16_to_f32(uint16_t h) {
  _Float16 v;
  memcpy(&v, &h, 2);
  return (float)v;
}
static inline float elem_to_f32(uint16_t bits, int is_f16) {
  return is_f16 ? f16_to_f32(bits) : bf16_to_f32(bits);
}

int oracle_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* Launchers such as torchrun export OMP_NUM_THREADS=1; the timed baseline asks for
 * the host's cores explicitly. */
void oracle_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

void oracle_f32_to_bf16(const float *src, uint16_t *dst, int64_t n) {
  for (int64_t i = 0; i < n; i++) dst[i] = f32_to_bf16(src[i]);
}
void oracle_bf16_to_f32(const uint16_t *src, float *dst, int64_t n) {
  for (int64_t i = 0; i < n; i++) dst[i] = bf16_to_f32(src[i]);
}

/* ------------------------------------------------------------------------ */
/* KV block write.  crates/mlx-paged-attn/metal/cache/reshape_and_cache.metal
 * :58-97 (non-fp8 branch): one token per outer iteration, slot < 0 skipped,
 * block = slot / block_size, offset = slot % block_size, then for every
 * i in [0, num_heads*head_size) the two destination index formulas.        */
void oracle_reshape_and_cache(const uint16_t *key, const uint16_t *value,
                              uint16_t *key_cache, uint16_t *value_cache,
                              const int64_t *slot_mapping, int64_t num_tokens,
                              int64_t key_stride, int64_t value_stride,
                              int num_heads, int head_size, int block_size,
                              int x) {
  for (int64_t token_idx = 0; token_idx < num_tokens; token_idx++) {
    const int64_t slot_idx = slot_mapping[token_idx];
    if (slot_idx < 0) continue;
    const int64_t block_idx = slot_idx / block_size;
    const int64_t block_offset = slot_idx % block_size;
    const int n = num_heads * head_size;
    for (int i = 0; i < n; i++) {
      const int64_t src_key_idx = token_idx * key_stride + i;
      const int64_t src_value_idx = token_idx * value_stride + i;
      const int head_idx = i / head_size;
      const int head_offset = i % head_size;
      const int x_idx = head_offset / x;
      const int x_offset = head_offset % x;
      const int64_t tgt_key_idx =
          block_idx * num_heads * (head_size / x) * block_size * x +
          (int64_t)head_idx * (head_size / x) * block_size * x +
          (int64_t)x_idx * block_size * x + block_offset * x + x_offset;
      const int64_t tgt_value_idx =
          block_idx * num_heads * head_size * block_size +
          (int64_t)head_idx * head_size * block_size +
          (int64_t)head_offset * block_size + block_offset;
      key_cache[tgt_key_idx] = key[src_key_idx];
      value_cache[tgt_value_idx] = value[src_value_idx];
    }
  }
}

/* Block-to-block copy of K and V (copy-on-write).
 * crates/mlx-paged-attn/metal/cache/copy_blocks.metal:6-36: pairs are
 * (src, dst) int64, processed in pair order.                               */
void oracle_copy_blocks(uint16_t *key_cache, uint16_t *value_cache,
                        const int64_t *block_mapping, int64_t num_pairs,
                        int64_t numel_per_block) {
  for (int64_t p = 0; p < num_pairs; p++) {
    const int64_t src = block_mapping[2 * p] * numel_per_block;
    const int64_t dst = block_mapping[2 * p + 1] * numel_per_block;
    for (int64_t i = 0; i < numel_per_block; i++) key_cache[dst + i] = key_cache[src + i];
    for (int64_t i = 0; i < numel_per_block; i++) value_cache[dst + i] = value_cache[src + i];
  }
}

/* ------------------------------------------------------------------------ */
/* Address of element (token t, head h, dim d) of one sequence, read through
 * the block table exactly as the kernels do
 * (crates/mlx-paged-attn/metal/attention/paged_attention.metal:890-929 for K,
 * :1041-1070 for V): physical block = table[t / BS] promoted to 64 bit.     */
static inline int64_t k_index(const int32_t *table, int64_t t, int h, int d,
                              int Hkv, int D, int BS, int x) {
  const int64_t blk = (int64_t)(uint32_t)table[t / BS];
  const int off = (int)(t % BS);
  return blk * Hkv * D * BS + (int64_t)h * D * BS + (int64_t)(d / x) * BS * x +
         (int64_t)off * x + (d % x);
}
static inline int64_t v_index(const int32_t *table, int64_t t, int h, int d,
                              int Hkv, int D, int BS) {
  const int64_t blk = (int64_t)(uint32_t)table[t / BS];
  const int off = (int)(t % BS);
  return blk * Hkv * D * BS + (int64_t)h * D * BS + (int64_t)d * BS + off;
}

/* One output row of paged attention: query vector qp (bf16, D values) of
 * query head hq against the first n keys of a sequence read through `table`.
 * logit/acc are caller-provided scratch (n and D doubles).                  */
static void attend_row(float *o, const uint16_t *qp, const uint16_t *k_cache,
                       const uint16_t *v_cache, const int32_t *table, int n,
                       int h, int Hkv, int D, int BS, float scale,
                       float softcap, double *logit, double *acc, int is_f16) {
  const int x = 8;
  if (n <= 0) {
    for (int d = 0; d < D; d++) o[d] = 0.f;
    return;
  }
  double mx = -INFINITY;
  for (int t = 0; t < n; t++) {
    const int64_t kb = k_index(table, t, h, 0, Hkv, D, BS, x);
    double dot = 0.0;
    for (int c = 0; c < D / x; c++)
      for (int e = 0; e < x; e++)
        dot += (double)elem_to_f32(qp[c * x + e], is_f16) *
               (double)elem_to_f32(k_cache[kb + (int64_t)c * BS * x + e], is_f16);
    double l = dot * (double)scale;
    if (softcap != 1.0f) l = tanh(l / (double)softcap) * (double)softcap;
    logit[t] = l;
    if (l > mx) mx = l;
  }
  double sum = 0.0;
  for (int t = 0; t < n; t++) {
    logit[t] = exp(logit[t] - mx);
    sum += logit[t];
  }
  for (int d = 0; d < D; d++) acc[d] = 0.0;
  for (int t = 0; t < n; t++) {
    const double p = logit[t];
    const int64_t vb = v_index(table, t, h, 0, Hkv, D, BS);
    for (int d = 0; d < D; d++)
      acc[d] += p * (double)elem_to_f32(v_cache[vb + (int64_t)d * BS], is_f16);
  }
  for (int d = 0; d < D; d++) o[d] = (float)(acc[d] / sum);
}

/* Variable-length paged attention, the semantic oracle.
 *
 * Sequence s holds kv_len = context_lens[s] tokens in the pool and
 * q_len = cu_q_lens[s+1]-cu_q_lens[s] query tokens that occupy the last q_len
 * positions; query j attends keys [0, kv_len - q_len + j].  q_len = 1 is the
 * reference decode (crates/mlx-sys/src/mlx.cpp:4080-4156: gather by table,
 * trim to context_len, kv_head = q_head / G, scores*scale, softmax, @V;
 * context_len == 0 -> zeros, :4084-4088).  q_len > 1 is dense causal
 * attention over prefix+chunk (the "causal" mode of
 * crates/mlx-sys/src/mlx.cpp:1403-1407).  Optional soft-capping follows
 * paged_attention.metal:937-940 (applied when softcap != 1).
 *
 * Inputs are bf16 bit patterns; logits, softmax and the P.V sum are fp64, so
 * the result is the exact-arithmetic answer for the given bf16 inputs up to
 * fp64 rounding.  The Metal kernel's "+1e-6" in the normaliser and its
 * rounding of P to the storage type are deliberately not reproduced.
 * Output: fp32 [total_q, Hq, D].  cu_q_lens == NULL means one query/seq.   */
void oracle_paged_attention_varlen_dt(float *out, const uint16_t *q,
                                      const uint16_t *k_cache,
                                      const uint16_t *v_cache,
                                      const int32_t *block_tables,
                                      const int32_t *context_lens,
                                      const int32_t *cu_q_lens, int S, int Hq,
                                      int Hkv, int D, int BS, int MB,
                                      int64_t q_stride, float scale,
                                      float softcap, int is_f16) {
  const int G = Hq / Hkv;
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
  for (int s = 0; s < S; s++) {
    for (int hq = 0; hq < Hq; hq++) {
      const int q0 = cu_q_lens ? cu_q_lens[s] : s;
      const int q_len = cu_q_lens ? cu_q_lens[s + 1] - cu_q_lens[s] : 1;
      const int kv_len = context_lens[s];
      const int32_t *table = block_tables + (int64_t)s * MB;
      double *logit = (double *)malloc(sizeof(double) * (size_t)(kv_len > 0 ? kv_len : 1));
      double *acc = (double *)malloc(sizeof(double) * (size_t)D);
      for (int j = 0; j < q_len; j++)
        attend_row(out + ((int64_t)(q0 + j) * Hq + hq) * D,
                   q + (int64_t)(q0 + j) * q_stride + (int64_t)hq * D, k_cache,
                   v_cache, table, kv_len - q_len + j + 1, hq / G, Hkv, D, BS,
                   scale, softcap, logit, acc, is_f16);
      free(logit);
      free(acc);
    }
  }
}
/* bf16 inputs (cache dtype 1). */
void oracle_paged_attention_varlen(float *out, const uint16_t *q,
                                   const uint16_t *k_cache,
                                   const uint16_t *v_cache,
                                   const int32_t *block_tables,
                                   const int32_t *context_lens,
                                   const int32_t *cu_q_lens, int S, int Hq,
                                   int Hkv, int D, int BS, int MB,
                                   int64_t q_stride, float scale,
                                   float softcap) {
  oracle_paged_attention_varlen_dt(out, q, k_cache, v_cache, block_tables, context_lens, cu_q_lens,
                                   S, Hq, Hkv, D, BS, MB, q_stride, scale, softcap, 0);
}

/* The same oracle restricted to a list of output rows, for spot checks at
 * sizes where the full result would take hours on a CPU.  rows = n_rows
 * triples (sequence, query index within the sequence, query head); out is
 * [n_rows, D] fp32 in list order.                                           */
void oracle_paged_attention_rows_dt(float *out, const int32_t *rows, int n_rows,
                                    const uint16_t *q, const uint16_t *k_cache,
                                    const uint16_t *v_cache,
                                    const int32_t *block_tables,
                                    const int32_t *context_lens,
                                    const int32_t *cu_q_lens, int Hq, int Hkv,
                                    int D, int BS, int MB, int64_t q_stride,
                                    float scale, float softcap, int is_f16) {
  const int G = Hq / Hkv;
#pragma omp parallel for schedule(dynamic, 1)
  for (int r = 0; r < n_rows; r++) {
    const int s = rows[3 * r], j = rows[3 * r + 1], hq = rows[3 * r + 2];
    const int q0 = cu_q_lens ? cu_q_lens[s] : s;
    const int q_len = cu_q_lens ? cu_q_lens[s + 1] - cu_q_lens[s] : 1;
    const int kv_len = context_lens[s];
    double *logit = (double *)malloc(sizeof(double) * (size_t)(kv_len > 0 ? kv_len : 1));
    double *acc = (double *)malloc(sizeof(double) * (size_t)D);
    attend_row(out + (int64_t)r * D, q + (int64_t)(q0 + j) * q_stride + (int64_t)hq * D,
               k_cache, v_cache, block_tables + (int64_t)s * MB,
               kv_len - q_len + j + 1, hq / G, Hkv, D, BS, scale, softcap, logit, acc, is_f16);
    free(logit);
    free(acc);
  }
}
void oracle_paged_attention_rows(float *out, const int32_t *rows, int n_rows,
                                 const uint16_t *q, const uint16_t *k_cache,
                                 const uint16_t *v_cache,
                                 const int32_t *block_tables,
                                 const int32_t *context_lens,
                                 const int32_t *cu_q_lens, int Hq, int Hkv,
                                 int D, int BS, int MB, int64_t q_stride,
                                 float scale, float softcap) {
  oracle_paged_attention_rows_dt(out, rows, n_rows, q, k_cache, v_cache, block_tables, context_lens,
                                 cu_q_lens, Hq, Hkv, D, BS, MB, q_stride, scale, softcap, 0);
}

/* Dense causal attention over contiguous K/V ([S][kv_len][Hkv][D] packed with
 * cu_kv_lens), used only to prove the paged oracle itself: the same queries
 * over the un-paged tensors must give the same result.                      */
void oracle_dense_causal(float *out, const uint16_t *q, const uint16_t *k,
                         const uint16_t *v, const int32_t *cu_q_lens,
                         const int32_t *cu_kv_lens, int S, int Hq, int Hkv,
                         int D, float scale) {
  const int G = Hq / Hkv;
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
  for (int s = 0; s < S; s++) {
    for (int hq = 0; hq < Hq; hq++) {
      const int q0 = cu_q_lens[s], q_len = cu_q_lens[s + 1] - cu_q_lens[s];
      const int k0 = cu_kv_lens[s], kv_len = cu_kv_lens[s + 1] - cu_kv_lens[s];
      const int h = hq / G;
      double *logit = (double *)malloc(sizeof(double) * (size_t)(kv_len > 0 ? kv_len : 1));
      for (int j = 0; j < q_len; j++) {
        float *o = out + ((int64_t)(q0 + j) * Hq + hq) * D;
        const int n = kv_len - q_len + j + 1;
        if (n <= 0) {
          for (int d = 0; d < D; d++) o[d] = 0.f;
          continue;
        }
        const uint16_t *qp = q + ((int64_t)(q0 + j) * Hq + hq) * D;
        double mx = -INFINITY;
        for (int t = 0; t < n; t++) {
          const uint16_t *kp = k + ((int64_t)(k0 + t) * Hkv + h) * D;
          double dot = 0.0;
          for (int d = 0; d < D; d++)
            dot += (double)bf16_to_f32(qp[d]) * (double)bf16_to_f32(kp[d]);
          logit[t] = dot * (double)scale;
          if (logit[t] > mx) mx = logit[t];
        }
        double sum = 0.0;
        for (int t = 0; t < n; t++) {
          logit[t] = exp(logit[t] - mx);
          sum += logit[t];
        }
        for (int d = 0; d < D; d++) {
          double a = 0.0;
          for (int t = 0; t < n; t++)
            a += logit[t] * (double)bf16_to_f32(v[((int64_t)(k0 + t) * Hkv + h) * D + d]);
          o[d] = (float)(a / sum);
        }
      }
      free(logit);
    }
  }
}

/* ------------------------------------------------------------------------ */
/* The timed CPU baseline: the reference's software path for decode,
 * crates/mlx-sys/src/mlx.cpp:4080-4159, step by step, with the materialised
 * intermediates it builds: take(k_cache, blocks) -> transpose {1,0,2,3,4} ->
 * transpose {0,1,3,2,4} -> reshape [Hkv, nb*BS, D] -> slice to context_len;
 * the same for V ({1,0,2,3} -> {0,1,3,2}); GQA repeat of every KV head G
 * times by concatenation (:4123-4137); scores = q @ K^T * scale; softmax;
 * @ V; stack over sequences.  bf16 storage with fp32 arithmetic; every
 * intermediate that MLX would store in the array dtype is rounded to bf16
 * (scores, weights, output).  Parallel over sequences (the outer loop of the
 * reference is serial; OpenMP here stands for the threads MLX's CPU backend
 * would use inside each op).  Returns 0, or -1 on allocation failure.       */
int baseline_mlx_paged_forward(uint16_t *out, const uint16_t *q,
                               const uint16_t *k_cache, const uint16_t *v_cache,
                               const int32_t *block_tables,
                               const int32_t *context_lens, int S, int Hq,
                               int Hkv, int D, int BS, int MB, float scale) {
  const int G = Hq / Hkv;
  const int x = 8;
  int failed = 0;
#pragma omp parallel for schedule(dynamic, 1)
  for (int s = 0; s < S; s++) {
    const int ctx = context_lens[s];
    const int nb = (ctx + BS - 1) / BS;
    uint16_t *o = out + (int64_t)s * Hq * D;
    if (ctx == 0 || nb == 0) {
      memset(o, 0, sizeof(uint16_t) * (size_t)Hq * D);
      continue;
    }
    const int64_t blk_elems = (int64_t)Hkv * D * BS;
    const int64_t T = (int64_t)nb * BS;
    uint16_t *gk = (uint16_t *)malloc(sizeof(uint16_t) * (size_t)(nb * blk_elems));
    uint16_t *gv = (uint16_t *)malloc(sizeof(uint16_t) * (size_t)(nb * blk_elems));
    uint16_t *kt = (uint16_t *)malloc(sizeof(uint16_t) * (size_t)(Hkv * T * D));
    uint16_t *vt = (uint16_t *)malloc(sizeof(uint16_t) * (size_t)(Hkv * T * D));
    uint16_t *ke = (uint16_t *)malloc(sizeof(uint16_t) * (size_t)Hq * ctx * D);
    uint16_t *ve = (uint16_t *)malloc(sizeof(uint16_t) * (size_t)Hq * ctx * D);
    float *sc = (float *)malloc(sizeof(float) * (size_t)ctx);
    if (!gk || !gv || !kt || !vt || !ke || !ve || !sc) {
      failed = 1;
      free(gk); free(gv); free(kt); free(vt); free(ke); free(ve); free(sc);
      continue;
    }
    /* take(cache, table[s, :nb], axis 0) */
    for (int b = 0; b < nb; b++) {
      const int64_t blk = (int64_t)block_tables[(int64_t)s * MB + b];
      memcpy(gk + b * blk_elems, k_cache + blk * blk_elems, sizeof(uint16_t) * (size_t)blk_elems);
      memcpy(gv + b * blk_elems, v_cache + blk * blk_elems, sizeof(uint16_t) * (size_t)blk_elems);
    }
    /* transposes + reshape: kt[h][b*BS+t][c*x+e] = gk[b][h][c][t][e],
     *                       vt[h][b*BS+t][d]     = gv[b][h][d][t]          */
    for (int h = 0; h < Hkv; h++)
      for (int b = 0; b < nb; b++)
        for (int t = 0; t < BS; t++) {
          uint16_t *kd = kt + ((int64_t)h * T + (int64_t)b * BS + t) * D;
          uint16_t *vd = vt + ((int64_t)h * T + (int64_t)b * BS + t) * D;
          const uint16_t *ks = gk + b * blk_elems + (int64_t)h * D * BS;
          const uint16_t *vs = gv + b * blk_elems + (int64_t)h * D * BS;
          for (int c = 0; c < D / x; c++)
            for (int e = 0; e < x; e++) kd[c * x + e] = ks[((int64_t)c * BS + t) * x + e];
          for (int d = 0; d < D; d++) vd[d] = vs[(int64_t)d * BS + t];
        }
    /* slice to ctx and repeat each KV head G times (concatenate) */
    for (int hq = 0; hq < Hq; hq++) {
      const int h = hq / G;
      memcpy(ke + (int64_t)hq * ctx * D, kt + (int64_t)h * T * D, sizeof(uint16_t) * (size_t)ctx * D);
      memcpy(ve + (int64_t)hq * ctx * D, vt + (int64_t)h * T * D, sizeof(uint16_t) * (size_t)ctx * D);
    }
    for (int hq = 0; hq < Hq; hq++) {
      const uint16_t *qp = q + ((int64_t)s * Hq + hq) * D;
      const uint16_t *kh = ke + (int64_t)hq * ctx * D;
      const uint16_t *vh = ve + (int64_t)hq * ctx * D;
      const float scale_bf = bf16_to_f32(f32_to_bf16(scale)); /* array(scale, q.dtype()) */
      float mx = -INFINITY;
      for (int t = 0; t < ctx; t++) {
        float dot = 0.f;
        for (int d = 0; d < D; d++) dot += bf16_to_f32(qp[d]) * bf16_to_f32(kh[(int64_t)t * D + d]);
        float v = bf16_to_f32(f32_to_bf16(dot));          /* matmul output dtype */
        v = bf16_to_f32(f32_to_bf16(v * scale_bf));        /* multiply */
        sc[t] = v;
        if (v > mx) mx = v;
      }
      float sum = 0.f;
      for (int t = 0; t < ctx; t++) {
        sc[t] = expf(sc[t] - mx);
        sum += sc[t];
      }
      for (int t = 0; t < ctx; t++) sc[t] = bf16_to_f32(f32_to_bf16(sc[t] / sum));
      for (int d = 0; d < D; d++) {
        float a = 0.f;
        for (int t = 0; t < ctx; t++) a += sc[t] * bf16_to_f32(vh[(int64_t)t * D + d]);
        o[(int64_t)hq * D + d] = f32_to_bf16(a);
      }
    }
    free(gk); free(gv); free(kt); free(vt); free(ke); free(ve); free(sc);
  }
  return failed ? -1 : 0;
}

/* ------------------------------------------------------------------------ */
/* Seeded synthetic inputs: a counter-based generator so that any consumer
 * can reproduce element i of tensor `stream` without shared state.
 * splitmix64(seed, stream, i) -> two 24-bit uniforms -> Box-Muller -> bf16. */
static inline uint64_t splitmix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
void oracle_fill_normal_bf16(uint16_t *dst, int64_t n, uint64_t seed,
                             uint64_t stream, int64_t first_index) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; i++) {
    const uint64_t r = splitmix64(splitmix64(seed * 0x100000001B3ull + stream) +
                                  (uint64_t)(first_index + i));
    const double u1 = ((double)((r >> 40) & 0xFFFFFF) + 1.0) / 16777216.0;
    const double u2 = (double)((r >> 16) & 0xFFFFFF) / 16777216.0;
    const double z = sqrt(-2.0 * log(u1)) * cos(6.283185307179586 * u2);
    dst[i] = f32_to_bf16((float)z);
  }
}

/* ------------------------------------------------------------------------- *
 * Producer of the write + attend pair: per-head RMS norm, then rotary
 * embedding at each token's position.  Restates steps 3 and 5 of
 * mlx_fused_attention_qkv (crates/mlx-sys/src/mlx.cpp:1343-1365) as they act on
 * one token at offset `positions[t]` (the per-sequence call of
 * crates/mlx-core/src/transformer/attention.rs:658-664), using the published
 * arithmetic of MLX's fast::rms_norm (w * T(x * rsqrt(mean(x^2) + eps))) and
 * fast::rope with traditional = false, scale 1: element i < dims/2 pairs with
 * i + dims/2, angle = float(position) * inv_freq[i],
 *   out[i]          = x[i] cos - x[i + dims/2] sin,
 *   out[i + dims/2] = x[i] sin + x[i + dims/2] cos,
 * elements >= dims unchanged.  MLX itself is an absent third-party dependency
 * (git submodule crates/mlx-sys/mlx, no pinned version in the tree).
 *
 * The mean of squares, the reciprocal square root and the trigonometric
 * functions are evaluated in double here; the rounding points (normalised value
 * to T, times weight to T, rotated value to T) and the fp32 angle are the
 * reference's.  `bound[t,h,d]` (optional) receives |a| + |b| of the rotated
 * pair after the norm: a difference of one unit in the last place of either
 * operand moves the result by at most 2^-8 (bf16) or 2^-11 (f16) of it.
 * x: [T, H, D] with row stride `stride` elements; w: [D] or NULL; out like x
 * (contiguous [T, H, D]).
 * ------------------------------------------------------------------------- */
static inline uint16_t f32_to_f16(float f) {
  _Float16 v = (_Float16)f;
  uint16_t h;
  memcpy(&h, &v, 2);
  return h;
}
static inline uint16_t f32_to_elem(float f, int is_f16) {
  return is_f16 ? f32_to_f16(f) : f32_to_bf16(f);
}

void oracle_qk_norm_rope(uint16_t *out, float *bound, const uint16_t *x, int64_t stride,
                         const uint16_t *w, double eps, const int32_t *positions,
                         double rope_base, int rope_dims, int64_t T, int H, int D,
                         int is_f16) {
  const int half = rope_dims / 2;
  float *inv_freq = (float *)malloc(sizeof(float) * (half > 0 ? half : 1));
  for (int i = 0; i < half; i++)
    inv_freq[i] = (float)pow(rope_base, -(double)i / (double)half);
#pragma omp parallel for schedule(static)
  for (int64_t t = 0; t < T; t++) {
    double *y = (double *)malloc(sizeof(double) * D);
    for (int h = 0; h < H; h++) {
      const uint16_t *xp = x + t * stride + (int64_t)h * D;
      if (w) {
        double ss = 0.0;
        for (int d = 0; d < D; d++) {
          const double v = elem_to_f32(xp[d], is_f16);
          ss += v * v;
        }
        const double inv = 1.0 / sqrt(ss / D + eps);
        for (int d = 0; d < D; d++) {
          const float n = elem_to_f32(f32_to_elem((float)(elem_to_f32(xp[d], is_f16) * inv), is_f16), is_f16);
          y[d] = elem_to_f32(f32_to_elem(n * elem_to_f32(w[d], is_f16), is_f16), is_f16);
        }
      } else {
        for (int d = 0; d < D; d++) y[d] = elem_to_f32(xp[d], is_f16);
      }
      uint16_t *op = out + (t * H + h) * (int64_t)D;
      float *bp = bound ? bound + (t * H + h) * (int64_t)D : NULL;
      for (int i = 0; i < half; i++) {
        const float theta = (float)positions[t] * inv_freq[i];
        const double c = cos((double)theta), s = sin((double)theta);
        const double a = y[i], b = y[i + half];
        op[i] = f32_to_elem((float)(a * c - b * s), is_f16);
        op[i + half] = f32_to_elem((float)(a * s + b * c), is_f16);
        if (bp) bp[i] = bp[i + half] = (float)(fabs(a) + fabs(b));
      }
      for (int d = 2 * half; d < D; d++) {
        op[d] = f32_to_elem((float)y[d], is_f16);
        if (bp) bp[d] = 0.f;
      }
    }
    free(y);
  }
  free(inv_freq);
}

/* ------------------------------------------------------------------------- *
 * FP8 (E4M3) KV cache.  The pools hold one byte per element, x = 16
 * (crates/mlx-paged-attn/src/cache_engine.rs:66-76): key cache
 * [num_blocks, num_kv_heads, head_size/16, block_size, 16], value cache
 * [num_blocks, num_kv_heads, head_size, block_size].
 *
 * The byte format is the reference's own, not the OCP "FN" variant
 * (crates/mlx-paged-attn/metal/float8.metal:11-33 decode, :63-121 encode):
 * bias 7; exponent field 15 decodes to infinity (mantissa 0) or NaN, so the
 * largest finite value is 1.75 * 2^7 = 240.  The encoder rounds the normal
 * range to nearest even and lets it overflow to the infinity code; below the
 * normal range magnitudes under 2^-9 become zero, the rest round half up, and a value that would round up to the
 * smallest normal number is returned as zero (the mantissa is masked to three
 * bits with the exponent field left at 0).  Inputs with an unbiased exponent
 * of 8 or more (|x| >= 256) are not in its normal range test and fall into
 * the same below-normal branch; for 256 <= |x| < 16384 that branch yields the
 * low three bits of a shifted mantissa, which is restated as is; from 16384 up
 * the reference's shift count is negative (undefined there) and the infinity
 * code is produced here instead.
 * ------------------------------------------------------------------------- */
float oracle_fp8_e4m3_decode(uint8_t v) {
  const unsigned s = v >> 7, e = (v >> 3) & 0xF, m = v & 7;
  float val;
  if (e == 0) val = ldexpf((float)m / 8.f, -6);
  else if (e == 0xF) val = m ? NAN : INFINITY;
  else val = ldexpf(1.f + (float)m / 8.f, (int)e - 7);
  return s ? -val : val;
}

uint8_t oracle_fp8_e4m3_encode(float f) {
  uint32_t bits;
  memcpy(&bits, &f, 4);
  const uint32_t s = bits >> 31, a = bits & 0x7FFFFFFFu;
  if (a >= 0x7F800000u) return (uint8_t)((s << 7) | 0x78u | (a != 0x7F800000u));
  const int e8 = (int)(a >> 23) - 127 + 7;
  const uint32_t m = a & 0x7FFFFFu;
  if (e8 >= 1 && e8 <= 14) {
    uint32_t mant = m >> 20;
    const uint32_t half = (m >> 19) & 1u, rest = (m & 0x7FFFFu) != 0u;
    mant += half & (rest | (mant & 1u));
    int e = e8;
    if (mant >> 3) {
      mant = 0;
      if (++e > 14) return (uint8_t)((s << 7) | 0x78u);
    }
    return (uint8_t)((s << 7) | ((uint32_t)e << 3) | (mant & 7u));
  }
  if (e8 < -2) return (uint8_t)(s << 7);
  const int rshift = (1 - e8) + 20;
  if (rshift < 1) return (uint8_t)((s << 7) | 0x78u);
  const uint32_t rounded = ((0x800000u | m) + (1u << (rshift - 1))) >> rshift;
  return (uint8_t)((s << 7) | (rounded & 7u));
}

/* KV block write into an FP8 cache.
 * crates/mlx-paged-attn/metal/cache/reshape_and_cache.metal:58-97, the
 * USE_FP8_SCALES branch (:88-92): the element is divided by the scale in fp32,
 * rounded to the input type, and encoded.  Index formulas as in
 * oracle_reshape_and_cache with x = 16.                                      */
void oracle_reshape_and_cache_fp8(const uint16_t *key, const uint16_t *value,
                                  uint8_t *key_cache, uint8_t *value_cache,
                                  const int64_t *slot_mapping, int64_t num_tokens,
                                  int64_t key_stride, int64_t value_stride,
                                  int num_heads, int head_size, int block_size,
                                  float k_scale, float v_scale, int is_f16) {
  const int x = 16;
  for (int64_t token_idx = 0; token_idx < num_tokens; token_idx++) {
    const int64_t slot_idx = slot_mapping[token_idx];
    if (slot_idx < 0) continue;
    const int64_t block_idx = slot_idx / block_size;
    const int64_t block_offset = slot_idx % block_size;
    const int n = num_heads * head_size;
    for (int i = 0; i < n; i++) {
      const int head_idx = i / head_size, head_offset = i % head_size;
      const int x_idx = head_offset / x, x_offset = head_offset % x;
      const int64_t tgt_key_idx =
          block_idx * num_heads * (head_size / x) * block_size * x +
          (int64_t)head_idx * (head_size / x) * block_size * x +
          (int64_t)x_idx * block_size * x + block_offset * x + x_offset;
      const int64_t tgt_value_idx =
          block_idx * num_heads * head_size * block_size +
          (int64_t)head_idx * head_size * block_size +
          (int64_t)head_offset * block_size + block_offset;
      const float kq = elem_to_f32(key[token_idx * key_stride + i], is_f16) / k_scale;
      const float vq = elem_to_f32(value[token_idx * value_stride + i], is_f16) / v_scale;
      key_cache[tgt_key_idx] =
          oracle_fp8_e4m3_encode(elem_to_f32(f32_to_elem(kq, is_f16), is_f16));
      value_cache[tgt_value_idx] =
          oracle_fp8_e4m3_encode(elem_to_f32(f32_to_elem(vq, is_f16), is_f16));
    }
  }
}

/* Attention over an FP8 cache: element = decode(byte) * scale
 * (crates/mlx-paged-attn/metal/attention/paged_attention.metal:569-571,
 * used at :920-929 for K and :1063-1071 for V), everything else as
 * oracle_paged_attention_varlen_dt, in fp64.  The reference rounds each
 * dequantised element to the query type before use; that rounding is a
 * precision loss of its kernel and is not reproduced.                       */
static void attend_row_fp8(float *o, const uint16_t *qp, const uint8_t *k_cache,
                           const uint8_t *v_cache, const int32_t *table, int n,
                           int h, int Hkv, int D, int BS, float scale, float softcap,
                           double *logit, double *acc, int is_f16, float k_scale,
                           float v_scale) {
  const int x = 16;
  if (n <= 0) {
    for (int d = 0; d < D; d++) o[d] = 0.f;
    return;
  }
  double mx = -INFINITY;
  for (int t = 0; t < n; t++) {
    const int64_t kb = k_index(table, t, h, 0, Hkv, D, BS, x);
    double dot = 0.0;
    for (int c = 0; c < D / x; c++)
      for (int e = 0; e < x; e++)
        dot += (double)elem_to_f32(qp[c * x + e], is_f16) *
               ((double)oracle_fp8_e4m3_decode(k_cache[kb + (int64_t)c * BS * x + e]) *
                (double)k_scale);
    double l = dot * (double)scale;
    if (softcap != 1.0f) l = tanh(l / (double)softcap) * (double)softcap;
    logit[t] = l;
    if (l > mx) mx = l;
  }
  double sum = 0.0;
  for (int t = 0; t < n; t++) {
    logit[t] = exp(logit[t] - mx);
    sum += logit[t];
  }
  for (int d = 0; d < D; d++) acc[d] = 0.0;
  for (int t = 0; t < n; t++) {
    const double p = logit[t];
    const int64_t vb = v_index(table, t, h, 0, Hkv, D, BS);
    for (int d = 0; d < D; d++)
      acc[d] += p * ((double)oracle_fp8_e4m3_decode(v_cache[vb + (int64_t)d * BS]) *
                     (double)v_scale);
  }
  for (int d = 0; d < D; d++) o[d] = (float)(acc[d] / sum);
}

void oracle_paged_attention_varlen_fp8(float *out, const uint16_t *q, const uint8_t *k_cache,
                                       const uint8_t *v_cache, const int32_t *block_tables,
                                       const int32_t *context_lens, const int32_t *cu_q_lens,
                                       int S, int Hq, int Hkv, int D, int BS, int MB,
                                       int64_t q_stride, float scale, float softcap,
                                       int is_f16, float k_scale, float v_scale) {
  const int G = Hq / Hkv;
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
  for (int s = 0; s < S; s++) {
    for (int hq = 0; hq < Hq; hq++) {
      const int q0 = cu_q_lens ? cu_q_lens[s] : s;
      const int q_len = cu_q_lens ? cu_q_lens[s + 1] - cu_q_lens[s] : 1;
      const int kv_len = context_lens[s];
      const int32_t *table = block_tables + (int64_t)s * MB;
      double *logit = (double *)malloc(sizeof(double) * (size_t)(kv_len > 0 ? kv_len : 1));
      double *acc = (double *)malloc(sizeof(double) * (size_t)D);
      for (int j = 0; j < q_len; j++)
        attend_row_fp8(out + ((int64_t)(q0 + j) * Hq + hq) * D,
                       q + (int64_t)(q0 + j) * q_stride + (int64_t)hq * D, k_cache, v_cache,
                       table, kv_len - q_len + j + 1, hq / G, Hkv, D, BS, scale, softcap,
                       logit, acc, is_f16, k_scale, v_scale);
      free(logit);
      free(acc);
    }
  }
}
