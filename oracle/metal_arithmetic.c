/*
 * Test infrastructure, not product: a CPU restatement of the ARITHMETIC of the
 * reference's Metal decode kernels, operation order and rounding points included,
 * so that the distance between that arithmetic and the exact-softmax oracle of
 * paged_oracle.c can be measured instead of asserted.  Only tests may call it.
 *
 * Follows crates/mlx-paged-attn/metal/attention/paged_attention.metal at the
 * template constants of head size 128, block size 16, 16-bit T, 256 threads, 32
 * lanes per SIMD group (THREAD_GROUP_SIZE 2, VEC_SIZE 4, NUM_VECS_PER_THREAD 16,
 * V_VEC_SIZE 8, NUM_ROWS_PER_THREAD 8, 8 warps):
 *   :865-874, 892-962   q.k in fp32: per thread of a 2-thread group a float4 of
 *                       running fma over its 16 vectors, x+y+z+w, the pair added,
 *                       times scale; optional soft cap; tokens past the context get
 *                       logit 0 and do not move the maximum
 *   :964-983            maximum over the partition
 *   :986-999            exp(logit - max), sum per thread (stride 256), butterfly over
 *                       the 32 lanes, then over the 8 warps; inv = 1 / (sum + 1e-6)
 *   :1016-1084          P rounded to T; per (lane, row) the 8 products of one 16-byte
 *                       V piece in T precision (bf16: each product rounded to bf16, summed
 *                       in fp32 pairwise; f16: each product rounded to f16 and the two
 *                       groups of four summed in f16), added to an fp32 accumulator per
 *                       warp over the blocks that warp takes (block index mod 8)
 *   :1086-1132          lane pair added, then warps combined 4-7 -> 0-3, 2-3 -> 0-1, 1 -> 0
 *   :1135-1146          T(acc): the output (V1, context <= 512) or the partition's
 *                       tmp_out (V2, partitions of 512 tokens,
 *                       crates/mlx-paged-attn/src/metal/paged_attention.rs:106, 964)
 *   :1149-1260          V2 reduce: max of partition maxima, exp sums rescaled, their sum
 *                       through block_sum, inv = 1 / (sum + 1e-6), out = T(sum_j
 *                       float(tmp_out_j) * rescaled_j * inv)
 * The threadgroup-level fast-math of the Metal compiler (exp, divide) cannot be
 * reproduced: expf and a true division stand in, which moves results by an ulp of
 * fp32 at most, far below the T-precision effects this file exists to measure.
 */
#include <float.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
static inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return 0x7FC0;
  return (uint16_t)((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
}
static inline float f16_to_f32(uint16_t h) {
  _Float16 v;
  memcpy(&v, &h, 2);
  return (float)v;
}
static inline uint16_t f32_to_f16(float f) {
  _Float16 v = (_Float16)f;
  uint16_t h;
  memcpy(&h, &v, 2);
  return h;
}
static inline float to_f32(uint16_t b, int f16) { return f16 ? f16_to_f32(b) : bf16_to_f32(b); }
/* round an fp32 value to T and come back */
static inline float round_t(float x, int f16) {
  return f16 ? f16_to_f32(f32_to_f16(x)) : bf16_to_f32(f32_to_bf16(x));
}

enum { HEAD = 128, BS = 16, X = 8, NT = 256, LANES = 32, WARPS = 8, PART = 512 };

/* butterfly sum over 32 lanes (every lane ends with the same value; lane 0's is used) */
static float simd_sum(float *v) {
  for (int mask = LANES / 2; mask >= 1; mask /= 2) {
    float t[LANES];
    for (int l = 0; l < LANES; l++) t[l] = v[l] + v[l ^ mask];
    memcpy(v, t, sizeof(t));
  }
  return v[0];
}
/* block_sum (:714-744): per-warp butterfly, then a butterfly over the 8 warp sums */
static float block_sum(const float *per_thread) {
  float warp_sum[LANES];
  for (int l = 0; l < LANES; l++) warp_sum[l] = 0.f;
  for (int w = 0; w < WARPS; w++) {
    float v[LANES];
    memcpy(v, per_thread + w * LANES, sizeof(v));
    warp_sum[w] = simd_sum(v);
  }
  /* lanes >= NUM_WARPS keep their own (already reduced) value in the kernel; only
   * lanes 0..7 feed lane 0 through masks 4, 2, 1 */
  for (int mask = WARPS / 2; mask >= 1; mask /= 2) {
    float t[WARPS];
    for (int l = 0; l < WARPS; l++) t[l] = warp_sum[l] + warp_sum[l ^ mask];
    memcpy(warp_sum, t, sizeof(t));
  }
  return warp_sum[0];
}

/* one partition [tok0, tok1) of one (sequence, query head): out_t[128] in T bits,
 * its maximum logit and exp sum */
static void partition(uint16_t *out_t, float *max_logit, float *exp_sum_out, const uint16_t *q,
                      const uint16_t *k_cache, const uint16_t *v_cache, const int32_t *table,
                      int kv_head, int Hkv, int context_len, int tok0, int tok1, float scale,
                      float softcap, int f16, float *logits /* [PART] */) {
  const int64_t block_stride = (int64_t)Hkv * HEAD * BS, head_stride = (int64_t)HEAD * BS;
  const int start_block = tok0 / BS, end_block = (tok1 + BS - 1) / BS;
  const int num_tokens = tok1 - tok0;
  const int num_context_blocks = (context_len + BS - 1) / BS;
  float qk_max = -FLT_MAX;
  for (int blk = start_block; blk < end_block; blk++) {
    const int64_t pb = table[blk];
    for (int off = 0; off < BS; off++) {  /* one 2-thread group per token */
      const int token = blk * BS + off;
      const uint16_t *kp = k_cache + pb * block_stride + kv_head * head_stride + off * X;
      float part[2];
      for (int tg = 0; tg < 2; tg++) {
        float acc[4];
        for (int j = 0; j < 16; j++) {
          const int vec = tg + j * 2;                 /* vec_idx */
          const int o1 = (vec * 4) / X, o2 = (vec * 4) % X;
          for (int e = 0; e < 4; e++) {
            const float qa = to_f32(q[vec * 4 + e], f16);
            const float ka = to_f32(kp[o1 * BS * X + o2 + e], f16);
            acc[e] = j == 0 ? qa * ka : fmaf(qa, ka, acc[e]);
          }
        }
        part[tg] = ((acc[0] + acc[1]) + acc[2]) + acc[3];
      }
      float qk = scale * (part[0] + part[1]);
      if (softcap != 1.0f) qk = tanhf(qk / softcap) * softcap;
      const int masked = token >= context_len;
      if (token - tok0 < PART) logits[token - tok0] = masked ? 0.f : qk;
      if (!masked && qk > qk_max) qk_max = qk;
    }
  }
  float per_thread[NT];
  for (int t = 0; t < NT; t++) {
    float s = 0.f;
    for (int i = t; i < num_tokens; i += NT) {
      const float val = expf(logits[i] - qk_max);
      logits[i] = val;
      s += val;
    }
    per_thread[t] = s;
  }
  const float exp_sum = block_sum(per_thread);
  const float inv_sum = 1.f / (exp_sum + 1e-6f);
  for (int i = 0; i < num_tokens; i++) logits[i] *= inv_sum;
  /* logits beyond num_tokens inside the last block are whatever the loop above stored
   * for masked tokens (0, then exp(0 - max) * inv): the kernel zeroes the V side instead */

  /* P.V: accs[warp][row] over the blocks the warp takes; the two lanes of a row hold
   * tokens 0-7 and 8-15 of the block */
  static _Thread_local float accs[WARPS][2][HEAD];
  memset(accs, 0, sizeof(accs));
  for (int blk = start_block; blk < end_block; blk++) {
    const int w = (blk - start_block) % WARPS;
    const int64_t pb = table[blk];
    const uint16_t *vp = v_cache + pb * block_stride + kv_head * head_stride;
    for (int half_i = 0; half_i < 2; half_i++) {
      const int off = half_i * 8, token = blk * BS + off;
      float pl[8];
      for (int j = 0; j < 8; j++) {
        const int li = token - tok0 + j;
        pl[j] = round_t(li < PART ? logits[li] : 0.f, f16);   /* from_float: P in T */
      }
      for (int row = 0; row < HEAD; row++) {
        float prod[8];
        for (int j = 0; j < 8; j++) {
          float v = to_f32(vp[row * BS + off + j], f16);
          if (blk == num_context_blocks - 1 && !(token + j < context_len)) v = 0.f;
          prod[j] = round_t(pl[j] * v, f16);                  /* mul<T8, T8, T8> */
        }
        float d;
        if (f16) {  /* sum(half4) adds in half, sum(Half8_) adds the two in float */
          float a = round_t(prod[0] + prod[1], 1);
          a = round_t(a + prod[2], 1);
          a = round_t(a + prod[3], 1);
          float b = round_t(prod[4] + prod[5], 1);
          b = round_t(b + prod[6], 1);
          b = round_t(b + prod[7], 1);
          d = a + b;
        } else {    /* sum(Bfloat2_) in float, pairs of pairs */
          d = ((prod[0] + prod[1]) + (prod[2] + prod[3])) + ((prod[4] + prod[5]) + (prod[6] + prod[7]));
        }
        accs[w][half_i][row] += d;
      }
    }
  }
  for (int row = 0; row < HEAD; row++) {
    float wsum[WARPS];
    for (int w = 0; w < WARPS; w++) wsum[w] = accs[w][0][row] + accs[w][1][row];  /* lane pair */
    for (int i = WARPS; i > 1; i /= 2) {
      const int mid = i / 2;
      for (int w = 0; w < mid; w++) wsum[w] += wsum[w + mid];
    }
    out_t[row] = f16 ? f32_to_f16(wsum[0]) : f32_to_bf16(wsum[0]);
  }
  *max_logit = qk_max;
  *exp_sum_out = exp_sum;
}

/* Decode attention as dispatch_paged_attention_auto runs it: V1 when max_context_len
 * <= 512, else V2 + reduce.  out: T bits [S, Hq, 128].  q stride Hq*128. */
void oracle_paged_attention_metal(uint16_t *out, const uint16_t *q, const uint16_t *k_cache,
                                  const uint16_t *v_cache, const int32_t *block_tables,
                                  const int32_t *context_lens, int S, int Hq, int Hkv, int MB,
                                  float scale, float softcap, int is_f16) {
  int max_ctx = 0;
  for (int s = 0; s < S; s++)
    if (context_lens[s] > max_ctx) max_ctx = context_lens[s];
  const int use_v2 = max_ctx > PART;
  const int max_parts = (max_ctx + PART - 1) / PART;
  const int G = Hq / Hkv;
#pragma omp parallel for collapse(2) schedule(dynamic)
  for (int s = 0; s < S; s++) {
    for (int h = 0; h < Hq; h++) {
      const int ctx = context_lens[s];
      uint16_t *o = out + ((int64_t)s * Hq + h) * HEAD;
      const uint16_t *qp = q + ((int64_t)s * Hq + h) * HEAD;
      const int32_t *table = block_tables + (int64_t)s * MB;
      float *logits = (float *)malloc(sizeof(float) * ((use_v2 ? PART : ((max_ctx + BS - 1) / BS) * BS) + BS));
      if (ctx <= 0) {   /* the kernels leave such rows alone; the callers never send them */
        memset(o, 0, HEAD * 2);
        free(logits);
        continue;
      }
      if (!use_v2) {
        float m, e;
        /* V1 sizes its logits array by the padded context, not by 512 */
        partition(o, &m, &e, qp, k_cache, v_cache, table, h / G, Hkv, ctx, 0, ctx, scale, softcap,
                  is_f16, logits);
      } else {
        const int np = (ctx + PART - 1) / PART;
        uint16_t *tmp = (uint16_t *)malloc((size_t)max_parts * HEAD * 2);
        float *mx = (float *)malloc(sizeof(float) * max_parts), *es = (float *)malloc(sizeof(float) * max_parts);
        for (int p = 0; p < np; p++) {
          const int t0 = p * PART, t1 = t0 + PART < ctx ? t0 + PART : ctx;
          partition(tmp + p * HEAD, &mx[p], &es[p], qp, k_cache, v_cache, table, h / G, Hkv, ctx, t0, t1,
                    scale, softcap, is_f16, logits);
        }
        if (np == 1) {
          memcpy(o, tmp, HEAD * 2);
        } else {
          float max_logit = -FLT_MAX;
          for (int p = 0; p < np; p++)
            if (mx[p] > max_logit) max_logit = mx[p];
          float per_thread[NT];
          float *resc = (float *)malloc(sizeof(float) * np);
          for (int t = 0; t < NT; t++) {
            float g = 0.f;
            for (int i = t; i < np; i += NT) {
              resc[i] = es[i] * expf(mx[i] - max_logit);
              g += resc[i];
            }
            per_thread[t] = g;
          }
          const float inv = 1.f / (block_sum(per_thread) + 1e-6f);
          for (int i = 0; i < HEAD; i++) {
            float acc = 0.f;
            for (int j = 0; j < np; j++) acc += to_f32(tmp[j * HEAD + i], is_f16) * resc[j] * inv;
            o[i] = is_f16 ? f32_to_f16(acc) : f32_to_bf16(acc);
          }
          free(resc);
        }
        free(tmp);
        free(mx);
        free(es);
      }
      free(logits);
    }
  }
}
