// Decode/prefill-side producer for the write + attend pair: per-head RMS norm of the
// projected queries and keys, rotary embedding at each token's own position, and the
// KV block write, in one launch for the whole batch.
//
// What it replaces: crates/mlx-core/src/transformer/attention.rs:637-691 calls the
// per-sequence graph builder once per sequence because each sequence has its own RoPE
// offset; steps 3-5 of crates/mlx-sys/src/mlx.cpp:1343-1365 (fast::rms_norm on the
// [.., heads, head_dim] view, then fast::rope with traditional = false, scale 1) run per
// sequence, the results are stacked and crates/mlx-core/src/transformer/block.rs:224-226
// hands keys and values to the cache write.  Here the projections of all tokens come in
// as [T, heads, 128] and leave as rotated queries (in place or to a second buffer) and
// as pool contents; the rotated keys are never materialised outside the pool.
//
// Arithmetic follows MLX's kernels with their rounding points: the normalised element
// x * rsqrt(mean(x^2) + eps) is rounded to the 16-bit type, multiplied by the weight and
// rounded again; the rotation runs in fp32 on those values and is rounded once.  The
// angle is float(position) * inv_freq[i] with inv_freq[i] = base^(-i / (dims/2)) taken
// from a host-computed fp32 table, so that any two implementations that share the table
// see the same angles.
#include "pa_common.cuh"

namespace pa {

namespace {

constexpr int kTok = 16;  // tokens per CTA (one pool block's worth of slots)
constexpr int kVPadP = 2;

template <bool F16>
__device__ __forceinline__ float elem_to_float(uint32_t bits16) {
  if (F16) {
    float f;
    asm("cvt.f32.f16 %0, %1;" : "=f"(f) : "h"((uint16_t)bits16));
    return f;
  }
  return __uint_as_float(bits16 << 16);
}

template <bool F16>
__global__ void __launch_bounds__(256)
qk_norm_rope_cache_kernel(const ProducerParams p) {
  __shared__ uint4 k_s[kTok][kHeadSize / 8];
  __shared__ __align__(16) uint16_t v_s[kTok][kHeadSize + kVPadP];
  __shared__ int64_t slot_s[kTok];
  __shared__ float2 cs_s[kTok][kHeadSize / 2];   // (cos, sin) per token and frequency
  __shared__ float row_s[8][kHeadSize];          // one normalised row per warp

  // The attention kernel that follows may set up; it reads neither the pool nor the
  // queries before its own griddepcontrol.wait.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int h = blockIdx.y;
  const int64_t t0 = (int64_t)blockIdx.x * p.tok_per_cta;
  // tokens of this CTA: 16 for long chunks (whole pool rows per store), fewer for small
  // batches so that the rows spread over more SMs
  const int n_tok = (int)min((int64_t)p.tok_per_cta, p.num_tokens - t0);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bs_log = 4 + p.bs_shift, bs = 1 << bs_log;  // tokens of a pool block
  const int64_t n_slots = (int64_t)p.num_blocks << bs_log;
  const int half = p.rope_dims >> 1;
  const int G = p.Hq / p.Hkv;

  if (tid < kTok) {
    int64_t s = -1;
    if (tid < n_tok) {
      s = p.slot_mapping[t0 + tid];
      if (s >= n_slots) {
        atomicOr(p.err, kErrSlotRange);
        s = -1;
      }
    }
    slot_s[tid] = s;
  }
  for (int e = tid; e < n_tok * half; e += 256) {
    const int tok = e / half, i = e - tok * half;
    {
      const float theta = (float)p.positions[t0 + tok] * p.inv_freq[i];
      float sn, cs;
      sincosf(theta, &sn, &cs);
      cs_s[tok][i] = make_float2(cs, sn);
    }
  }
  // V: plain staging, thread -> (token, 16-byte piece)
  {
    const int tok = tid >> 4, piece = tid & 15;
    if (tok < n_tok) {
      const uint4 vv = *reinterpret_cast<const uint4 *>(p.v + (t0 + tok) * p.v_stride +
                                                        (int64_t)h * kHeadSize + piece * 8);
      uint32_t *vd = reinterpret_cast<uint32_t *>(&v_s[tok][piece * 8]);
      vd[0] = vv.x; vd[1] = vv.y; vd[2] = vv.z; vd[3] = vv.w;
    }
  }
  __syncthreads();

  // Rows of this CTA: (token, r) with r = 0 the key head, r = 1..G the query heads of
  // this KV head.  Each lane owns elements 4*lane .. 4*lane+3 of a row.
  const int rows = n_tok * (G + 1);
  for (int row = warp; row < rows; row += 8) {
    const int tok = row / (G + 1), r = row - tok * (G + 1);
    const bool is_k = r == 0;
    const elem16 *src = is_k ? p.k + (t0 + tok) * p.k_stride + (int64_t)h * kHeadSize
                             : p.q_in + (t0 + tok) * p.q_stride +
                                   (int64_t)(h * G + r - 1) * kHeadSize;
    const elem16 *w = is_k ? p.k_norm_w : p.q_norm_w;
    const uint2 raw = *reinterpret_cast<const uint2 *>(src + 4 * lane);
    float x[4] = {elem_to_float<F16>(raw.x & 0xffffu), elem_to_float<F16>(raw.x >> 16),
                  elem_to_float<F16>(raw.y & 0xffffu), elem_to_float<F16>(raw.y >> 16)};
    if (w) {
      float ss = x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      const float inv = 1.0f / sqrtf(ss * (1.0f / kHeadSize) + p.eps);
      const uint2 wr = *reinterpret_cast<const uint2 *>(w + 4 * lane);
      const float wf[4] = {elem_to_float<F16>(wr.x & 0xffffu), elem_to_float<F16>(wr.x >> 16),
                           elem_to_float<F16>(wr.y & 0xffffu), elem_to_float<F16>(wr.y >> 16)};
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const float n = elem_to_float<F16>(to_elem<F16>(x[i] * inv));
        x[i] = elem_to_float<F16>(to_elem<F16>(n * wf[i]));
      }
    }
    __syncwarp();
    *reinterpret_cast<float4 *>(&row_s[warp][4 * lane]) = make_float4(x[0], x[1], x[2], x[3]);
    __syncwarp();
    float y[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int d = 4 * lane + i;
      if (d < half) {
        const float2 c = cs_s[tok][d];
        y[i] = x[i] * c.x - row_s[warp][d + half] * c.y;
      } else if (d < 2 * half) {
        const float2 c = cs_s[tok][d - half];
        y[i] = row_s[warp][d - half] * c.y + x[i] * c.x;
      } else {
        y[i] = x[i];
      }
    }
    const uint2 packed = make_uint2(pack2<F16>(y[0], y[1]), pack2<F16>(y[2], y[3]));
    if (is_k) {
      reinterpret_cast<uint2 *>(&k_s[tok][0])[lane] = packed;
    } else {
      *reinterpret_cast<uint2 *>(p.q_out + (t0 + tok) * p.q_out_stride +
                                 (int64_t)(h * G + r - 1) * kHeadSize + 4 * lane) = packed;
    }
  }
  __syncthreads();

  // Pool write, token index fastest across threads (same store pattern as the plain
  // KV write kernel).
  {
    const int tok = tid & 15, c = tid >> 4;
    const int64_t slot = slot_s[tok];
    if (slot >= 0) {
      const int64_t blk = slot >> bs_log;
      const int off = (int)(slot & (bs - 1));
      elem16 *dst = p.k_pool + (((blk * p.Hkv + h) * (int64_t)kHeadSize) << bs_log) + c * (bs * 8) +
                    off * 8;
      *reinterpret_cast<uint4 *>(dst) = k_s[tok][c];
    }
  }
  for (int e = tid; e < kTok * kHeadSize; e += 256) {
    const int tok = e & 15, d = e >> 4;
    const int64_t slot = slot_s[tok];
    if (slot >= 0) {
      const int64_t blk = slot >> bs_log;
      const int off = (int)(slot & (bs - 1));
      reinterpret_cast<uint16_t *>(p.v_pool)[(((blk * p.Hkv + h) * (int64_t)kHeadSize) << bs_log) +
                                             d * bs + off] = v_s[tok][d];
    }
  }
}

}  // namespace

cudaError_t launch_qk_norm_rope_cache(const ProducerParams &p_in, bool f16, int num_sms,
                                      cudaStream_t st) {
  if (p_in.num_tokens <= 0) return cudaSuccess;
  ProducerParams p = p_in;
  // about two CTAs per SM before a CTA takes more than one token
  const int64_t want = p.num_tokens * p.Hkv / (2 * (int64_t)num_sms);
  p.tok_per_cta = (int)(want < 1 ? 1 : (want > kTok ? kTok : want));
  const int64_t groups = (p.num_tokens + p.tok_per_cta - 1) / p.tok_per_cta;
  dim3 grid((unsigned)groups, (unsigned)p.Hkv);
  if (f16) qk_norm_rope_cache_kernel<true><<<grid, 256, 0, st>>>(p);
  else qk_norm_rope_cache_kernel<false><<<grid, 256, 0, st>>>(p);
  __atomic_fetch_add(&g_launch_count, 1ull, __ATOMIC_RELAXED);
  return cudaGetLastError();
}

}  // namespace pa
