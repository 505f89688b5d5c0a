// Tile kernel for long-query sequences (chunked prefill) over the paged cache,
// warp-level tensor-core version (mma.sync m16n8k16, bf16 in / fp32 out).
//
// The reference has no paged prefill kernel: its prefill is dense causal
// attention followed by a scatter into the pool
// (crates/mlx-core/src/transformer/block.rs:279-317).  This kernel attends
// directly over the pool: query j of a sequence sees keys
// [0, kv_len - q_len + j].
//
// One CTA = 128 rows of one (sequence, kv head): a row is a (query token, query
// head of the GQA group) pair, token-major, so a CTA covers 128/G consecutive
// query tokens and reads each KV block once for all of them.  Eight warps of 16
// rows.  KV blocks (4 KB K chunk + 4 KB V chunk) stream through a CTA-wide ring
// of bulk async copies (TMA, untiled, no multicast); full/empty mbarriers hand
// stages between the issuing lane and the eight consuming warps.
//   S[16 x 16 tok] = Q[16 x 128] . K^T      (K chunk [D/8][BS][8] is B-operand
//                                            order for ldmatrix, no transpose)
//   O[16 x 128]   += P[16 x 16] . V          (V chunk [D][BS] likewise)
// with P taken from the S accumulators in registers, online softmax per block.
#include "pa_common.cuh"

namespace pa {

namespace {

constexpr int kTWarps = 8;
constexpr int kTThreads = kTWarps * 32;
constexpr int kRows = kTWarps * 16;
constexpr int kTStages = 8;
constexpr int kTStageBytes = 2 * kChunkBytes;
constexpr int kTableCap = 2048;  // block ids kept in shared memory per CTA
constexpr int kTSmemBytes = kTStages * kTStageBytes + kTableCap * 4 + 2 * kTStages * 8;

__global__ void __launch_bounds__(kTThreads, 1)
tile_attention_kernel(const AttnParams p, const TileWork *__restrict__ work) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t *ring = smem;
  int *tbl = reinterpret_cast<int *>(smem + kTStages * kTStageBytes);
  uint64_t *full = reinterpret_cast<uint64_t *>(smem + kTStages * kTStageBytes + kTableCap * 4);
  uint64_t *empty = full + kTStages;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gid = lane >> 2, tig = lane & 3, mi = lane >> 3, mr = lane & 7;
  const TileWork w = work[blockIdx.x];
  const int seq = w.seq, h = w.kv_head, G = p.G;
  const int kv_len = p.context_lens[seq];
  const int q0 = p.cu_q_lens[seq];
  const int q_len = p.cu_q_lens[seq + 1] - q0;
  // keys visible to the last query of the tile
  const int kv_hi = min(kv_len, kv_len - q_len + w.q_begin + w.q_count);
  const int nblk = kv_hi > 0 ? (kv_hi + kBlockSize - 1) / kBlockSize : 0;
  const int32_t *table = p.block_tables + (int64_t)seq * p.MB;

  for (int i = tid; i < nblk && i < kTableCap; i += kTThreads) {
    uint32_t id = (uint32_t)table[i];
    if (id >= p.num_blocks) {
      atomicOr(p.err, kErrBlockRange);
      id = 0;
    }
    tbl[i] = (int)id;
  }
  if (tid == 0) {
    for (int s = 0; s < kTStages; s++) {
      mbar_init(smem_u32(&full[s]), 1);
      mbar_init(smem_u32(&empty[s]), kTWarps);
    }
    mbar_fence_init();
  }
  __syncthreads();

  auto block_id = [&](int b) -> uint32_t {
    if (b < kTableCap) return (uint32_t)tbl[b];
    uint32_t id = (uint32_t)table[b];
    if (id >= p.num_blocks) {
      atomicOr(p.err, kErrBlockRange);
      id = 0;
    }
    return id;
  };
  auto issue = [&](int b) {  // one thread
    const int st = b % kTStages;
    const size_t chunk = (size_t)block_id(b) * p.Hkv + h;
    const uint32_t bar = smem_u32(&full[st]), dst = smem_u32(ring) + st * kTStageBytes;
    mbar_expect_tx(bar, kTStageBytes);
    bulk_g2s(dst, p.k_pool + chunk * kChunkElems, kChunkBytes, bar);
    bulk_g2s(dst + kChunkBytes, p.v_pool + chunk * kChunkElems, kChunkBytes, bar);
  };
  if (tid == 0)
    for (int b = 0; b < kTStages && b < nblk; b++) issue(b);

  // ---- this warp's 16 rows -----------------------------------------------------
  // rows gid and gid+8 of the warp; row -> (query token, head of group)
  int lim[2];             // keys visible to the row (0 for an absent row)
  const __nv_bfloat16 *qrow[2];
  __nv_bfloat16 *orow[2];
#pragma unroll
  for (int r = 0; r < 2; r++) {
    const int row = warp * 16 + gid + 8 * r;
    const int qi = row / G, g = row - qi * G;
    if (qi < w.q_count) {
      const int qj = w.q_begin + qi;
      lim[r] = max(kv_len - q_len + qj + 1, 0);
      qrow[r] = p.q + (int64_t)(q0 + qj) * p.q_stride + (int64_t)(h * G + g) * kHeadSize;
      orow[r] = p.out + (int64_t)(q0 + qj) * p.out_stride + (int64_t)(h * G + g) * kHeadSize;
    } else {
      lim[r] = 0;
      qrow[r] = nullptr;
      orow[r] = nullptr;
    }
  }
  uint32_t qa[8][4];
#pragma unroll
  for (int j = 0; j < 8; j++) {
#pragma unroll
    for (int r = 0; r < 2; r++) {
      if (qrow[r]) {
        const uint32_t *qp = reinterpret_cast<const uint32_t *>(qrow[r]);
        qa[j][r] = __ldg(qp + 8 * j + tig);
        qa[j][2 + r] = __ldg(qp + 8 * j + 4 + tig);
      } else {
        qa[j][r] = qa[j][2 + r] = 0u;
      }
    }
  }
  // smallest limit among the warp's rows that exist (for the mask test)
  int warp_min_lim = qrow[0] ? lim[0] : 0x7fffffff;
  if (qrow[1]) warp_min_lim = min(warp_min_lim, lim[1]);
#pragma unroll
  for (int o = 4; o <= 16; o <<= 1)
    warp_min_lim = min(warp_min_lim, __shfl_xor_sync(0xffffffffu, warp_min_lim, o));

  float o[16][4];
#pragma unroll
  for (int n = 0; n < 16; n++)
#pragma unroll
    for (int i = 0; i < 4; i++) o[n][i] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  const float sc_log2 = p.scale * kLog2e;
  const bool use_cap = p.softcap != 1.0f;
  bool dead = false;

  for (int b = 0; b < nblk; b++) {
    const int st = b % kTStages;
    const uint32_t par = (b / kTStages) & 1;
    if (!dead) {
      const bool ok = mbar_wait_bounded(smem_u32(&full[st]), par);
      if (!__all_sync(0xffffffffu, ok)) {
        dead = true;
        if (lane == 0) atomicOr(p.err, kErrTimeout);
      }
    }
    if (!dead) {
      const uint32_t ks = smem_u32(ring) + st * kTStageBytes, vs = ks + kChunkBytes;
      float s[2][4];
#pragma unroll
      for (int n = 0; n < 2; n++)
#pragma unroll
        for (int i = 0; i < 4; i++) s[n][i] = 0.f;
#pragma unroll
      for (int j = 0; j < 8; j++) {
        uint32_t kb[4];
        ldmatrix_x4(kb, ks + (2 * j + (mi & 1)) * 256 + ((mi >> 1) * 8 + mr) * 16);
        mma_bf16_16816(s[0], qa[j], kb[0], kb[1]);
        mma_bf16_16816(s[1], qa[j], kb[2], kb[3]);
      }
      const bool need_mask = (b + 1) * kBlockSize > warp_min_lim;
#pragma unroll
      for (int n = 0; n < 2; n++) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
          float x = s[n][i];
          if (use_cap) x = tanhf(x * p.scale / p.softcap) * p.softcap * kLog2e;
          else x *= sc_log2;
          if (need_mask) {
            const int tok = b * kBlockSize + n * 8 + 2 * tig + (i & 1);
            if (tok >= lim[i >> 1]) x = -INFINITY;
          }
          s[n][i] = x;
        }
      }
      float alpha[2];
#pragma unroll
      for (int r = 0; r < 2; r++) {
        float mx = fmaxf(fmaxf(s[0][2 * r], s[0][2 * r + 1]), fmaxf(s[1][2 * r], s[1][2 * r + 1]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m[r], mx);
        const float m_safe = m_new == -INFINITY ? 0.f : m_new;
        alpha[r] = fast_exp2(m[r] - m_safe);
        m[r] = m_new;
        float sum = 0.f;
#pragma unroll
        for (int n = 0; n < 2; n++)
#pragma unroll
          for (int c = 0; c < 2; c++) {
            const float e = fast_exp2(s[n][2 * r + c] - m_safe);
            s[n][2 * r + c] = e;
            sum += e;
          }
        l[r] = l[r] * alpha[r] + sum;
      }
      uint32_t pa_[4];
      pa_[0] = pack_bf16(s[0][0], s[0][1]);
      pa_[1] = pack_bf16(s[0][2], s[0][3]);
      pa_[2] = pack_bf16(s[1][0], s[1][1]);
      pa_[3] = pack_bf16(s[1][2], s[1][3]);
      // Clear V lanes of tokens past the context (they may hold NaN).
      const int valid = kv_len - b * kBlockSize;
      uint32_t vmask[2] = {0xffffffffu, 0xffffffffu};
      if (valid < kBlockSize) {
#pragma unroll
        for (int hh = 0; hh < 2; hh++) {
          const int t = hh * 8 + 2 * tig;
          vmask[hh] = (t < valid ? 0x0000ffffu : 0u) | (t + 1 < valid ? 0xffff0000u : 0u);
        }
      }
#pragma unroll
      for (int np = 0; np < 8; np++) {
        uint32_t vb[4];
        ldmatrix_x4(vb, vs + (np * 16 + (mi >> 1) * 8 + mr) * 32 + (mi & 1) * 16);
        vb[0] &= vmask[0]; vb[1] &= vmask[1]; vb[2] &= vmask[0]; vb[3] &= vmask[1];
#pragma unroll
        for (int q = 0; q < 2; q++) {
          float *oo = o[2 * np + q];
          oo[0] *= alpha[0]; oo[1] *= alpha[0]; oo[2] *= alpha[1]; oo[3] *= alpha[1];
        }
        mma_bf16_16816(o[2 * np], pa_, vb[0], vb[1]);
        mma_bf16_16816(o[2 * np + 1], pa_, vb[2], vb[3]);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(&empty[st]));
    // The issuing thread refills the stage once every warp has released it.
    if (tid == 0 && b + kTStages < nblk) {
      if (!mbar_wait_bounded(smem_u32(&empty[st]), par)) atomicOr(p.err, kErrTimeout);
      else issue(b + kTStages);
    }
  }

#pragma unroll
  for (int r = 0; r < 2; r++) {
    float v = l[r];
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    const float inv = v > 0.f ? 1.f / v : 0.f;
    if (orow[r]) {
      uint32_t *op = reinterpret_cast<uint32_t *>(orow[r]);
#pragma unroll
      for (int n = 0; n < 16; n++)
        op[n * 4 + tig] = pack_bf16(o[n][2 * r] * inv, o[n][2 * r + 1] * inv);
    }
  }
}

}  // namespace

int tile_queries_per_cta(int G) { return kRows / G; }

cudaError_t tile_configure() {
  return cudaFuncSetAttribute(tile_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              kTSmemBytes);
}

cudaError_t launch_tile_attention(const AttnParams &p, const TileWork *work_dev, int num_work,
                                  cudaStream_t st) {
  if (num_work <= 0) return cudaSuccess;
  tile_attention_kernel<<<num_work, kTThreads, kTSmemBytes, st>>>(p, work_dev);
  __atomic_fetch_add(&g_launch_count, 1ull, __ATOMIC_RELAXED);
  return cudaGetLastError();
}

}  // namespace pa
