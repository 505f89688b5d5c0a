// Tile kernel for long-query sequences (chunked prefill) over 16-bit pools of
// 16-token blocks: tcgen05 tensor cores, TMEM accumulators, every KV operand
// brought in by the copy engine through the block table (TMA gather), sm_100a.
//
// The reference has no paged prefill kernel: its prefill is dense causal
// attention followed by a scatter into the pool
// (crates/mlx-core/src/transformer/block.rs:279-317).  This kernel attends
// directly over the pool: query j of a sequence sees keys [0, kv_len-q_len+j].
//
// One CTA = 256 rows of one (sequence, kv head): a row is a (query token, query
// head of the GQA group) pair, token-major, i.e. two 128-row Q tiles that share
// every KV tile.  KV tiles are 64 tokens (4 blocks) and the logits of a Q tile
// are DOUBLE-BUFFERED in TMEM, so that S(j+1) = Q.K(j+1)^T is computed while
// the softmax warps still work on S(j): per Q tile the only serial chain left
// is the softmax itself, and the tensor pipe always has the other Q tile's
// P.V and the next logits to run.
//
// Roles (12 warps):
//   warps 0-3   softmax of Q tile 0 (thread = row = TMEM lane)
//   warps 4-7   softmax of Q tile 1; both groups first stage Q (16-byte cp.async,
//               128-byte swizzle K-major)
//   warps 8-10  copy issue (a tensor copy costs its issuing thread about a hundred
//               cycles, so the twenty copies of a tile are shared out).  K tile: sixteen gather copies
//               (cp.async.bulk.tensor.2d.tile::gather4) over the K pool viewed as rows
//               of 256 bytes, row = (chunk, d/8): one copy fetches row d/8 of the
//               tile's four blocks and lands them side by side, which is the
//               un-swizzled K-major core-matrix order [d/8][block][token][8] the MMA
//               reads.  V tile: one tiled copy per block with the 32-byte swizzle (a
//               V chunk [d][token] is K-major for P.V once swizzled).  This CTA's
//               shared memory only; no multicast.
//   warp 11     allocates TMEM; one elected lane issues every tcgen05.mma
//
// TMEM (512 columns): per Q tile i two logit buffers of 64 fp32 columns
// (columns i*128 + b*64) and the output accumulator of 128 columns (256 + i*128).
// P (16-bit) is written over the first 32 columns of its logit buffer and fed back
// as the A operand of P.V, so P never touches shared memory.
//   S_i(j) = Q_i . K(j)^T    A = Q_i (smem), B = K tile (smem), 8 x (M128 N64 K16)
//   O_i   += P_i(j) . V(j)   A = P_i (TMEM), B = V block (smem), 4 x (M128 N128 K16)
// Issue order: S_0(0) S_1(0) S_0(1) S_1(1), then per tile j:
//   [P_0(j) ready] PV_0(j) S_1(j+1)   [P_1(j) ready] PV_1(j) S_0(j+2)
// Online softmax keeps a stale row maximum and rescales O only when the
// maximum grows by more than 2^8.
//
// Every wait is bounded; on expiry the CTA raises the error word, every role
// leaves its loop, copies in flight are drained and TMEM is freed.
#include <cuda.h>

#include "pa_common.cuh"
#include "tile_common.cuh"

namespace pa {

namespace {

using namespace tile;

constexpr int kTileTok = 64;           // tokens per KV tile
constexpr int kTileBlocks = kTileTok / kBlockSize;
constexpr int kSlab = 128 * 128;       // one Q operand slab: 128 rows x 128 B
constexpr int kQBytes = 4 * kSlab;     // 2 Q tiles x 2 slabs
constexpr int kStage = kTileTok * kHeadSize * 2;  // one K or V tile: 16 KB
constexpr int kNK = 4, kNV = 4;        // ring depths
constexpr int kTblCap = 2048;          // block ids staged per CTA (32768 tokens' worth)
enum {
  B_QFULL = 0,
  B_KFULL = 1,                 // kNK
  B_VFULL = B_KFULL + kNK,     // kNV
  B_KEMPTY = B_VFULL + kNV,    // kNK
  B_VEMPTY = B_KEMPTY + kNK,   // kNV
  B_SFULL = B_VEMPTY + kNV,    // [tile][buf]
  B_PREADY = B_SFULL + 4,      // [tile][buf]
  B_PVDONE = B_PREADY + 4,     // [tile]
  B_VTAIL = B_PVDONE + 2,
  kNumBars = B_VTAIL + 1
};
constexpr int kSmem64 = 1024 + kQBytes + (kNK + kNV) * kStage + kTblCap * 4 + kNumBars * 8 + 16;
static_assert(kSmem64 <= 232448, "shared memory per CTA");
constexpr int kThreads64 = 12 * 32;
constexpr int kProducers = 3;

// Four rows of the K pool's row view -> 1 KB of shared memory (rows side by side).
__device__ __forceinline__ void tma_gather4(uint32_t dst, const CUtensorMap *map, int r0, int r1, int r2,
                                            int r3, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3, %4, %5, %6}], [%7];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(0), "r"(r0), "r"(r1), "r"(r2), "r"(r3), "r"(bar)
      : "memory");
}

// K tile of 64 tokens, K-major without swizzle: core matrix = 8 tokens x 16 B contiguous;
// 8-token groups 128 B apart (stride byte offset); the two 8-element d-chunks of one K=16
// step 1024 B apart (leading byte offset).
__device__ __forceinline__ uint64_t k_tile64_desc(uint32_t smem_addr) {
  return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | (64ull << 16) | (8ull << 32) | (1ull << 46);
}
__host__ __device__ constexpr uint32_t idesc_of(bool f16, uint32_t n) {
  return (1u << 4) | (f16 ? 0u : ((1u << 7) | (1u << 10))) | ((n >> 3) << 17) | ((128u >> 4) << 24);
}

// One pass over a row's 64 logits (thread = row): probabilities against the reference
// maximum (mc = m_used * c), the raw row maximum and the row sum.  Each 32-column chunk's
// probabilities are packed to 16-bit pairs and stored to TMEM (over the first 32 columns
// of the logit buffer, whose values live in registers by now) as soon as they exist.
template <bool CAP, bool MASK, bool F16>
__device__ __forceinline__ void row_pass64(uint32_t s_t, const uint32_t (&s0)[32], const uint32_t (&s1)[32],
                                           float c, float mc, int lim, int tok0, float cap_in,
                                           float cap_out, float &mx_out, float &sum_out) {
  float mxa[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
  float sma[4] = {0.f, 0.f, 0.f, 0.f};
  auto process32 = [&](const uint32_t (&r)[32], int col0) {
    uint32_t t16[16];
#pragma unroll
    for (int e = 0; e < 32; e += 2) {
      float x0 = __uint_as_float(r[e]), x1 = __uint_as_float(r[e + 1]);
      if (CAP) {
        x0 = tanhf(x0 * cap_in) * cap_out;
        x1 = tanhf(x1 * cap_in) * cap_out;
      }
      if (MASK) {
        if (tok0 + col0 + e >= lim) x0 = -INFINITY;
        if (tok0 + col0 + e + 1 >= lim) x1 = -INFINITY;
      }
      mxa[(e >> 1) & 3] = fmaxf(mxa[(e >> 1) & 3], fmaxf(x0, x1));
      const float p0 = fast_exp2(fmaf(x0, c, -mc)), p1 = fast_exp2(fmaf(x1, c, -mc));
      sma[(e >> 1) & 3] += p0 + p1;
      t16[e >> 1] = pack2<F16>(p0, p1);
    }
    tmem_st16(s_t + (col0 >> 1), t16);
  };
  process32(s0, 0);
  process32(s1, 32);
  mx_out = fmaxf(fmaxf(mxa[0], mxa[1]), fmaxf(mxa[2], mxa[3]));
  sum_out = (sma[0] + sma[1]) + (sma[2] + sma[3]);
}

template <bool CAP, bool F16>
__global__ void __launch_bounds__(kThreads64, 1)
tile_attention_tc64_kernel(const AttnParams p, const TileWork *__restrict__ work,
                           const __grid_constant__ CUtensorMap k_map,
                           const __grid_constant__ CUtensorMap v_map) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *gen = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t q_s = base, k_s = base + kQBytes, v_s = k_s + kNK * kStage;
  int *tbl = reinterpret_cast<int *>(gen + kQBytes + (kNK + kNV) * kStage);
  uint64_t *bars = reinterpret_cast<uint64_t *>(gen + kQBytes + (kNK + kNV) * kStage + kTblCap * 4);
  uint32_t *tmem_holder = reinterpret_cast<uint32_t *>(bars + kNumBars);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_holder + 1);
  auto bar = [&](int i) { return smem_u32(&bars[i]); };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const TileWork w = work[blockIdx.x];
  const int seq = w.seq, h = w.kv_head, G = p.G;
  const int kv_len = p.context_lens[seq];
  const int q0 = p.cu_q_lens[seq];
  const int q_len = p.cu_q_lens[seq + 1] - q0;
  const int kv_hi = max(0, min(kv_len, kv_len - q_len + w.q_begin + w.q_count));
  const int n_tiles = (kv_hi + kTileTok - 1) / kTileTok;
  const int nblk = (kv_hi + kBlockSize - 1) / kBlockSize;
  const int32_t *table = p.block_tables + (int64_t)seq * p.MB;

  // ---- set-up ---------------------------------------------------------------------
  for (int i = tid; i < nblk && i < kTblCap; i += kThreads64) {
    uint32_t id = (uint32_t)table[i];
    if (id >= p.num_blocks) {
      atomicOr(p.err, kErrBlockRange);
      id = 0;
    }
    tbl[i] = (int)id;
  }
  if (tid == 0) {
    mbar_init(bar(B_QFULL), 256);
    for (int s = 0; s < kNK; s++) {
      mbar_init(bar(B_KFULL + s), 1);
      mbar_init(bar(B_KEMPTY + s), 1);
    }
    for (int s = 0; s < kNV; s++) {
      mbar_init(bar(B_VFULL + s), 2);  // the two warps that fetch V, each once its blocks are in order
      mbar_init(bar(B_VEMPTY + s), 1);
    }
    for (int s = 0; s < 4; s++) {
      mbar_init(bar(B_SFULL + s), 1);
      mbar_init(bar(B_PREADY + s), 128);
    }
    mbar_init(bar(B_PVDONE + 0), 1);
    mbar_init(bar(B_PVDONE + 1), 1);
    mbar_init(bar(B_VTAIL), 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 11) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(
        smem_u32(tmem_holder)));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_holder;
  bool failed = false;
  auto block_id = [&](int b) -> uint32_t {
    if (b < kTblCap) return (uint32_t)tbl[b];
    uint32_t id = (uint32_t)table[b];
    if (id >= p.num_blocks) {
      atomicOr(p.err, kErrBlockRange);
      id = 0;
    }
    return id;
  };

  if (n_tiles > 0) {
    if (warp >= 8 && warp < 8 + kProducers) {
      // =========================== copy issue =======================================
      const int pw = warp - 8;
      const int total_chunks = (int)p.num_blocks * p.Hkv;
      // Tokens past the context inside the last block may hold anything; P is 0 there but
      // 0*NaN is NaN, so that block lands on a barrier of its own and its stray columns are
      // cleared before the tile is published.
      const int last_gb = (kv_len - 1) >> 4;
      const int last_valid = kv_len - last_gb * kBlockSize;
      const bool have_tail = last_valid < kBlockSize && last_gb < nblk;
      // K rows d/8 = pw, pw + 3, ... of the tile's four blocks, one gather copy per lane.
      // Warp 0 announces the tile's bytes; copies of the other warps may land before that,
      // which the barrier allows (the phase cannot complete before the announcing arrival).
      auto issue_k = [&](int t) {
        if (t >= kNK && !wait_bar(bar(B_KEMPTY + t % kNK), ((t / kNK) - 1) & 1, abort_flag)) {
          failed = true;
          return;
        }
        const uint32_t full = bar(B_KFULL + t % kNK);
        if (pw == 0 && lane == 0) mbar_expect_tx(full, kStage);
        const int c = pw + kProducers * lane;
        if (c < 16) {
          int r[4];
#pragma unroll
          for (int b = 0; b < 4; b++) {
            // blocks past the last one repeat it: their logits are masked (every row's
            // limit is at most the tile's last key), so any finite-or-not value will do
            const int gb = min(t * kTileBlocks + b, nblk - 1);
            r[b] = ((int)block_id(gb) * p.Hkv + h) * 16 + c;
          }
          tma_gather4(k_s + (t % kNK) * kStage + c * 1024, &k_map, r[0], r[1], r[2], r[3], full);
        }
      };
      // V blocks 2 (pw - 1) and 2 (pw - 1) + 1 of the tile, by warps 1 and 2
      auto issue_v = [&](int t) {
        if (t >= kNV && !wait_bar(bar(B_VEMPTY + t % kNV), ((t / kNV) - 1) & 1, abort_flag)) {
          failed = true;
          return;
        }
        const uint32_t full = bar(B_VFULL + t % kNV);
        const int tail_b = (have_tail && last_gb / kTileBlocks == t) ? last_gb % kTileBlocks : -1;
        const int b0 = 2 * (pw - 1);
        const bool own_tail = tail_b == b0 || tail_b == b0 + 1;
        if (lane < 2) {
          const int b = b0 + lane, gb = t * kTileBlocks + b;
          const int chunk = gb < nblk ? (int)block_id(gb) * p.Hkv + h : total_chunks;
          const uint32_t dst = v_s + (t % kNV) * kStage + b * kChunkBytes;
          if (b == tail_b) {
            mbar_expect_tx(bar(B_VTAIL), kChunkBytes);
            tma_load_v_block(dst, &v_map, 0, chunk, bar(B_VTAIL));
          } else {
            tma_load_v_block(dst, &v_map, 0, chunk, full);
          }
        }
        if (own_tail) {
          if (!wait_bar(bar(B_VTAIL), 0, abort_flag)) {
            failed = true;
            return;
          }
          uint8_t *vgen = gen + kQBytes + kNK * kStage + (t % kNV) * kStage + tail_b * kChunkBytes;
          for (int d = lane; d < 128; d += 32)
            for (int tk = last_valid; tk < kBlockSize; tk++)
              *reinterpret_cast<uint16_t *>(vgen + d * 32 + ((((tk >> 3) ^ (d >> 2)) & 1) << 4) + (tk & 7) * 2) = 0;
          fence_proxy_async();
          __syncwarp();
        }
        if (lane == 0) mbar_expect_tx(full, (uint32_t)(own_tail ? 1 : 2) * kChunkBytes);
      };
      issue_k(0);
      if (n_tiles > 1 && !failed) issue_k(1);
      for (int t = 0; t < n_tiles && !failed; t++) {
        if (t + 2 < n_tiles) issue_k(t + 2);
        if (pw > 0 && !failed) issue_v(t);
      }
    } else if (warp == 11) {
      // =========================== MMA issuer ========================================
      // The whole warp walks the loop so that descriptors and addresses stay warp-uniform
      // (uniform registers feed tcgen05.mma directly); one elected lane issues.
      constexpr uint32_t kIdescS = idesc_of(F16, kTileTok), kIdescPV = idesc_of(F16, 128);
      const bool leader = elect_one();
      auto issue_s = [&](int i, int t) {  // S_i(t) into logit buffer t & 1
        const uint32_t kst = k_s + (t % kNK) * kStage;
        const uint32_t d = tmem + i * 128 + (t & 1) * 64;
#pragma unroll
        for (int kk = 0; kk < 8; kk++) {
          const uint32_t koff = (kk >> 2) * kSlab + (kk & 3) * 32;
          if (leader)
            umma_ss(d, sw128_desc(q_s + i * 2 * kSlab + koff), k_tile64_desc(kst + kk * 2048), kIdescS,
                    kk > 0 ? 1u : 0u);
        }
        if (leader) tc_commit(bar(B_SFULL + i * 2 + (t & 1)));
      };
      auto issue_pv = [&](int i, int t) {
        const uint32_t vst = v_s + (t % kNV) * kStage;
        const uint32_t pa = tmem + i * 128 + (t & 1) * 64;
#pragma unroll
        for (int kk = 0; kk < kTileBlocks; kk++) {
          if (leader)
            umma_ts(tmem + 256 + i * 128, pa + kk * 8, v_block_desc(vst + kk * kChunkBytes), kIdescPV,
                    (t > 0 || kk > 0) ? 1u : 0u);
        }
        if (leader) tc_commit(bar(B_PVDONE + i));
      };
      do {
        if (!wait_bar(bar(B_QFULL), 0, abort_flag)) { failed = true; break; }
        for (int t = 0; t < 2 && t < n_tiles && !failed; t++) {
          if (!wait_bar(bar(B_KFULL + t), 0, abort_flag)) { failed = true; break; }
          tc_fence_after();
          issue_s(0, t);
          issue_s(1, t);
          if (leader) tc_commit(bar(B_KEMPTY + t));
        }
        // Steady state, the two Q tiles half a period apart:
        //   [P_0(j)] PV_0(j) S_1(j+1)   [P_1(j)] PV_1(j) S_0(j+2)
        // A logit buffer is overwritten by S two tiles on; the tensor pipe starts an MMA
        // before the one ahead of it has finished reading its operands, so an overwrite
        // issued right behind the P.V that reads the buffer can clobber what that P.V has
        // yet to fetch (seen as wrong rows 64-127 of a tile).  In this order at least the
        // other Q tile's four P.V MMAs run between a P.V and the overwrite of its P.
        auto k_ready = [&](int t) {
          return wait_bar(bar(B_KFULL + t % kNK), (t / kNK) & 1, abort_flag);
        };
        for (int j = 0; j < n_tiles && !failed; j++) {
          if (!wait_bar(bar(B_PREADY + 0 + (j & 1)), (j >> 1) & 1, abort_flag)) { failed = true; break; }
          if (!wait_bar(bar(B_VFULL + j % kNV), (j / kNV) & 1, abort_flag)) { failed = true; break; }
          tc_fence_after();
          issue_pv(0, j);
          if (j >= 1 && j + 1 < n_tiles) {  // K(j+1) was waited for when S_0(j+1) was issued
            issue_s(1, j + 1);
            if (leader) tc_commit(bar(B_KEMPTY + (j + 1) % kNK));
          }
          if (!wait_bar(bar(B_PREADY + 2 + (j & 1)), (j >> 1) & 1, abort_flag)) { failed = true; break; }
          tc_fence_after();
          issue_pv(1, j);
          if (leader) tc_commit(bar(B_VEMPTY + j % kNV));
          if (j + 2 < n_tiles) {
            if (!k_ready(j + 2)) { failed = true; break; }
            tc_fence_after();
            issue_s(0, j + 2);
          }
          __syncwarp();
        }
      } while (false);
    } else {
      // =========================== softmax + epilogue ================================
      // Q first: 2 tiles x 128 rows x 16 pieces of 16 B, every softmax thread its share
      for (int it = 0; it < 16; it++) {
        const int e = it * 256 + tid;
        const int row = e >> 4, c = e & 15;  // row 0..255
        const int tile_i = row >> 7, r = row & 127;
        const int qi = row / G, g = row - qi * G;
        const bool have = qi < w.q_count;
        const elem16 *src =
            have ? p.q + (int64_t)(q0 + w.q_begin + qi) * p.q_stride + (int64_t)(h * G + g) * kHeadSize + c * 8
                 : p.q;
        cp_async16(q_s + (tile_i * 2 + (c >> 3)) * kSlab + sw128_off(r, c & 7), src, have ? 16u : 0u);
      }
      cp_async_commit();
      cp_async_wait<0>();
      fence_proxy_async();
      mbar_arrive(bar(B_QFULL));

      const int i = warp >> 2;                     // Q tile
      const int row = (warp & 3) * 32 + lane;      // row within the tile = TMEM lane
      const int grow = i * 128 + row;              // row within the CTA
      const int qi = grow / G, g = grow - qi * G;
      const bool have = qi < w.q_count;
      const int lim = have ? max(kv_len - q_len + w.q_begin + qi + 1, 0) : 0;
      int warp_min_lim = lim;
#pragma unroll
      for (int o = 16; o >= 1; o >>= 1)
        warp_min_lim = min(warp_min_lim, __shfl_xor_sync(0xffffffffu, warp_min_lim, o));
      const uint32_t lane_base = ((uint32_t)((warp & 3) * 32)) << 16;
      const uint32_t s_base = tmem + lane_base + i * 128;
      const uint32_t o_t = tmem + lane_base + 256 + i * 128;
      const float c = p.scale * kLog2e;
      // soft-capping: x -> tanh(x*scale/cap)*cap/scale, so that x*c is the capped logit
      const float cap_in = p.scale / p.softcap, cap_out = p.softcap / p.scale;
      float m_used = -INFINITY, l = 0.f;
      uint32_t s0[32], s1[32];  // the row's logits of the current tile

      for (int j = 0; j < n_tiles && !failed; j++) {
        const uint32_t s_t = s_base + (j & 1) * 64;
        if (!wait_bar(bar(B_SFULL + i * 2 + (j & 1)), (j >> 1) & 1, abort_flag)) { failed = true; break; }
        tc_fence_after();
        const bool need_mask = (j + 1) * kTileTok > warp_min_lim;
        const int tok0 = j * kTileTok;
        float mx, sum;
        tmem_ld32(s_t, s0);
        tmem_ld32(s_t + 32, s1);
        tmem_wait_ld32(s0);  // waits for both loads
        tmem_wait_ld32(s1);  // already complete: ties the registers to the wait
        auto pass = [&]() {
          const float mc = m_used == -INFINITY ? 0.f : m_used * c;
          if (need_mask) row_pass64<CAP, true, F16>(s_t, s0, s1, c, mc, lim, tok0, cap_in, cap_out, mx, sum);
          else row_pass64<CAP, false, F16>(s_t, s0, s1, c, mc, lim, tok0, cap_in, cap_out, mx, sum);
        };
        // Optimistic pass against the maximum carried from earlier tiles (for the first
        // tile: against 0, result discarded unless the logits happen to be small).  It
        // already writes P; a second pass, from the same registers, overwrites it.
        pass();
        // P.V of tile j-1 has long completed by now (it was issued a whole pass ago); the
        // wait is made on EVERY tile so that this warp sees every phase of the barrier: a
        // parity wait that skipped phases could not tell phase j-1 from phase j-3 or j+1.
        // After it, O_i holds tiles 0..j-1.
        if (j > 0 && !wait_bar(bar(B_PVDONE + i), (j - 1) & 1, abort_flag)) { failed = true; break; }
        // stale-maximum rule: move the reference only when it would grow by > 2^8
        const bool grew = mx > m_used && !((mx - m_used) * c <= 8.f);
        if (__any_sync(0xffffffffu, grew)) {
          float factor = 1.f;
          if (grew) {
            factor = m_used == -INFINITY ? 0.f : fast_exp2((m_used - mx) * c);
            m_used = mx;
          }
          if (j > 0) {
            tc_fence_after();
#pragma unroll
            for (int ch = 0; ch < 4; ch++) {
              uint32_t r[32];
              tmem_ld32(o_t + ch * 32, r);
              tmem_wait_ld32(r);
#pragma unroll
              for (int e = 0; e < 32; e++) r[e] = __float_as_uint(__uint_as_float(r[e]) * factor);
              tmem_st32(o_t + ch * 32, r);
            }
            tmem_wait_st();
          }
          l *= factor;
          pass();
        }
        l += sum;
        // P (16-bit) now covers the first 32 columns of this logit buffer
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(bar(B_PREADY + i * 2 + (j & 1)));
      }
      // epilogue: O / l -> 16-bit rows (phase n-2 of the barrier was seen in the last tile)
      if (!failed && wait_bar(bar(B_PVDONE + i), (n_tiles - 1) & 1, abort_flag)) {
        tc_fence_after();
        const float inv = l > 0.f ? 1.f / l : 0.f;
        elem16 *orow = have ? p.out + (int64_t)(q0 + w.q_begin + qi) * p.out_stride +
                                         (int64_t)(h * G + g) * kHeadSize
                                   : nullptr;
#pragma unroll
        for (int ch = 0; ch < 4; ch++) {
          uint32_t r[32];
          tmem_ld32(o_t + ch * 32, r);
          tmem_wait_ld32(r);
          if (have) {
#pragma unroll
            for (int e = 0; e < 32; e += 8) {
              uint4 v;
              v.x = pack2<F16>(__uint_as_float(r[e]) * inv, __uint_as_float(r[e + 1]) * inv);
              v.y = pack2<F16>(__uint_as_float(r[e + 2]) * inv, __uint_as_float(r[e + 3]) * inv);
              v.z = pack2<F16>(__uint_as_float(r[e + 4]) * inv, __uint_as_float(r[e + 5]) * inv);
              v.w = pack2<F16>(__uint_as_float(r[e + 6]) * inv, __uint_as_float(r[e + 7]) * inv);
              *reinterpret_cast<uint4 *>(orow + ch * 32 + e) = v;
            }
          }
        }
      } else {
        failed = true;
      }
    }
  } else if (warp < 8) {
    // nothing to attend: zero rows
    const int grow = (warp >> 2) * 128 + (warp & 3) * 32 + lane;
    const int qi = grow / G, g = grow - qi * G;
    if (qi < w.q_count) {
      uint4 *orow = reinterpret_cast<uint4 *>(p.out + (int64_t)(q0 + w.q_begin + qi) * p.out_stride +
                                              (int64_t)(h * G + g) * kHeadSize);
      for (int e = 0; e < 16; e++) orow[e] = make_uint4(0, 0, 0, 0);
    }
  }

  if (failed) atomicOr(p.err, kErrTimeout);
  // ---- teardown -------------------------------------------------------------------
  // A role that gave up may have left copies in flight towards this CTA's shared memory;
  // the CTA must not exit (and its memory be handed on) before they have landed.  Every
  // copy that was issued completes on its barrier whether or not anybody waits, so a
  // bounded wait on the full barriers of the last tiles is enough; in the normal case they
  // completed long ago.
  tc_fence_before();
  __syncthreads();
  if (*abort_flag && warp == 8) {
    const long long t0 = clock64();
    while (clock64() - t0 < (1ll << 22)) {
    }  // ~2 ms: far longer than any copy takes; nothing below reads shared memory
  }
  __syncthreads();
  if (warp == 11) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem));
  }
}

}  // namespace

int tile64_queries_per_cta(int G) { return 256 / G; }

cudaError_t tile64_configure() {
  cudaError_t e = cudaSuccess;
  auto set = [&](auto kernel) {
    if (e == cudaSuccess) e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem64);
  };
  set(tile_attention_tc64_kernel<false, false>);
  set(tile_attention_tc64_kernel<true, false>);
  set(tile_attention_tc64_kernel<false, true>);
  set(tile_attention_tc64_kernel<true, true>);
  return e;
}

// Tensor map over one K pool of 16-token blocks viewed as rows of 256 bytes: row
// (chunk * 16 + d/8) holds [token][8 elements] of that chunk; box = one row, so that a
// gather copy fetches the same d/8 row of four blocks.  The encoder is a driver entry
// point, fetched through the runtime so that the library does not link against the driver.
cudaError_t tile64_encode_k_map(TensorMapBlob *out, const void *k_pool, uint64_t num_chunks) {
  static_assert(sizeof(CUtensorMap) == sizeof(TensorMapBlob), "tensor map size");
  using EncodeFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  void *fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
  if (e != cudaSuccess) return e;
  if (!fn || qres != cudaDriverEntryPointSuccess) return cudaErrorNotSupported;
  const cuuint64_t dims[2] = {128, num_chunks * 16};
  const cuuint64_t strides[1] = {256};
  const cuuint32_t box[2] = {128, 1}, elem_strides[2] = {1, 1};
  const CUresult r = reinterpret_cast<EncodeFn>(fn)(
      reinterpret_cast<CUtensorMap *>(out), CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void *>(k_pool),
      dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

cudaError_t launch_tile64_attention(const AttnParams &p, const TileWork *work_dev, int num_work,
                                    const TensorMapBlob *k_map, const TensorMapBlob *v_map, cudaStream_t st) {
  if (num_work <= 0) return cudaSuccess;
  if (!k_map || !v_map || p.is_fp8 || p.bs_shift != 0) return cudaErrorInvalidValue;
  const CUtensorMap &km = *reinterpret_cast<const CUtensorMap *>(k_map);
  const CUtensorMap &vm = *reinterpret_cast<const CUtensorMap *>(v_map);
  const bool cap = p.softcap != 1.0f, f16 = p.is_f16 != 0;
  auto go = [&](auto kernel) { kernel<<<num_work, kThreads64, kSmem64, st>>>(p, work_dev, km, vm); };
  if (cap && f16) go(tile_attention_tc64_kernel<true, true>);
  else if (cap) go(tile_attention_tc64_kernel<true, false>);
  else if (f16) go(tile_attention_tc64_kernel<false, true>);
  else go(tile_attention_tc64_kernel<false, false>);
  __atomic_fetch_add(&g_launch_count, 1ull, __ATOMIC_RELAXED);
  return cudaGetLastError();
}

}  // namespace pa
