// Tile kernel for long-query sequences (chunked prefill) over the paged cache:
// tcgen05 tensor cores with TMEM accumulators, sm_100a.
//
// The reference has no paged prefill kernel: its prefill is dense causal
// attention followed by a scatter into the pool
// (crates/mlx-core/src/transformer/block.rs:279-317).  This kernel attends
// directly over the pool: query j of a sequence sees keys [0, kv_len-q_len+j].
//
// One CTA = 256 rows of one (sequence, kv head): a row is a (query token, query
// head of the GQA group) pair, token-major, i.e. two 128-row Q tiles that share
// every KV tile.  KV tiles are 128 tokens (8 blocks).
//
// Roles (16 warps, four warpgroups):
//   warps 0-3   softmax of Q tile 0 (thread = row = TMEM lane)
//   warps 4-7   softmax of Q tile 1
//   warps 8-11  producers: gather the 4 KB K and V chunks of the tile's blocks
//               through the block table with 16-byte cp.async.  The pool layouts
//               are already tensor-core operand layouts up to a block interleave:
//               K chunk [d/8][tok][8] is the un-swizzled K-major core-matrix order
//               (256-byte runs placed as [d/8][block][tok][8]); V chunk [d][tok] is
//               the 32-byte-swizzle K-major order (halves of rows 4..7 swapped).
//               Runs stay contiguous on both sides of the copy.
//   warp 12     allocates TMEM; one lane issues every tcgen05.mma (warps 13-15 complete
//               the fourth warpgroup; with an FP8 cache they convert the V tiles)
//
// TMEM (512 columns): S0 | S1 | O0 | O1, 128 fp32 columns each.  P (bf16) is
// written over the first 64 columns of its S and fed back as the A operand of
// the P.V product, so P never touches shared memory.
//   S_i = Q_i . K^T        A = Q_i (smem), B = K tile (smem), 8 x (M128 N128 K16)
//   O_i += P_i . V         A = P_i (TMEM), B = V tile (smem), 8 x (M128 N128 K16)
// Issue order S0 S1 | PV0 S0' PV1 S1' | ... so that the softmax of one Q tile
// overlaps the tensor work of the other.  Online softmax keeps a stale row
// maximum and rescales O only when the maximum grows by more than 2^8.
//
// FP8 (E4M3) pools (template flag FP8): the cache bytes of a tile come in by cp.async one
// tile ahead into a 32 KB staging area, are turned into f16 by the integer conversion of
// fp8x4_to_f16 (K by the producers, V by warps 13-15; the variant that reads exponent
// field 15 as infinity / NaN once the cache may hold such a byte) and stored where the
// 16-bit copies would have landed; the tensor cores run on f16
// operands (bf16 queries are converted on the way in, P is packed as f16) and the
// dequantisation factors ride on the logit scale and on the final normalisation.
//
// Every wait is bounded; on expiry the CTA raises the error word, every role
// leaves its loop, in-flight copies are drained and TMEM is freed.
#include <cuda.h>

#include <type_traits>

#include "pa_common.cuh"
#include "tile_common.cuh"

namespace pa {

namespace {

using namespace tile;

constexpr int kQRows = 128;            // rows per Q tile
constexpr int kTileTok = 128;          // tokens per KV tile
constexpr int kSlab = 128 * 128;       // one operand slab: 128 rows x 128 B
constexpr int kQBytes = 4 * kSlab;     // 2 Q tiles x 2 slabs
constexpr int kStage = 2 * kSlab;      // one K or V tile
// Block ids staged per CTA (ids beyond are read from the table in memory): 32768 tokens'
// worth, or 7168 with an FP8 cache, whose raw bytes take 32 KB of the shared memory.
template <bool FP8> constexpr int kTblCapOf = FP8 ? 448 : 2048;
constexpr int kRawTile = 16384;        // FP8: cache bytes of one K or V tile
constexpr int kNumBars = 16;
template <bool FP8>
constexpr int kSmemTcOf = 1024 + kQBytes + 4 * kStage + (FP8 ? 2 * kRawTile : 0) + kTblCapOf<FP8> * 4 +
                          kNumBars * 8 + 16;
static_assert(kSmemTcOf<true> <= 232448 && kSmemTcOf<false> <= 232448, "shared memory per CTA");
constexpr int kTcThreads = 16 * 32;  // four warpgroups
constexpr int kRegsSoftmax = 200, kRegsOther = 56;

// barrier slots
enum { B_QFULL = 0, B_KFULL = 1, B_VFULL = 3, B_KEMPTY = 5, B_VEMPTY = 7, B_SFULL = 9,
       B_PREADY = 11, B_PVDONE = 13, B_VTAIL = 15 };

// One pass over a row's 128 logits of the current KV tile (thread = row), which the caller
// holds in registers (fetched from TMEM with four loads in flight at once: one latency
// instead of several, which is why the softmax warps raise their register budget):
// probabilities against the reference maximum (mc = m_used*c), the raw row maximum and the
// row sum.  Each 32-column chunk's probabilities are packed to 16-bit pairs and stored to
// TMEM (over the first 64 columns of S, whose values live in registers by now) as soon as
// they exist, so that the stores run under the arithmetic of the next chunk.  MASK and
// CAP are compile-time so the common loop is five instructions per element, no branches.
template <bool CAP, bool MASK, bool F16>
__device__ __forceinline__ void row_pass(uint32_t s_t, const uint32_t (&s0)[32],
                                         const uint32_t (&s1)[32], const uint32_t (&s2)[32],
                                         const uint32_t (&s3)[32], float c, float mc, int lim,
                                         int tok0, float cap_in, float cap_out, float &mx_out,
                                         float &sum_out) {
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
  process32(s2, 64);
  process32(s3, 96);
  mx_out = fmaxf(fmaxf(mxa[0], mxa[1]), fmaxf(mxa[2], mxa[3]));
  sum_out = (sma[0] + sma[1]) + (sma[2] + sma[3]);
}

// F16: format of q and out (and, without FP8, of the pools).  FP8: the pools hold E4M3 bytes.
template <bool CAP, bool F16, bool FP8>
__global__ void __launch_bounds__(kTcThreads, 1)
tile_attention_tc_kernel(const AttnParams p, const TileWork *__restrict__ work,
                         const __grid_constant__ CUtensorMap v_map) {
  constexpr bool MF16 = F16 || FP8;  // operand format of the MMAs
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *gen = smem_raw + (base - smem_u32(smem_raw));
  constexpr int kTblCap = kTblCapOf<FP8>;
  constexpr int kRawBytes = FP8 ? 2 * kRawTile : 0;
  const uint32_t q_s = base, k_s = base + kQBytes, v_s = k_s + 2 * kStage;
  const uint32_t raw_k = v_s + 2 * kStage, raw_v = raw_k + kRawTile;  // FP8 only
  int *tbl = reinterpret_cast<int *>(gen + kQBytes + 4 * kStage + kRawBytes);
  uint64_t *bars =
      reinterpret_cast<uint64_t *>(gen + kQBytes + 4 * kStage + kRawBytes + kTblCap * 4);
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
  // "block" below is a 16-token unit; with 32-token pool blocks (sh = 1) two consecutive
  // units share a table entry and a pool chunk
  const int sh = p.bs_shift;
  for (int i = tid; i < nblk && i < kTblCap; i += kTcThreads) {
    uint32_t id = (uint32_t)table[i >> sh];
    if (id >= p.num_blocks) {
      atomicOr(p.err, kErrBlockRange);
      id = 0;
    }
    tbl[i] = (int)id;
  }
  if (tid == 0) {
    mbar_init(bar(B_QFULL), 128);
    for (int s = 0; s < 2; s++) {
      mbar_init(bar(B_KFULL + s), 128);  // every producer thread, after its pieces landed
      // 16-bit pools: "bytes announced" and "tail of the last block cleared"; FP8: every
      // thread of warps 13-15, after its converted pieces are stored
      mbar_init(bar(B_VFULL + s), FP8 ? 96 : 2);
      mbar_init(bar(B_KEMPTY + s), 1);
      mbar_init(bar(B_VEMPTY + s), 1);
      mbar_init(bar(B_SFULL + s), 1);
      mbar_init(bar(B_PREADY + s), 128);
      mbar_init(bar(B_PVDONE + s), 1);
    }
    mbar_init(bar(B_VTAIL), 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 12) {
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
    uint32_t id = (uint32_t)table[b >> sh];
    if (id >= p.num_blocks) {
      atomicOr(p.err, kErrBlockRange);
      id = 0;
    }
    return id;
  };
  // FP8: exponent field 15 of a cache byte means infinity / NaN; the cheaper conversion
  // serves while the cache is known to hold no such byte
  const bool fp8_exact = FP8 ? *p.fp8_special != 0u : false;

  if (n_tiles > 0) {
    if (warp >= 8 && warp < 12) {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsOther));
      // =========================== producers ========================================
      const int pt = tid - 256;  // 0..127
      const int pw = warp - 8;
      // Q: 2 tiles x 128 rows x 16 pieces of 16 B
      for (int it = 0; it < 32; it++) {
        const int e = it * 128 + pt;
        const int row = e >> 4, c = e & 15;  // row 0..255
        const int tile = row >> 7, r = row & 127;
        const int qi = row / G, g = row - qi * G;
        const bool have = qi < w.q_count;
        const elem16 *src =
            have ? p.q + (int64_t)(q0 + w.q_begin + qi) * p.q_stride + (int64_t)(h * G + g) * kHeadSize + c * 8
                 : p.q;
        const uint32_t dst = q_s + (tile * 2 + (c >> 3)) * kSlab + sw128_off(r, c & 7);
        if (FP8 && !F16) {  // bf16 queries become f16 operands
          uint4 v = make_uint4(0u, 0u, 0u, 0u);
          if (have) v = __ldg(reinterpret_cast<const uint4 *>(src));
          st_shared16(dst, bf16x2_to_f16x2(v.x), bf16x2_to_f16x2(v.y), bf16x2_to_f16x2(v.z),
                      bf16x2_to_f16x2(v.w));
        } else {
          cp_async16(dst, src, have ? 16u : 0u);
        }
      }
      cp_async_commit();
      // K tiles: 16-byte cp.async pieces, every thread its share, published with a proxy
      // fence and one arrival per thread.  A K block is sixteen 256-byte runs that go to
      // sixteen different places (chunk order [d/8][tok][8] -> tile order
      // [d/8][block][tok][8]); as 256-byte bulk copies they measured slower than this.
      auto issue_k = [&](int j) {
        const uint32_t stage = k_s + (j & 1) * kStage;
        for (int bb = 0; bb < 2; bb++) {
          const int b = pw * 2 + bb;           // block within the tile
          const int gb = j * 8 + b;            // block within the sequence
          const bool have = gb < nblk;
          const size_t chunk = have ? (size_t)block_id(gb) * p.Hkv + h : 0;
          // rows of the chunk are (16 << sh) tokens long; the unit starts (gb & sh) * 16 tokens in
          const elem16 *src = p.k_pool + ((chunk * kChunkElems) << sh) + (gb & sh) * 128;
#pragma unroll
          for (int it = 0; it < 8; it++) {
            const int e = it * 32 + lane;  // 16-byte piece of the unit's 4 KB, in memory order
            const int c = e >> 4, t = e & 15;
            cp_async16(stage + c * 2048 + b * 256 + t * 16, src + ((c * 128) << sh) + t * 8,
                       have ? 16u : 0u);
          }
        }
        cp_async_commit();
      };
      // FP8: a K block is 128 pieces of 16 bytes, piece (g, t) = head dimensions 16g..16g+15
      // of token t, which become the two 16-byte pieces (2g, t) and (2g+1, t) of the tile.
      // The bytes of a tile come in by cp.async one tile ahead into a staging area in which
      // every thread owns the pieces it fetched (slot-major, 16 bytes per thread), so that
      // the conversion needs no synchronisation and its loads never wait for memory.
      auto fetch_k_fp8 = [&](int j) {
        for (int bb = 0; bb < 2; bb++) {
          const int b = pw * 2 + bb;
          const int gb = j * 8 + b;
          const bool have = gb < nblk;
          const size_t chunk = have ? (size_t)block_id(gb) * p.Hkv + h : 0;
          const uint8_t *src = reinterpret_cast<const uint8_t *>(p.k_pool) +
                               ((chunk * kChunkElems) << sh) + (gb & sh) * 256;
#pragma unroll
          for (int it = 0; it < 4; it++) {
            const int e = it * 32 + lane, g = e >> 4, t = e & 15;
            cp_async16(raw_k + ((bb * 4 + it) * 128 + pt) * 16, src + ((g * 256) << sh) + t * 16,
                       have ? 16u : 0u);
          }
        }
        cp_async_commit();
      };
      auto convert_k_fp8 = [&](int j, auto exact_tag) {
        constexpr bool EX = decltype(exact_tag)::value;
        const uint32_t stage = k_s + (j & 1) * kStage;
#pragma unroll
        for (int bb = 0; bb < 2; bb++) {
          const int b = pw * 2 + bb;
#pragma unroll
          for (int it = 0; it < 4; it++) {
            const int e = it * 32 + lane, g = e >> 4, t = e & 15;
            const uint4 raw = ld_shared16(raw_k + ((bb * 4 + it) * 128 + pt) * 16);
            uint32_t f[8];
            fp8x4_to_f16<EX>(raw.x, f[0], f[1]);
            fp8x4_to_f16<EX>(raw.y, f[2], f[3]);
            fp8x4_to_f16<EX>(raw.z, f[4], f[5]);
            fp8x4_to_f16<EX>(raw.w, f[6], f[7]);
            const uint32_t dst = stage + (2 * g) * 2048 + b * 256 + t * 16;
            st_shared16(dst, f[0], f[1], f[2], f[3]);
            st_shared16(dst + 2048, f[4], f[5], f[6], f[7]);
          }
        }
      };
      auto land_k = [&](int j) {  // this thread's pieces of K(j) (and of Q before K(0)) are in
        __syncwarp();
        fence_proxy_async();
        if (j == 0) mbar_arrive(bar(B_QFULL));
        mbar_arrive(bar(B_KFULL + (j & 1)));
      };
      // V tiles come in through the copy engine: one tensor-map copy of 4 KB per block (the
      // map's 32-byte swizzle is the layout the MMA reads), eight per tile, completion
      // counted in bytes on the tile's "full" barrier.
      // Tokens past the context inside the last block may hold anything; P is 0 there but
      // 0*NaN is NaN, so that block lands on a barrier of its own and its stray columns are
      // cleared before the tile is published.
      const int last_gb = (kv_len - 1) >> 4;
      const int last_valid = kv_len - last_gb * kBlockSize;
      const bool have_tail = last_valid < kBlockSize && last_gb < nblk;
      const int total_chunks = (int)p.num_blocks * p.Hkv;
      if (FP8) fetch_k_fp8(0);  // the first tile's bytes
      for (int j = 0; j < n_tiles && !failed; j++) {
        const int nb_here = min(8, nblk - j * 8);  // blocks of this tile that exist
        if (j >= 2 && !wait_bar(bar(B_KEMPTY + (j & 1)), ((j >> 1) - 1) & 1, abort_flag)) {
          failed = true;
          break;
        }
        // Published as soon as it has landed (the producers have time to wait here): a
        // tile announced only after the next one could be issued would be held back by the
        // release of that next tile's stage.
        if (FP8) {
          // the bytes of this tile (and the queries) have been on their way for a tile's time;
          // once converted, those of the next tile start
          cp_async_wait<0>();
          if (fp8_exact) convert_k_fp8(j, std::true_type{});
          else convert_k_fp8(j, std::false_type{});
          if (j + 1 < n_tiles) fetch_k_fp8(j + 1);
        } else {
          issue_k(j);
          cp_async_wait<0>();
        }
        land_k(j);
        if (FP8) continue;  // V tiles of an FP8 cache are the work of warps 13-15
        if (j >= 2 && !wait_bar(bar(B_VEMPTY + (j & 1)), ((j >> 1) - 1) & 1, abort_flag)) {
          failed = true;
          break;
        }
        {
          const uint32_t vfull = bar(B_VFULL + (j & 1));
          const int tail_b = (have_tail && (last_gb >> 3) == j) ? (last_gb & 7) : -1;
          if (pt == 0) mbar_expect_tx(vfull, (uint32_t)(tail_b >= 0 ? 7 : 8) * kChunkBytes);
          if (pt < 8) {
            const int b = pt;
            const int chunk = b < nb_here ? (int)block_id(j * 8 + b) * p.Hkv + h : total_chunks;
            const int x0 = (b & sh) * 16;  // j * 8 is even: the unit's half is b's low bit
            const uint32_t dst = v_s + (j & 1) * kStage + b * 4096;
            if (b == tail_b) {
              mbar_expect_tx(bar(B_VTAIL), kChunkBytes);
              tma_load_v_block(dst, &v_map, x0, chunk, bar(B_VTAIL));
            } else {
              tma_load_v_block(dst, &v_map, x0, chunk, vfull);
            }
          }
          if (pw == 1) {  // second arrival: nothing left to clear in this tile
            if (tail_b >= 0) {
              if (!wait_bar(bar(B_VTAIL), 0, abort_flag)) {
                failed = true;
                break;
              }
              uint8_t *vgen = gen + kQBytes + 2 * kStage + (j & 1) * kStage + tail_b * 4096;
              for (int d = lane; d < 128; d += 32)
                for (int t = last_valid; t < kBlockSize; t++)
                  *reinterpret_cast<uint16_t *>(vgen + d * 32 + ((((t >> 3) ^ (d >> 2)) & 1) << 4) +
                                                (t & 7) * 2) = 0;
              fence_proxy_async();
              __syncwarp();
            }
            if (lane == 0) mbar_arrive(vfull);
          }
        }
      }
      if (FP8) cp_async_wait<0>();  // a loop left early may still have bytes on their way
    } else if (warp >= 12) {
      // =========================== MMA issuer ========================================
      asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsOther));
      // The whole warp walks the loop so that descriptors and addresses stay warp-uniform
      // (uniform registers feed tcgen05.mma directly); one elected lane issues.
      if (warp == 12) {
        constexpr uint32_t kIdesc = MF16 ? kIdescF16 : kIdescBf16;
        const bool leader = elect_one();
        auto issue_s = [&](int i, int j) {
          const uint32_t kst = k_s + (j & 1) * kStage;
#pragma unroll
          for (int kk = 0; kk < 8; kk++) {
            const uint32_t koff = (kk >> 2) * kSlab + (kk & 3) * 32;
            if (leader)
              umma_ss(tmem + i * 128, sw128_desc(q_s + i * 2 * kSlab + koff),
                      k_tile_desc(kst + kk * 4096), kIdesc, kk > 0 ? 1u : 0u);
          }
          if (leader) tc_commit(bar(B_SFULL + i));
        };
        auto issue_pv = [&](int i, int j) {
          const uint32_t vst = v_s + (j & 1) * kStage;
#pragma unroll
          for (int kk = 0; kk < 8; kk++) {
            if (leader)
              umma_ts(tmem + 256 + i * 128, tmem + i * 128 + kk * 8, v_block_desc(vst + kk * 4096),
                      kIdesc, (j > 0 || kk > 0) ? 1u : 0u);
          }
          if (leader) tc_commit(bar(B_PVDONE + i));
        };
        do {
          if (!wait_bar(bar(B_QFULL), 0, abort_flag)) { failed = true; break; }
          if (!wait_bar(bar(B_KFULL + 0), 0, abort_flag)) { failed = true; break; }
          tc_fence_after();
          issue_s(0, 0);
          issue_s(1, 0);
          if (leader) tc_commit(bar(B_KEMPTY + 0));
          for (int j = 0; j < n_tiles && !failed; j++) {
            if (!wait_bar(bar(B_VFULL + (j & 1)), (j >> 1) & 1, abort_flag)) { failed = true; break; }
            const bool more = j + 1 < n_tiles;
            if (more && !wait_bar(bar(B_KFULL + ((j + 1) & 1)), ((j + 1) >> 1) & 1, abort_flag)) {
              failed = true;
              break;
            }
            for (int i = 0; i < 2; i++) {
              if (!wait_bar(bar(B_PREADY + i), j & 1, abort_flag)) { failed = true; break; }
              tc_fence_after();
              issue_pv(i, j);
              if (i == 1 && leader) tc_commit(bar(B_VEMPTY + (j & 1)));
              if (more) issue_s(i, j + 1);
            }
            if (more && !failed && leader) tc_commit(bar(B_KEMPTY + ((j + 1) & 1)));
            __syncwarp();
          }
        } while (false);
      } else if (FP8) {
        // ===================== V tiles of an FP8 cache (warps 13-15) ====================
        // A V tile is 1024 pieces of 16 bytes: piece (b, d) = the 16 tokens of head dimension
        // d in block b, which become the two 16-byte halves of row d of that block, placed as
        // the 32-byte swizzle of v_block_desc wants them.  The 96 threads take the pieces
        // round robin; each fetches its pieces by cp.async into slots of its own in the
        // staging area one tile ahead and converts them when the tile's stage is free.
        // Tokens past the context are cleared on the way (0 * NaN is NaN).
        const int vt = tid - 13 * 32;  // 0..95
        auto fetch_v = [&](int j) {
          const int nb_here = min(8, nblk - j * 8);
          for (int i = vt; i < 1024; i += 96) {
            const int b = i >> 7, d = i & 127, gb = j * 8 + b;
            const bool have = b < nb_here;
            const size_t chunk = have ? (size_t)block_id(gb) * p.Hkv + h : 0;
            cp_async16(raw_v + i * 16,
                       reinterpret_cast<const uint8_t *>(p.v_pool) + ((chunk * kChunkElems) << sh) +
                           ((d * 16) << sh) + (gb & sh) * 16,
                       have ? 16u : 0u);
          }
          cp_async_commit();
        };
        auto convert_v = [&](int j, auto exact_tag) {
          constexpr bool EX = decltype(exact_tag)::value;
          // units of this tile that end inside the context need no clearing
          const int full_units = (kv_len >> 4) - j * 8;
          for (int i = vt; i < 1024; i += 96) {
            const int b = i >> 7, d = i & 127;
            uint4 raw = ld_shared16(raw_v + i * 16);
            if (b >= full_units) {
              const int valid = kv_len - (j * 8 + b) * kBlockSize;  // tokens inside the context
              uint32_t wv[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
              for (int wi = 0; wi < 4; wi++) {
                uint32_t m = 0u;
#pragma unroll
                for (int bi = 0; bi < 4; bi++)
                  if (wi * 4 + bi < valid) m |= 0xffu << (8 * bi);
                wv[wi] &= m;
              }
              raw = make_uint4(wv[0], wv[1], wv[2], wv[3]);
            }
            uint32_t f[8];
            fp8x4_to_f16<EX>(raw.x, f[0], f[1]);
            fp8x4_to_f16<EX>(raw.y, f[2], f[3]);
            fp8x4_to_f16<EX>(raw.z, f[4], f[5]);
            fp8x4_to_f16<EX>(raw.w, f[6], f[7]);
            const uint32_t sw = (uint32_t)((d >> 2) & 1) << 4;
            const uint32_t dst = v_s + (j & 1) * kStage + b * 4096 + d * 32;
            st_shared16(dst + sw, f[0], f[1], f[2], f[3]);
            st_shared16(dst + (sw ^ 16u), f[4], f[5], f[6], f[7]);
          }
        };
        fetch_v(0);
        for (int j = 0; j < n_tiles && !failed; j++) {
          if (j >= 2 && !wait_bar(bar(B_VEMPTY + (j & 1)), ((j >> 1) - 1) & 1, abort_flag)) {
            failed = true;
            break;
          }
          cp_async_wait<0>();
          if (fp8_exact) convert_v(j, std::true_type{});
          else convert_v(j, std::false_type{});
          if (j + 1 < n_tiles) fetch_v(j + 1);
          fence_proxy_async();
          mbar_arrive(bar(B_VFULL + (j & 1)));
        }
        cp_async_wait<0>();
      }
    } else {
      // =========================== softmax + epilogue ================================
      asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsSoftmax));
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
      const uint32_t s_t = tmem + lane_base + i * 128;
      const uint32_t o_t = tmem + lane_base + 256 + i * 128;
      // FP8: the converted bytes are value / 2^8; that and the dequantisation factor of the
      // keys ride on the logit scale
      const float qk_scale = FP8 ? p.scale * p.k_scale * kFp8Unbias : p.scale;
      const float c = qk_scale * kLog2e;
      // soft-capping: x -> tanh(x*scale/cap)*cap/scale, so that x*c is the capped logit
      const float cap_in = qk_scale / p.softcap, cap_out = p.softcap / qk_scale;
      float m_used = -INFINITY, l = 0.f;
      uint32_t s0[32], s1[32], s2[32], s3[32];  // the row's logits of the current tile
      auto pass = [&](bool need_mask, int tok0, float &mx, float &sum) {
        const float mc = m_used == -INFINITY ? 0.f : m_used * c;
        if (need_mask)
          row_pass<CAP, true, MF16>(s_t, s0, s1, s2, s3, c, mc, lim, tok0, cap_in, cap_out, mx, sum);
        else
          row_pass<CAP, false, MF16>(s_t, s0, s1, s2, s3, c, mc, lim, tok0, cap_in, cap_out, mx, sum);
      };

      for (int j = 0; j < n_tiles && !failed; j++) {
        if (!wait_bar(bar(B_SFULL + i), j & 1, abort_flag)) { failed = true; break; }
        tc_fence_after();
        const bool need_mask = (j + 1) * kTileTok > warp_min_lim;
        const int tok0 = j * kTileTok;
        float mx, sum;
        tmem_ld32(s_t, s0);
        tmem_ld32(s_t + 32, s1);
        tmem_ld32(s_t + 64, s2);
        tmem_ld32(s_t + 96, s3);
        tmem_wait_ld32(s0);  // waits for all four loads
        tmem_wait_ld32(s1);  // already complete: these tie the registers to the wait
        tmem_wait_ld32(s2);
        tmem_wait_ld32(s3);
        // Optimistic pass against the maximum carried from earlier tiles (for the first
        // tile: against 0, result discarded unless the logits happen to be small).  It
        // already writes P; a second pass, from the same registers, overwrites it.
        pass(need_mask, tok0, mx, sum);
        // stale-maximum rule: move the reference only when it would grow by > 2^8
        const bool grew = mx > m_used && !((mx - m_used) * c <= 8.f);
        if (__any_sync(0xffffffffu, grew)) {
          float factor = 1.f;
          if (grew) {
            factor = m_used == -INFINITY ? 0.f : fast_exp2((m_used - mx) * c);
            m_used = mx;
          }
          if (j > 0) {
            // O_i of the previous tile is complete: its P.V was issued before this S
            if (!wait_bar(bar(B_PVDONE + i), (j - 1) & 1, abort_flag)) { failed = true; break; }
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
          pass(need_mask, tok0, mx, sum);
        }
        l += sum;
        // P (16-bit) now covers the first 64 columns of S
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(bar(B_PREADY + i));
      }
      // epilogue: O / l -> bf16 rows
      if (!failed && wait_bar(bar(B_PVDONE + i), (n_tiles - 1) & 1, abort_flag)) {
        tc_fence_after();
        float inv = l > 0.f ? 1.f / l : 0.f;
        if (FP8) inv *= p.v_scale * kFp8Unbias;
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
  tc_fence_before();
  __syncthreads();
  if (warp == 12) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem));
  }
}

}  // namespace


int tile_queries_per_cta(int G) { return 2 * kQRows / G; }

cudaError_t tile_configure() {
  cudaError_t e = cudaSuccess;
  auto set = [&](auto kernel, int smem) {
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  };
  set(tile_attention_tc_kernel<false, false, false>, kSmemTcOf<false>);
  set(tile_attention_tc_kernel<true, false, false>, kSmemTcOf<false>);
  set(tile_attention_tc_kernel<false, true, false>, kSmemTcOf<false>);
  set(tile_attention_tc_kernel<true, true, false>, kSmemTcOf<false>);
  set(tile_attention_tc_kernel<false, false, true>, kSmemTcOf<true>);
  set(tile_attention_tc_kernel<true, false, true>, kSmemTcOf<true>);
  set(tile_attention_tc_kernel<false, true, true>, kSmemTcOf<true>);
  set(tile_attention_tc_kernel<true, true, true>, kSmemTcOf<true>);
  return e;
}

// Tensor map of one V pool: 16-bit elements, {16 tokens, 128 head dimensions, chunks},
// box = one (block, kv head) chunk, 32-byte swizzle.  The encoder is a driver entry point,
// fetched through the runtime so that the library does not link against the driver.
cudaError_t tile_encode_v_map(TensorMapBlob *out, const void *v_pool, uint64_t num_chunks,
                              int block_size) {
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
  const cuuint64_t dims[3] = {(cuuint64_t)block_size, 128, num_chunks};
  const cuuint64_t strides[2] = {(cuuint64_t)block_size * 2, (cuuint64_t)block_size * 256};
  const cuuint32_t box[3] = {16, 128, 1}, elem_strides[3] = {1, 1, 1};
  const CUresult r = reinterpret_cast<EncodeFn>(fn)(
      reinterpret_cast<CUtensorMap *>(out), CU_TENSOR_MAP_DATA_TYPE_UINT16, 3,
      const_cast<void *>(v_pool), dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
      CU_TENSOR_MAP_SWIZZLE_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

cudaError_t launch_tile_attention(const AttnParams &p, const TileWork *work_dev, int num_work,
                                  const TensorMapBlob *v_map, cudaStream_t st) {
  if (num_work <= 0) return cudaSuccess;
  if (!v_map) return cudaErrorInvalidValue;
  const CUtensorMap &m = *reinterpret_cast<const CUtensorMap *>(v_map);
  const bool cap = p.softcap != 1.0f, f16 = p.is_f16 != 0;
  const int smem = p.is_fp8 ? kSmemTcOf<true> : kSmemTcOf<false>;
  auto go = [&](auto kernel) { kernel<<<num_work, kTcThreads, smem, st>>>(p, work_dev, m); };
  if (p.is_fp8) {
    if (cap && f16) go(tile_attention_tc_kernel<true, true, true>);
    else if (cap) go(tile_attention_tc_kernel<true, false, true>);
    else if (f16) go(tile_attention_tc_kernel<false, true, true>);
    else go(tile_attention_tc_kernel<false, false, true>);
  } else {
    if (cap && f16) go(tile_attention_tc_kernel<true, true, false>);
    else if (cap) go(tile_attention_tc_kernel<true, false, false>);
    else if (f16) go(tile_attention_tc_kernel<false, true, false>);
    else go(tile_attention_tc_kernel<false, false, false>);
  }
  __atomic_fetch_add(&g_launch_count, 1ull, __ATOMIC_RELAXED);
  return cudaGetLastError();
}

}  // namespace pa
