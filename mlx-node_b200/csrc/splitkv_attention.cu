// Split-KV ("flash-decoding") paged attention for sm_100a: the memory-bound
// kernel for decode and short multi-token (speculative-verify) sequences.
//
// Replaces the per-(sequence, query head, 512-token partition) kernel and its
// reduce pass, crates/mlx-paged-attn/metal/attention/paged_attention.metal
// :760-1147 and :1149-1260, which stream the KV blocks once per QUERY head.
// Here one read of a (block, kv head) chunk serves every query head of the GQA
// group and every query token of the sequence.
//
// Work decomposition.  A unit is one (sequence, kv head, 16-token block): a 4 KB
// K chunk plus a 4 KB V chunk, each contiguous in the pool.  Units are numbered
// item-major (item = sequence*Hkv + kv head, then block index) and the flat range
// [0, W) is cut into gridDim.x pieces of equal COST, one persistent CTA per SM each:
// cost = units + item_cost per item start (starting an item costs a CTA about 4 us of
// query loads, warp combine, partial store and merge during which its ring idles), so
// that a CTA whose range holds many short sequences gets fewer units and all CTAs
// finish together.  The boundaries of all pieces are computed once per CTA into shared
// memory (bnd[]); which CTAs hold pieces of an item is read from that table.  A CTA
// walks the items its piece overlaps ("segments").  A segment that covers its whole item writes
// the final bf16 rows; a segment that starts or ends inside an item writes an
// unnormalised partial (running max, sum, accumulator) to one of the CTA's two
// workspace slots and counts itself on the item's arrival counter; the CTA that
// arrives last combines the item's partials, always in CTA order, so the result
// does not depend on who was last (deterministic).  There is no second kernel:
// this replaces the reduce pass paged_attention.metal:1149-1260 as the tail of
// the attention launch itself.
//
// Decode step in one launch (p.k_new set; 16-bit pools of 16-token blocks): the warp
// that attends the last block of a (sequence, kv head) also stores the step's new
// token of that head, from the caller's [S, Hkv, 128] rows, into its pool slot and
// into the copy of the block it has just staged in shared memory, so that the
// KV write of crates/mlx-core/src/transformer/block.rs:223-232 needs no launch
// of its own and attention sees the token it must see.
//
// Data movement.  Each warp owns a ring of NST stages of 8 KB.  Lane 0 issues two
// 4 KB bulk async copies (TMA, untiled, this CTA only) per unit, completion
// counted on the stage's mbarrier; the warp consumes its own stages, so no
// cross-warp hand-off sits on the critical path.  8 warps x NST stages x 8 KB
// of loads are in flight per SM.  Block ids for the next 32 units of a warp are
// looked up one batch ahead, one unit per lane, and handed to lane 0 by shuffle.
//
// Arithmetic.  Tensor cores through mma.sync m16n8k16 (bf16 in, fp32 out), in the
// transposed form so that the 16 tokens of a block are the M dimension:
//   S^T[16 tok x 8 col] = K[16 tok x 128] . Q^T[128 x 8 col]
//   O^T[128 x 8 col]   += V^T[128 x 16 tok] . P^T[16 tok x 8 col]
// A column is a (query token, query head of the group) pair.  The reference K
// layout [D/8][BS][8] is exactly the 8x(16 B) core-matrix order ldmatrix wants
// for K as the A operand, and V's [D][BS] is A-operand order for V^T, so both
// tiles are consumed straight from the raw 4 KB chunks.  P^T is produced from the
// S^T accumulators with one movmatrix transpose per 8x8 tile.  Online softmax in
// fp32 with exp2; column maxima by warp shuffles.  Where the ring has three stages the
// loop over a warp's units is software-pipelined: the logits of the next unit are
// computed next to the softmax and P.V of the current one, so that the two dependency
// chains (ldmatrix -> MMA chain, and max -> exp2 -> movmatrix -> MMA) overlap.
//
// 32-token pool blocks (p.bs_shift = 1).  16-bit pools (template flag B32): a unit is a
// whole block, one contiguous 8 KB bulk copy per operand into a 16 KB stage (one stage per
// warp), and the warp takes the block's two 16-token halves one after the other from it;
// the halves interleave row by row in the chunk, which is an ldmatrix address term.  FP8
// pools: the unit stays 16 tokens and comes in through two tensor-map copies (a [D/16] x
// 256 B box of the K chunk, a [D] x 16 B box of the V chunk) that land in the ring stage
// in exactly the layout of a 16-token chunk; everything after the copy is the same code.
//
// 8-token pool blocks (p.bs_shift = -1, template flag B8; 16-bit pools): a unit is two pool
// blocks with ids of their own, four 2 KB bulk copies into the stage (K of the first block,
// K of the second, V of the first, V of the second), and the ldmatrix addresses take the
// token half from the 2 KB sub-chunk instead of from the row.  Block ids are looked up 16
// units at a time, lane 2i and 2i+1 holding the two blocks of unit i; a last unit of eight
// tokens or fewer has no second block and copies half the bytes.
//
// Head sizes other than 128 (template parameter HD, 16-bit pools of 16-token blocks): chunks
// of 32 * HD bytes, ceil(HD / 16) steps of the head dimension and as many row tiles of O^T
// (120 runs with its last step half empty); up to head size 80 the narrow kernel runs two
// CTAs per SM, from 192 on the ring is one stage per warp.
//
// Several launches of one call may run at the same time, one per width class of a mixed
// batch ("lanes"): each keeps its partial slots and arrival counters from cta_base on.
//
// FP8 (E4M3) pools: the same kernel on 2 KB chunks.  K.Q^T runs on the FP8 tensor-core
// path straight from the cache bytes (queries split into two E4M3 numbers) unless the
// cache may hold bytes that the tensor cores read differently from the cache format; then,
// and always for V^T.P^T, the bytes become f16 by integer operations; see the comments at
// fp8x4_to_f16 and in the main loop.
#include <cuda.h>

#include <cstring>
#include <mutex>
#include <type_traits>

#include "pa_common.cuh"

namespace pa {

namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kMaxSeqsPerLaunch = 2048;
constexpr int kMaxNT = 3;  // up to 24 columns per item

// FP8: an E4M3 cache, one byte per element; a unit is a 2 KB K chunk laid out
// [D/16][BS][16] plus a 2 KB V chunk [D][BS], and the ring holds twice as many stages.
constexpr int kTwoCtaMaxHead = 80;  // largest head size whose narrow kernel runs two CTAs per SM
// SUB: 16-token sub-units a warp takes from one stage (2 = a whole 32-token pool block).
template <int NT, bool FP8 = false, int HD = kHeadSize, int SUB = 1>
struct Cfg {
  // (a head size that is a multiple of 8 only - 120 - runs with its last 16-wide step half
  // empty: the missing eight dimensions are zeros in Q and in the K fragments and are never stored)
  static_assert(HD % 8 == 0 && HD >= 32 && HD <= 256, "head sizes built: multiples of 8 from 32 to 256");
  static_assert(SUB == 1 || (SUB == 2 && HD <= kHeadSize && !FP8),
                "whole 32-token blocks: 16-bit pools, head sizes up to 128 (a stage is 64 * HD bytes)");
  static constexpr int kSteps = (HD + 15) / 16;  // 16-wide steps of the head dimension (K.Q^T) = 16-row tiles of O^T
  static constexpr int kChunk = (FP8 ? kChunkBytes / 2 : kChunkBytes) * HD / kHeadSize * SUB;  // bytes of one K or V chunk
  static constexpr int kStageBytes = 2 * kChunk;
  // The narrow FP8 variant runs two CTAs per SM (its per-unit work is latency-bound, so
  // it wants 16 warps per SM; 128 registers per thread allow it): two 4 KB stages per
  // warp there, otherwise the ring keeps its byte size and holds twice as many stages.
  // The narrow kernel on head sizes up to 80 shares an SM as well: a unit is 5 KB or less, so
  // the per-unit latency chain weighs as in the FP8 case (measured on configuration 2 / 3
  // shapes: head 64 0.84 / 0.87 of the HBM peak with one CTA per SM, 0.94 / 0.99 with two;
  // head 32 0.48 -> 0.72 / 0.80).  From 96 on, two CTAs' rings no longer fit an SM.
  static constexpr int kCtasPerSm = (NT == 1 && SUB == 1 && (FP8 || HD <= kTwoCtaMaxHead)) ? 2 : 1;
  // Head sizes up to 64 halve the stage (or more), so the ring holds twice as many; head
  // sizes from 192 and whole 32-token blocks make it 12 or 16 KB and the 227 KB of an SM
  // hold one stage per warp (the eight warps then overlap each other's copies instead of
  // each its own).
  static constexpr int kStages = (HD >= 192 || SUB == 2) ? 1
                                 : kCtasPerSm == 2 ? (HD <= 32 ? 4 : 2)
                                                   : (NT == 1 ? 3 : 2) * (FP8 ? 2 : 1) * (HD <= 64 ? 2 : 1);
  static constexpr int kAcc = 4 * kSteps;      // O^T accumulators per thread and column tile
  static constexpr int kRegs = (kAcc + 4) * NT;  // per thread: accumulators, 2NT maxima, 2NT sums
  static constexpr int kRingBytes = kWarps * kStages * kStageBytes;
  static constexpr int kMergeBytes = (kWarps / 2) * kRegs * 32 * 4;
  static constexpr int kPreBytes = (kMaxSeqsPerLaunch + 1) * 4;
  static constexpr int kBarBytes = kWarps * kStages * 8;
  static constexpr int kBndOffset = (kRingBytes + kMergeBytes + kPreBytes + 12 + kBarBytes + 15) / 16 * 16;
  static constexpr int kBndBytes = (kMaxSplitCtas + 1) * 8;         // first unit of every CTA
  static constexpr int kCntBytes = (kMaxSeqsPerLaunch + 2) / 2 * 4;  // eligible sequences before each
  static constexpr int kSmemBytes = kBndOffset + kBndBytes + kCntBytes;
};
// What a CTA pays for every item it starts (queries fetched, eight warps combined, a
// partial stored, possibly a merge), in units of streaming: measured at about 4 us
// against 0.16 us per 8 KB unit.  The partition charges it, so that a CTA whose range
// holds many short sequences gets fewer units and all CTAs finish together.
constexpr int kItemCostUnits = 24;
constexpr int kItemCostUnitsFp8 = 16;
constexpr int kSlotFloats = 36 * kMaxNT * 32;  // one workspace slot, sized for the widest kernel
static_assert(Cfg<1, false, 256>::kRegs * 32 <= kSlotFloats && Cfg<2, false, 192>::kRegs * 32 <= kSlotFloats &&
                  Cfg<3, false, 112>::kRegs * 32 <= kSlotFloats,
              "a partial of every kernel variant fits a workspace slot");

__device__ __forceinline__ int q_len_of(const AttnParams &p, int seq) {
  return p.cu_q_lens ? p.cu_q_lens[seq + 1] - p.cu_q_lens[seq] : 1;
}
// Blocks of a sequence this kernel family handles (0 if the sequence belongs to
// the tile kernel or has nothing to attend).
__device__ __forceinline__ int eligible_blocks(const AttnParams &p, int seq, int unit_tokens = kBlockSize) {
  const int ql = q_len_of(p, seq);
  if (ql < 1 || ql * p.G > p.max_cols || ql * p.G < p.min_cols) return 0;
  const int ctx = p.context_lens[seq];
  return ctx > 0 ? (ctx + unit_tokens - 1) / unit_tokens : 0;
}

// D(16x8,f32) += A(16x32,row) * B(32x8,col), both operands E4M3 bytes.  The tensor cores
// read exponent field 15 as finite values (the OCP variant of the format); every other
// byte means the same as in the cache format, so this path serves the fast variant only.
__device__ __forceinline__ void mma_fp8_16832(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                              uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// Four floats -> four E4M3 bytes (x0 in the low byte), round to nearest, saturating.
__device__ __forceinline__ uint32_t pack_e4m3x4(float x0, float x1, float x2, float x3) {
  uint16_t lo, hi;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(x1), "f"(x0));
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(x3), "f"(x2));
  return (uint32_t)lo | ((uint32_t)hi << 16);
}
__device__ __forceinline__ float f16lo_to_float(uint32_t h2) {
  float f;
  asm("cvt.f32.f16 %0, %1;" : "=f"(f) : "h"((uint16_t)(h2 & 0xffffu)));
  return f;
}
__device__ __forceinline__ float f16hi_to_float(uint32_t h2) {
  float f;
  asm("cvt.f32.f16 %0, %1;" : "=f"(f) : "h"((uint16_t)(h2 >> 16)));
  return f;
}
// FP8 path: row r of a 16-token MMA tile holds token fp8_row_token(r) of the block, so
// that the token pairs a thread gets from one 32-bit piece of a V row (tokens 4t..4t+3)
// are the pairs its P^T fragment holds.
__device__ __forceinline__ int fp8_row_token(int r) {
  return 4 * ((r & 7) >> 1) + 2 * (r >> 3) + (r & 1);
}

// The K and V maps of encode_unit_maps as the kernel parameter they have to be.
struct KvMaps {
  CUtensorMap k, v;
};
// One unit through a tensor map {x: elements of a chunk row, y: row, z: chunk}; x0 picks
// the unit within the row (a multiple of 16 bytes).  This CTA's shared memory only.
__device__ __forceinline__ void tma_load_unit(uint32_t dst, const CUtensorMap *map, int x0, int chunk,
                                              uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x0), "r"(0), "r"(chunk), "r"(bar)
      : "memory");
}

// Combines the partials of one split item, (sequence, kv head), whose pieces lie in
// CTAs [c_first, c_last], and writes the item's final rows.  Called by all threads
// of the CTA that arrived last; reads go to L2 (the other CTAs wrote these slots).
// Thread layout: d = tid mod HD (head dimension); a thread takes every (256 / HD)-th
// column, four of them per pass, and issues all loads of a pass before it uses any (one
// round trip to L2 per pass instead of one per column).
template <int NT, bool F16, int HD>
__device__ __forceinline__ void merge_item(const AttnParams &p, const long long *bnd, int c_first,
                                           int c_last, int q0, int h, int ncols, int tid) {
  constexpr int CP = 4;  // columns per pass and thread
  constexpr int PP = 4;  // pieces per pass
  constexpr int CS = kThreads / HD;  // column stride of a thread
  constexpr int kAcc = 4 * ((HD + 15) / 16);
  if (tid >= CS * HD) return;        // head sizes that do not divide the block leave some threads out
  const int d = tid % HD;
  const int mt = d >> 4, gid = d & 7, upper = (d >> 3) & 1;
  for (int col0 = tid / HD; col0 < ncols; col0 += CS * CP) {
    float mm[CP], acc[CP], lsum[CP];
#pragma unroll
    for (int i = 0; i < CP; i++) { mm[i] = -INFINITY; acc[i] = 0.f; lsum[i] = 0.f; }
    // partials in CTA order
    for (int c0 = c_first; c0 <= c_last; c0 += PP) {
      float mj[CP][PP], oj[CP][PP], lj[CP][PP];
#pragma unroll
      for (int k = 0; k < PP; k++) {
        const int c = c0 + k;
        // CTAs between c_first and c_last may own nothing
        const bool piece = c <= c_last && bnd[c + 1] > bnd[c];
        const float *slot = p.ws + (size_t)(2 * (p.cta_base + c) + (c == c_first ? 1 : 0)) * kSlotFloats;
#pragma unroll
        for (int i = 0; i < CP; i++) {
          const int col = col0 + CS * i;
          const bool use = piece && col < ncols;
          const int nt = col >> 3, tig = (col & 7) >> 1, par = col & 1;
          const int lane = gid * 4 + tig;
          mj[i][k] = use ? __ldcg(slot + (kAcc * NT + nt * 2 + par) * 32 + lane) : -INFINITY;
          oj[i][k] = use ? __ldcg(slot + ((mt * NT + nt) * 4 + upper * 2 + par) * 32 + lane) : 0.f;
          lj[i][k] = use ? __ldcg(slot + ((kAcc + 2) * NT + nt * 2 + par) * 32 + lane) : 0.f;
        }
      }
#pragma unroll
      for (int i = 0; i < CP; i++) {
        const float m_new = fmaxf(fmaxf(fmaxf(mj[i][0], mj[i][1]), fmaxf(mj[i][2], mj[i][3])), mm[i]);
        const float keep = mm[i] == -INFINITY ? 0.f : exp2f(mm[i] - m_new);
        acc[i] *= keep;
        lsum[i] *= keep;
#pragma unroll
        for (int k = 0; k < PP; k++) {
          const float w = mj[i][k] == -INFINITY ? 0.f : exp2f(mj[i][k] - m_new);
          acc[i] += oj[i][k] * w;
          lsum[i] += lj[i][k] * w;
        }
        mm[i] = m_new;
      }
    }
#pragma unroll
    for (int i = 0; i < CP; i++) {
      const int col = col0 + CS * i;
      if (col < ncols) {
        const int qj = col / p.G, g = col - qj * p.G;
        p.out[(int64_t)(q0 + qj) * p.out_stride + (int64_t)(h * p.G + g) * HD + d] =
            to_elem<F16>(lsum[i] > 0.f ? acc[i] / lsum[i] : 0.f);
      }
    }
  }
}

constexpr uint32_t kNoBlock = 0xffffffffu;  // B8: the unit has no second pool block

// FUSE: the variant that also writes the step's new tokens (p.k_new).  It is an
// instantiation of its own because the mere presence of that code cost the plain
// kernel 1.5 % (measured), and it exists for the narrow 16-bit kernel only.
// B32: pools of 32-token blocks, 16-bit, head size 128: a unit is a whole block, fetched as one
// contiguous 8 KB copy per operand, and the warp takes its two 16-token halves one after the
// other from the same stage (the interleave of the halves is an ldmatrix address term).
template <int NT, bool F16, bool FP8, bool B8 = false, bool FUSE = false, int HD = kHeadSize, bool B32 = false>
__global__ void __launch_bounds__(kThreads, Cfg<NT, FP8, HD, B32 ? 2 : 1>::kCtasPerSm)
splitkv_kernel(const AttnParams p, const __grid_constant__ KvMaps maps) {
  static_assert(!(FP8 && B8), "8-token blocks exist for 16-bit pools only");
  static_assert(!FUSE || (NT == 1 && !FP8 && !B8), "the fused write exists for the narrow 16-bit kernel");
  static_assert(HD == kHeadSize || (!FP8 && !B8 && !FUSE), "other head sizes: 16-bit pools, 16- or 32-token blocks");
  static_assert(!B32 || (!FP8 && !B8 && !FUSE && HD <= kHeadSize), "whole 32-token blocks: 16-bit pools, head sizes up to 128");
  constexpr int SUB = B32 ? 2 : 1;       // 16-token sub-units per unit
  using C = Cfg<NT, FP8, HD, SUB>;
  constexpr int KS = C::kSteps;          // 16-wide steps of the head dimension / 16-row tiles of O^T
  constexpr int KSA = KS < 8 ? 8 : KS;   // array extent (the FP8 code, head size 128 only, indexes 8)
  constexpr int kAcc = C::kAcc;
  constexpr int NST = C::kStages;
  constexpr int kStageBytes = C::kStageBytes;
  constexpr int kChunk = C::kChunk;
  constexpr bool MF16 = F16 || FP8;  // operand type of the MMAs
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t *ring = smem;
  float *merge_buf = reinterpret_cast<float *>(smem + C::kRingBytes);
  int *pre = reinterpret_cast<int *>(smem + C::kRingBytes + C::kMergeBytes);
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + C::kRingBytes + C::kMergeBytes +
                                                ((C::kPreBytes + 15) / 16) * 16);
  long long *bnd = reinterpret_cast<long long *>(smem + C::kBndOffset);
  uint16_t *cnt = reinterpret_cast<uint16_t *>(smem + C::kBndOffset + C::kBndBytes);

  __shared__ int s_last;  // this CTA arrived last at a split item and combines it

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gid = lane >> 2, tig = lane & 3;
  const int mi = lane >> 3, mr = lane & 7;  // ldmatrix: matrix index, row within it
  const int S = p.S, Hkv = p.Hkv, G = p.G;

  // The next kernel of the stream may be scheduled now (it orders itself with its own
  // griddepcontrol.wait).  Its CTAs then sit on the SMs until this grid ends, holding
  // registers, so the early trigger is skipped when another kernel is meant to use
  // the SMs this grid leaves free.
  if (p.early_trigger) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // ---- per-launch prefix sum of block counts --------------------------------
  for (int s = tid; s < S; s += kThreads) pre[s + 1] = eligible_blocks(p, p.seq_base + s, kBlockSize * SUB);
  if (tid == 0) pre[0] = 0;
  if (lane == 0) {
    for (int st = 0; st < NST; st++) mbar_init(smem_u32(&bars[warp * NST + st]), 1);
    mbar_fence_init();
  }
  __syncthreads();
  if (warp == 0) {
    int running = 0, running_n = 0;
    if (lane == 0) cnt[0] = 0;
    for (int base = 0; base < S; base += 32) {
      int v = (base + lane < S) ? pre[base + lane + 1] : 0;
      const unsigned have = __ballot_sync(0xffffffffu, v > 0);
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += n;
      }
      if (base + lane < S) {
        pre[base + lane + 1] = running + v;
        cnt[base + lane + 1] = (uint16_t)(running_n + __popc(have & (0xffffffffu >> (31 - lane))));
      }
      running += __shfl_sync(0xffffffffu, v, 31);
      running_n += __popc(have);
    }
  }
  __syncthreads();

  // ---- the partition: bnd[c] = first unit of CTA c ------------------------------
  // Equal shares of units + item_cost per item: in that weighted order an item is
  // item_cost slots of padding followed by its units, CTA c starts at share c of the
  // weighted total, and a start inside the padding moves to the item's first unit.
  const long long W = (long long)Hkv * pre[S];
  {
    const int K = p.item_cost;
    const long long Wt = W + (long long)Hkv * K * cnt[S];
    for (int c = tid; c <= (int)gridDim.x; c += kThreads) {
      long long f;
      if (c == (int)gridDim.x) {
        f = W;
      } else if (K <= 0) {
        f = (long long)c * W / gridDim.x;
      } else {
        const long long t = (long long)c * Wt / gridDim.x;
        int a = 0, b = S - 1;  // smallest s whose weighted range ends beyond t
        while (a < b) {
          const int mid = (a + b) >> 1;
          if ((long long)Hkv * (pre[mid + 1] + (long long)K * cnt[mid + 1]) > t) b = mid; else a = mid + 1;
        }
        const int nb_a = pre[a + 1] - pre[a];
        const long long r = t - (long long)Hkv * (pre[a] + (long long)K * cnt[a]);
        const long long hh = r / (nb_a + K), off = r - hh * (nb_a + K);
        f = (long long)Hkv * pre[a] + hh * nb_a + (off > K ? off - K : 0);
      }
      bnd[c] = f;
    }
  }
  __syncthreads();
  const long long lo = bnd[blockIdx.x];
  const long long hi = bnd[blockIdx.x + 1];
  // the CTA whose range holds unit u
  auto cta_of = [&](long long u) {
    int a = 0, b = (int)gridDim.x - 1;
    while (a < b) {
      const int mid = (a + b + 1) >> 1;
      if (bnd[mid] <= u) a = mid; else b = mid - 1;
    }
    return a;
  };
  const int n_local = (int)(hi - lo);
  const int n_w = n_local > warp ? (n_local - warp + kWarps - 1) / kWarps : 0;

  // smallest s with Hkv*pre[s+1] > u
  auto seq_of = [&](long long u) {
    int a = 0, b = S - 1;
    while (a < b) {
      const int mid = (a + b) >> 1;
      if ((long long)Hkv * pre[mid + 1] > u) b = mid; else a = mid + 1;
    }
    return a;
  };
  // Pool chunk index (block id * Hkv + kv head) of this warp's j-th unit; with 32-token
  // blocks, twice that plus the unit's place in the chunk.
  // B8: the argument is 2 * j + (0: first, 1: second pool block of the unit).
  // In two halves, so that the table reads of several look-ups can be in flight together:
  // locate() finds the table entry, resolve() turns what was read there into the chunk.
  struct Loc {
    const int32_t *entry;  // null: no table entry to read (see `fixed`)
    uint32_t fixed;        // the result then: 0 (no such unit) or kNoBlock
    int h, b;
  };
  auto locate = [&](int jj) -> Loc {
    const int j = B8 ? jj >> 1 : jj;
    if (j >= n_w) return Loc{nullptr, 0u, 0, 0};
    const long long u = lo + warp + (long long)kWarps * j;
    const int s = seq_of(u);
    const int r = (int)(u - (long long)Hkv * pre[s]);
    const int nb = pre[s + 1] - pre[s];
    const int h = r / nb, b = r - h * nb;
    const int row = p.seq_row ? p.seq_row[p.seq_base + s] : p.seq_base + s;
    int col;  // block-table column
    if (B8) {
      col = 2 * b + (jj & 1);
      if (col * 8 >= p.context_lens[p.seq_base + s]) return Loc{nullptr, kNoBlock, h, b};
    } else {
      col = B32 ? b : b >> p.bs_shift;
    }
    return Loc{p.block_tables + (long long)row * p.MB + col, 0u, h, b};
  };
  auto resolve = [&](const Loc &at, int32_t raw) -> uint32_t {
    if (!at.entry) return at.fixed;
    uint32_t id = (uint32_t)raw;
    if (id >= p.num_blocks) {
      atomicOr(p.err, kErrBlockRange);
      id = 0;
    }
    const uint32_t chunk = id * (uint32_t)Hkv + (uint32_t)at.h;
    return (!B8 && !B32 && p.bs_shift) ? 2u * chunk + (uint32_t)(at.b & 1) : chunk;
  };
  auto lookup = [&](int jj) -> uint32_t {
    const Loc at = locate(jj);
    return resolve(at, at.entry ? *at.entry : 0);
  };
  // The first two batches of look-ups, both reads in flight together.  Like the context
  // lengths above, the block tables are read before the wait below.
  uint32_t first_ids, second_ids;
  {
    const Loc a0 = locate(lane), a1 = locate(32 + lane);
    const int32_t r0 = a0.entry ? *a0.entry : 0;
    const int32_t r1 = a1.entry ? *a1.entry : 0;
    first_ids = resolve(a0, r0);
    second_ids = resolve(a1, r1);
  }

  // This grid may have started while the KV write before it was still running: the
  // pool (and the workspace and output rows a previous call may still be reading or
  // writing) must not be touched before the predecessor has completed.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  // Sequences of this launch's width class with nothing to attend get zero rows
  // (crates/mlx-sys/src/mlx.cpp:4084-4088).
  for (int s2 = blockIdx.x; s2 < S; s2 += gridDim.x) {
    if (pre[s2 + 1] != pre[s2]) continue;
    const int seq = p.seq_base + s2;
    const int ql = q_len_of(p, seq);
    if (ql < 1 || ql * G > p.max_cols || ql * G < p.min_cols) continue;
    const int q0 = p.cu_q_lens ? p.cu_q_lens[seq] : seq;
    const int row_elems = p.Hq * HD;
    for (int e = tid; e < ql * row_elems; e += kThreads)
      p.out[(int64_t)(q0 + e / row_elems) * p.out_stride + e % row_elems] = (elem16)0;
  }
  // FP8: one pass of the main loop is compiled per decoding variant; which one runs is
  // decided by a device word the cache write sets when it produces an exponent-15 byte.
  auto main_loop = [&](auto exact_tag) {
    constexpr bool EXACT = decltype(exact_tag)::value;
  const uint32_t ring_w = smem_u32(ring) + warp * NST * kStageBytes;
  const uint32_t bar_w = smem_u32(&bars[warp * NST]);
  uint32_t cur_ids = first_ids, nxt_ids = second_ids;
  int ji = 0;  // units issued by this warp
  constexpr int kBatch = B8 ? 16 : 32;  // units per lookup
  // A launch that reads more than L2 holds reads every chunk once: its lines are marked
  // "evict first", so that they do not push out what is reused - the queries and partials
  // of this grid and, in a mixed batch, the KV tiles the tile kernel's CTAs share.  A
  // small batch (everything fits in L2) keeps the default: the next layer's or step's
  // call may find its blocks still there.
  const bool stream_once = W * (long long)kStageBytes > (96ll << 20);
  const uint64_t evict_first = l2_evict_first();
  auto issue = [&]() {  // whole warp calls; lane 0 issues unit ji
    if ((ji & (kBatch - 1)) == 0 && ji > 0) {
      cur_ids = nxt_ids;
      nxt_ids = lookup((B8 ? 2 : 1) * (ji + kBatch) + lane);
    }
    const uint32_t chunk = __shfl_sync(0xffffffffu, cur_ids, B8 ? 2 * (ji & 15) : ji & 31);
    uint32_t chunk_b = 0u;
    if (B8) chunk_b = __shfl_sync(0xffffffffu, cur_ids, 2 * (ji & 15) + 1);
    if (lane == 0) {
      const int st = ji % NST;
      const uint32_t bar = bar_w + st * 8, dst = ring_w + st * kStageBytes;
      if (B8) {
        // stage: K of the first block | K of the second | V of the first | V of the second
        const uint8_t *kp = reinterpret_cast<const uint8_t *>(p.k_pool);
        const uint8_t *vp = reinterpret_cast<const uint8_t *>(p.v_pool);
        const bool two = chunk_b != kNoBlock;
        mbar_expect_tx(bar, two ? kStageBytes : kStageBytes / 2);
        bulk_g2s(dst, kp + (size_t)chunk * (kChunk / 2), kChunk / 2, bar);
        bulk_g2s(dst + kChunk, vp + (size_t)chunk * (kChunk / 2), kChunk / 2, bar);
        if (two) {
          bulk_g2s(dst + kChunk / 2, kp + (size_t)chunk_b * (kChunk / 2), kChunk / 2, bar);
          bulk_g2s(dst + kChunk + kChunk / 2, vp + (size_t)chunk_b * (kChunk / 2), kChunk / 2, bar);
        }
      } else if (!B32 && p.bs_shift) {
        // elements of a K row per unit: 16 tokens x 8 (16-bit) or x 16 (bytes); of a V row: 16
        const int unit = (int)(chunk & 1u), ch = (int)(chunk >> 1);
        mbar_expect_tx(bar, kStageBytes);
        tma_load_unit(dst, &maps.k, unit * (FP8 ? 256 : 128), ch, bar);
        tma_load_unit(dst + kChunk, &maps.v, unit * 16, ch, bar);
      } else if (stream_once) {
        mbar_expect_tx(bar, kStageBytes);
        bulk_g2s_hint(dst, reinterpret_cast<const uint8_t *>(p.k_pool) + (size_t)chunk * kChunk,
                      kChunk, bar, evict_first);
        bulk_g2s_hint(dst + kChunk, reinterpret_cast<const uint8_t *>(p.v_pool) + (size_t)chunk * kChunk,
                      kChunk, bar, evict_first);
      } else {
        mbar_expect_tx(bar, kStageBytes);
        bulk_g2s(dst, reinterpret_cast<const uint8_t *>(p.k_pool) + (size_t)chunk * kChunk, kChunk,
                 bar);
        bulk_g2s(dst + kChunk, reinterpret_cast<const uint8_t *>(p.v_pool) + (size_t)chunk * kChunk,
                 kChunk, bar);
      }
    }
    ji++;
  };
  // 16-bit pools: the first copies are issued inside the first segment below, right
  // behind its query loads (see there); FP8 converts its queries as they arrive, so
  // there the copies go first.
  if constexpr (FP8)
    for (int j = 0; j < NST && j < n_w; j++) issue();

  int jc = 0;          // units consumed by this warp
  bool dead = false;   // a wait ran out: stop touching data, keep the barriers balanced
  // k_scale: FP8 dequantisation (with the conversion's missing 2^8), else 1
  const float qk_scale = p.scale * p.k_scale * (FP8 ? kFp8Unbias : 1.f);
  const float v_unscale = p.v_scale * (FP8 ? kFp8Unbias : 1.f);
  const float sc_log2 = qk_scale * kLog2e;
  const bool use_cap = p.softcap != 1.0f;

  constexpr bool kCanFuseWrite = FUSE;
  const bool fuse_write = kCanFuseWrite && p.k_new != nullptr;

  // ---- walk the segments of [lo, hi) -----------------------------------------
  int s = seq_of(lo);
  int nb = pre[s + 1] - pre[s];
  int h, b0;
  {
    const int r = (int)(lo - (long long)Hkv * pre[s]);
    h = r / nb;
    b0 = r - h * nb;
  }
  int a = 0;  // CTA-local unit index of the segment start
  while (a < n_local) {
    const int seglen = min(nb - b0, n_local - a);
    const int b1 = b0 + seglen;
    const int seq = p.seq_base + s;
    const int kv_len = p.context_lens[seq];
    const int q0 = p.cu_q_lens ? p.cu_q_lens[seq] : seq;
    const int q_len = q_len_of(p, seq);
    const int ncols = q_len * G;

    // Q^T B-fragments: column nt*8+gid, k = 16j + 2tig (+8).
    // FP8 fast variant: S = K.Q^T runs on the FP8 tensor-core path straight from the
    // cache bytes.  The query row is scaled by a power of two (largest element into
    // [64, 128)) and split into two E4M3 numbers per element, hi = rn(q') and
    // lo = rn(q' - hi), which together carry eight significant bits (all of a bf16 query);
    // qf[.][0..3] hold hi and qf[.][4..7] lo of the four 32-wide steps, and the power of
    // two comes back out in the column's logit scale.
    constexpr bool QK8 = FP8 && !EXACT;
    uint32_t qf[NT][KSA][2];
    int lim[NT][2];  // keys visible to columns nt*8 + 2tig + {0,1}
    float col_lin[NT][2];  // S accumulator -> logit, for columns nt*8 + 2tig + {0,1}
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
      const int col = nt * 8 + gid;
      int q_exp = 0;  // QK8: the row was multiplied by 2^q_exp
      if (QK8) {
        // step s: b0 carries d = 32s + 4tig .. +3, b1 carries d = 32s + 16 + 4tig .. +3.
        // Every lane runs this block (columns beyond the item carry zeros): the shuffles
        // below need the whole warp.
        const bool have_col = col < ncols;
        const int qj = have_col ? col / G : 0, g = have_col ? col - qj * G : 0;
        const uint32_t *qp = reinterpret_cast<const uint32_t *>(
            p.q + (int64_t)(q0 + qj) * p.q_stride + (int64_t)(h * G + g) * HD);
        float qv[8][4];
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 8; j++) {
          uint2 w = make_uint2(0u, 0u);
          if (have_col) w = __ldg(reinterpret_cast<const uint2 *>(qp) + 4 * j + tig);
          if (F16) {
            qv[j][0] = f16lo_to_float(w.x); qv[j][1] = f16hi_to_float(w.x);
            qv[j][2] = f16lo_to_float(w.y); qv[j][3] = f16hi_to_float(w.y);
          } else {
            qv[j][0] = __uint_as_float(w.x << 16); qv[j][1] = __uint_as_float(w.x & 0xffff0000u);
            qv[j][2] = __uint_as_float(w.y << 16); qv[j][3] = __uint_as_float(w.y & 0xffff0000u);
          }
#pragma unroll
          for (int i = 0; i < 4; i++) amax = fmaxf(amax, fabsf(qv[j][i]));
        }
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        const int ex = (int)((__float_as_uint(amax) >> 23) & 0xffu);
        q_exp = (ex == 0 || ex == 255) ? 0 : min(133 - ex, 120);
        const float up = __uint_as_float((uint32_t)(q_exp + 127) << 23);
#pragma unroll
        for (int j = 0; j < 8; j++) {
          const float x0 = qv[j][0] * up, x1 = qv[j][1] * up, x2 = qv[j][2] * up,
                      x3 = qv[j][3] * up;
          const uint32_t hi8 = pack_e4m3x4(x0, x1, x2, x3);
          uint32_t ha, hb;
          fp8x4_to_f16<false>(hi8, ha, hb);
          const uint32_t lo8 = pack_e4m3x4(x0 - f16lo_to_float(ha) * kFp8Unbias,
                                           x1 - f16hi_to_float(ha) * kFp8Unbias,
                                           x2 - f16lo_to_float(hb) * kFp8Unbias,
                                           x3 - f16hi_to_float(hb) * kFp8Unbias);
          qf[nt][j >> 1][j & 1] = hi8;
          qf[nt][4 + (j >> 1)][j & 1] = lo8;
        }
      } else if (col < ncols) {
        const int qj = col / G, g = col - qj * G;
        const uint32_t *qp = reinterpret_cast<const uint32_t *>(
            p.q + (int64_t)(q0 + qj) * p.q_stride + (int64_t)(h * G + g) * HD);
#pragma unroll
        for (int j = 0; j < KS; j++) {
          if (FP8) {
            // k-slots {2tig, 2tig+1, 2tig+8, 2tig+9} of step j carry d = 16j + 4tig .. +3,
            // the four bytes a thread gets from one 16-byte K row piece
            const uint2 w = __ldg(reinterpret_cast<const uint2 *>(qp) + 4 * j + tig);
            qf[nt][j][0] = F16 ? w.x : bf16x2_to_f16x2(w.x);
            qf[nt][j][1] = F16 ? w.y : bf16x2_to_f16x2(w.y);
          } else {
            qf[nt][j][0] = __ldg(qp + 8 * j + tig);
            qf[nt][j][1] = (HD % 16 != 0 && j == KS - 1) ? 0u : __ldg(qp + 8 * j + 4 + tig);
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < KS; j++) qf[nt][j][0] = qf[nt][j][1] = 0u;
      }
      if (QK8) {
#pragma unroll
        for (int c = 0; c < 2; c++) {
          // the exponent of column 2tig+c sits with the threads whose gid is that column;
          // in the fast variant the K bytes are taken at face value (no 2^8 left out)
          const int e = __shfl_sync(0xffffffffu, q_exp, (2 * tig + c) * 4);
          col_lin[nt][c] = p.scale * p.k_scale * __uint_as_float((uint32_t)(127 - e) << 23);
        }
      }
    }
    // First segment: the ring starts here, behind the query loads issued above and before
    // anything waits for them or for the context length.  Issued the other way round,
    // those few loads queue behind the first ~28 MB of bulk copies of the whole grid
    // (measured: 3 us instead of 1).
    if constexpr (!FP8) {
      if (a == 0)
        for (int j = 0; j < NST && j < n_w; j++) issue();
    }
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
      for (int c = 0; c < 2; c++) {
        const int cc = nt * 8 + 2 * tig + c;
        lim[nt][c] = cc < ncols ? kv_len - q_len + cc / G + 1 : 0;
      }
    const int min_lim = kv_len - q_len + 1;

    float o[KSA][NT][4];
    float m[NT][2], l[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
      m[nt][0] = m[nt][1] = -INFINITY;
      l[nt][0] = l[nt][1] = 0.f;
#pragma unroll
      for (int mt = 0; mt < KS; mt++)
#pragma unroll
        for (int i = 0; i < 4; i++) o[mt][nt][i] = 0.f;
    }

    // S^T = K.Q^T of the unit in ring stage `st`
    auto s_phase = [&](int st, float (&sacc)[NT][4], int sub = 0) {
        const uint32_t ks = ring_w + st * kStageBytes;
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
          for (int i = 0; i < 4; i++) sacc[nt][i] = 0.f;
        if (QK8) {
          float slo[NT][4];
#pragma unroll
          for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int i = 0; i < 4; i++) slo[nt][i] = 0.f;
#pragma unroll
          for (int st32 = 0; st32 < 4; st32++) {
            // one 32-wide step: 16-byte row pieces of chunks 2s and 2s+1, rows 0-7 and 8-15,
            // land in the registers in the order the A operand wants them
            uint32_t r[4];
            ldmatrix_x4(r, ks + (2 * st32 + (mi >> 1)) * 256 + fp8_row_token((mi & 1) * 8 + mr) * 16);
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
              mma_fp8_16832(sacc[nt], r, qf[nt][st32][0], qf[nt][st32][1]);
              // a second accumulator halves the dependent chain (not for the widest
              // variant, which has no registers to spare)
              mma_fp8_16832(NT < 3 ? slo[nt] : sacc[nt], r, qf[nt][4 + st32][0], qf[nt][4 + st32][1]);
            }
          }
#pragma unroll
          for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int i = 0; i < 4; i++) sacc[nt][i] += slo[nt][i];
        } else if (FP8) {
#pragma unroll
          for (int jj = 0; jj < 4; jj++) {
            // matrices: (rows 0-7, step 2jj), (rows 8-15, step 2jj), then the same of step 2jj+1;
            // a row of a matrix is the 16 bytes (one whole k-step) of one token
            uint32_t r[4];
            ldmatrix_x4(r, ks + (2 * jj + (mi >> 1)) * 256 + fp8_row_token((mi & 1) * 8 + mr) * 16);
#pragma unroll
            for (int hf = 0; hf < 2; hf++) {
              uint32_t af[4];
              fp8x4_to_f16<EXACT>(r[2 * hf], af[0], af[2]);
              fp8x4_to_f16<EXACT>(r[2 * hf + 1], af[1], af[3]);
#pragma unroll
              for (int nt = 0; nt < NT; nt++)
                mma_16816<MF16>(sacc[nt], af, qf[nt][2 * jj + hf][0], qf[nt][2 * jj + hf][1]);
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < KS; j++) {
            uint32_t af[4];
            // B8: tokens 0-7 and 8-15 sit in the two 2 KB sub-chunks, rows of 8 tokens
            // B32: a K row holds 32 tokens (512 B), the sub-unit's 16 at offset sub * 256
            if (B8) ldmatrix_x4(af, ks + (mi & 1) * 2048 + (2 * j + (mi >> 1)) * 128 + mr * 16);
            else if (B32) ldmatrix_x4(af, ks + (2 * j + (mi >> 1)) * 512 + sub * 256 + ((mi & 1) * 8 + mr) * 16);
            else ldmatrix_x4(af, ks + (2 * j + (mi >> 1)) * 256 + ((mi & 1) * 8 + mr) * 16);
            // the K chunk has no second row for a half-empty last step: what was read there
            // belongs to the V chunk and 0 * NaN is NaN
            if (HD % 16 != 0 && j == KS - 1) af[2] = af[3] = 0u;
#pragma unroll
            for (int nt = 0; nt < NT; nt++) mma_16816<MF16>(sacc[nt], af, qf[nt][j][0], qf[nt][j][1]);
          }
        }
    };
    // softmax of the unit's logits and O^T += V^T.P^T, V from ring stage `st`
    // (blk counts 16-token sub-units of the item)
    auto finish = [&](int st, int blk, float (&sacc)[NT][4], int sub = 0) {
        const uint32_t vs = ring_w + st * kStageBytes + kChunk;
        const int tok0 = blk * kBlockSize + (FP8 ? fp8_row_token(gid) : gid);
        const int tok1 = FP8 ? tok0 + 2 : tok0 + 8;
        const bool need_mask = (blk + 1) * kBlockSize > min_lim;
        float alpha[NT][2];
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
#pragma unroll
          for (int i = 0; i < 4; i++) {
            float x = sacc[nt][i];
            if (QK8) {
              x *= col_lin[nt][i & 1];
              if (use_cap) x = tanhf(x / p.softcap) * p.softcap;
              x *= kLog2e;
            } else if (use_cap) {
              x = tanhf(x * qk_scale / p.softcap) * p.softcap * kLog2e;
            } else {
              x *= sc_log2;
            }
            sacc[nt][i] = x;
          }
          if (need_mask) {
            if (tok0 >= lim[nt][0]) sacc[nt][0] = -INFINITY;
            if (tok0 >= lim[nt][1]) sacc[nt][1] = -INFINITY;
            if (tok1 >= lim[nt][0]) sacc[nt][2] = -INFINITY;
            if (tok1 >= lim[nt][1]) sacc[nt][3] = -INFINITY;
          }
#pragma unroll
          for (int c = 0; c < 2; c++) {
            float mx = fmaxf(sacc[nt][c], sacc[nt][c + 2]);
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
            const float m_new = fmaxf(m[nt][c], mx);
            const float m_safe = m_new == -INFINITY ? 0.f : m_new;
            const float al = fast_exp2(m[nt][c] - m_safe);
            const float p0 = fast_exp2(sacc[nt][c] - m_safe);
            const float p1 = fast_exp2(sacc[nt][c + 2] - m_safe);
            m[nt][c] = m_new;
            l[nt][c] = l[nt][c] * al + p0 + p1;
            sacc[nt][c] = p0;
            sacc[nt][c + 2] = p1;
            alpha[nt][c] = al;
          }
        }
        uint32_t pb[NT][2];
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
          pb[nt][0] = movmatrix_trans(pack2<MF16>(sacc[nt][0], sacc[nt][1]));
          pb[nt][1] = movmatrix_trans(pack2<MF16>(sacc[nt][2], sacc[nt][3]));
        }
        // Tokens past the context in the last block may hold anything (NaN
        // included) and 0*NaN is NaN: clear them in the V fragments
        // (crates/.../paged_attention.metal:1073-1080 does the same per lane).
        const int valid = kv_len - blk * kBlockSize;  // >= 1
        uint32_t vmask[2] = {0xffffffffu, 0xffffffffu};
        if (valid < kBlockSize) {
          if (FP8) {  // one byte per token; a thread's piece holds tokens 4tig .. 4tig+3
            vmask[0] = 0u;
#pragma unroll
            for (int i = 0; i < 4; i++)
              if (4 * tig + i < valid) vmask[0] |= 0xffu << (8 * i);
          } else {
#pragma unroll
            for (int hh = 0; hh < 2; hh++) {
              const int t = hh * 8 + 2 * tig;
              vmask[hh] = (t < valid ? 0x0000ffffu : 0u) | (t + 1 < valid ? 0xffff0000u : 0u);
            }
          }
        }
        if (FP8) {
#pragma unroll
          for (int mm = 0; mm < 4; mm++) {
            // matrices: d rows 0-7 and 8-15 of m-tile 2mm, then of m-tile 2mm+1; a row is
            // the 16 tokens of one head dimension
            uint32_t r[4];
            ldmatrix_x4(r, vs + (32 * mm + (mi >> 1) * 16 + (mi & 1) * 8 + mr) * 16);
#pragma unroll
            for (int hf = 0; hf < 2; hf++) {
              const int mt = 2 * mm + hf;
              uint32_t vf[4];
              fp8x4_to_f16<EXACT>(r[2 * hf] & vmask[0], vf[0], vf[2]);
              fp8x4_to_f16<EXACT>(r[2 * hf + 1] & vmask[0], vf[1], vf[3]);
#pragma unroll
              for (int nt = 0; nt < NT; nt++) {
                o[mt][nt][0] *= alpha[nt][0]; o[mt][nt][1] *= alpha[nt][1];
                o[mt][nt][2] *= alpha[nt][0]; o[mt][nt][3] *= alpha[nt][1];
                mma_16816<MF16>(o[mt][nt], vf, pb[nt][0], pb[nt][1]);
              }
            }
          }
        } else {
#pragma unroll
          for (int mt = 0; mt < KS; mt++) {
            uint32_t vf[4];
            // B32: a V row holds 32 tokens (64 B), the sub-unit's 16 at offset sub * 32
            if (B8) ldmatrix_x4(vf, vs + (mi >> 1) * 2048 + (16 * mt + (mi & 1) * 8 + mr) * 16);
            else if (B32) ldmatrix_x4(vf, vs + (16 * mt + (mi & 1) * 8 + mr) * 64 + sub * 32 + (mi >> 1) * 16);
            else ldmatrix_x4(vf, vs + (16 * mt + (mi & 1) * 8 + mr) * 32 + (mi >> 1) * 16);
            vf[0] &= vmask[0]; vf[1] &= vmask[0]; vf[2] &= vmask[1]; vf[3] &= vmask[1];
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
              o[mt][nt][0] *= alpha[nt][0]; o[mt][nt][1] *= alpha[nt][1];
              o[mt][nt][2] *= alpha[nt][0]; o[mt][nt][3] *= alpha[nt][1];
              mma_16816<MF16>(o[mt][nt], vf, pb[nt][0], pb[nt][1]);
            }
          }
        }
    };
    // Decode step in one launch: if this segment reaches the item's last block, the warp
    // that gets that block stores the step's new token of this kv head to its pool slot and
    // into the staged copy of the block (fetched before the token was in the pool).
    // Exactly one warp of the grid handles a given (sequence, kv head, last block), so
    // nobody else reads that slot during this launch.  The token's rows are fetched here,
    // next to the queries, so that their latency is not paid at the end of the segment.
    uint4 new_k = make_uint4(0u, 0u, 0u, 0u);
    uint2 new_v = make_uint2(0u, 0u);
    int64_t new_slot = -1;
    uint32_t new_id = 0u;
    if constexpr (kCanFuseWrite) {
      if (fuse_write && b1 == nb) {
        new_slot = p.slot_mapping[seq];
        const int row = p.seq_row ? p.seq_row[seq] : seq;
        new_id = (uint32_t)p.block_tables[(long long)row * p.MB + ((kv_len - 1) >> 4)];
        if (lane < 16)
          new_k = __ldg(reinterpret_cast<const uint4 *>(
                            p.k_new + (int64_t)seq * p.k_new_stride + h * HD) + lane);
        new_v = __ldg(reinterpret_cast<const uint2 *>(
                          p.v_new + (int64_t)seq * p.v_new_stride + h * HD) + lane);
      }
    }
    auto write_new_token = [&](int st) {
      if (new_slot < 0) return;  // "no write" (crates/.../reshape_and_cache.metal:59-63)
      const int off = (kv_len - 1) & (kBlockSize - 1);
      if (new_id >= p.num_blocks || new_slot != (int64_t)new_id * kBlockSize + off) {
        if (lane == 0) atomicOr(p.err, kErrStepSlot);
        return;
      }
      const size_t chunk = (size_t)new_id * Hkv + h;
      const uint32_t ks = ring_w + st * kStageBytes, vs = ks + kChunk;
      uint8_t *kg = const_cast<uint8_t *>(reinterpret_cast<const uint8_t *>(p.k_pool)) + chunk * kChunk;
      uint8_t *vg = const_cast<uint8_t *>(reinterpret_cast<const uint8_t *>(p.v_pool)) + chunk * kChunk;
      if (lane < 16) {  // K: sixteen 16-byte pieces, piece c to [c][off][0..7]
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(ks + lane * 256 + off * 16),
                     "r"(new_k.x), "r"(new_k.y), "r"(new_k.z), "r"(new_k.w) : "memory");
        *reinterpret_cast<uint4 *>(kg + lane * 256 + off * 16) = new_k;
      }
      // V: element d to [d][off]; a lane takes d = 4 lane .. 4 lane + 3
      const uint16_t e[4] = {(uint16_t)(new_v.x & 0xffffu), (uint16_t)(new_v.x >> 16),
                             (uint16_t)(new_v.y & 0xffffu), (uint16_t)(new_v.y >> 16)};
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const int d = 4 * lane + i;
        asm volatile("st.shared.u16 [%0], %1;" ::"r"(vs + d * 32 + off * 2), "h"(e[i]) : "memory");
        *reinterpret_cast<uint16_t *>(vg + d * 32 + off * 2) = e[i];
      }
      // the stage is refilled by a bulk copy later on: order these writes before it
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
    };
    // Waits for the next unit of this warp (block `blk` of the item); false once a wait
    // has run out.
    auto wait_unit = [&](int j, int blk) {
      const bool ok = mbar_wait_bounded(bar_w + (j % NST) * 8, (j / NST) & 1);
      if (!__all_sync(0xffffffffu, ok)) {
        dead = true;
        if (lane == 0) atomicOr(p.err, kErrTimeout);
      }
      if constexpr (kCanFuseWrite)
        if (fuse_write && !dead && blk == nb - 1) write_new_token(j % NST);
      return !dead;
    };
    // The warp's units of this segment, software-pipelined: the logits of unit i+1 are
    // computed in the same straight-line block as the softmax and P.V of unit i, so that
    // the two dependency chains fill each other's latencies.  Two units are then held at
    // once, so a third ring stage is needed for a copy to be in flight meanwhile; the
    // two-stage variant takes its units one at a time.
    constexpr bool kPipelined = NST >= 3;
    if constexpr (!kPipelined) {
      for (int k = a + ((warp - a) & (kWarps - 1)); k < a + seglen; k += kWarps) {
        if (!dead && wait_unit(jc, b0 + (k - a))) {
#pragma unroll
          for (int sub = 0; sub < SUB; sub++) {
            const int blk16 = (b0 + (k - a)) * SUB + sub;
            if (sub > 0 && blk16 * kBlockSize >= kv_len) break;  // the block's second half is empty
            float s_cur[NT][4];
            s_phase(jc % NST, s_cur, sub);
            finish(jc % NST, blk16, s_cur, sub);
          }
        }
        __syncwarp();
        jc++;
        if (ji < n_w) issue();
      }
    } else {
      int k = a + ((warp - a) & (kWarps - 1));
      const int k_end = a + seglen;
      float s_cur[NT][4];
      bool cur_ok = false;
      if (k < k_end && !dead && wait_unit(jc, b0 + (k - a))) {
        s_phase(jc % NST, s_cur);
        cur_ok = true;
      }
      while (k < k_end) {
        const int kn = k + kWarps;
        if (cur_ok && kn < k_end && wait_unit(jc + 1, b0 + (kn - a))) {
          float s_next[NT][4];
          s_phase((jc + 1) % NST, s_next);
          finish(jc % NST, b0 + (k - a), s_cur);
#pragma unroll
          for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int i = 0; i < 4; i++) s_cur[nt][i] = s_next[nt][i];
        } else {
          if (cur_ok && !dead) finish(jc % NST, b0 + (k - a), s_cur);
          cur_ok = false;
        }
        __syncwarp();
        jc++;
        if (ji < n_w) issue();
        k = kn;
      }
    }

    // ---- combine the eight warps' partials (fixed order) -----------------------
    // Warps 4-7 hand theirs to warps 0-3 through four slots; warps 1-3 then put their
    // sums back into the slot they have just read (a lane reads and writes its own
    // column only) and warp 0 adds them in order: three barriers per item.
    auto put = [&](int slot) {
      float *dst = merge_buf + slot * (C::kRegs * 32) + lane;
#pragma unroll
      for (int mt = 0; mt < KS; mt++)
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
          for (int i = 0; i < 4; i++) dst[((mt * NT + nt) * 4 + i) * 32] = o[mt][nt][i];
#pragma unroll
      for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int c = 0; c < 2; c++) {
          dst[(kAcc * NT + nt * 2 + c) * 32] = m[nt][c];
          dst[((kAcc + 2) * NT + nt * 2 + c) * 32] = l[nt][c];
        }
    };
    auto take = [&](int slot) {
      const float *src = merge_buf + slot * (C::kRegs * 32) + lane;
#pragma unroll
      for (int nt = 0; nt < NT; nt++) {
        float wa[2], wb[2];
#pragma unroll
        for (int c = 0; c < 2; c++) {
          const float mb = src[(kAcc * NT + nt * 2 + c) * 32];
          const float lb = src[((kAcc + 2) * NT + nt * 2 + c) * 32];
          const float mm = fmaxf(m[nt][c], mb);
          wa[c] = m[nt][c] == -INFINITY ? 0.f : fast_exp2(m[nt][c] - mm);
          wb[c] = mb == -INFINITY ? 0.f : fast_exp2(mb - mm);
          m[nt][c] = mm;
          l[nt][c] = l[nt][c] * wa[c] + lb * wb[c];
        }
#pragma unroll
        for (int mt = 0; mt < KS; mt++)
#pragma unroll
          for (int i = 0; i < 4; i++)
            o[mt][nt][i] = o[mt][nt][i] * wa[i & 1] + src[((mt * NT + nt) * 4 + i) * 32] * wb[i & 1];
      }
    };
    if (warp >= kWarps / 2) put(warp - kWarps / 2);
    __syncthreads();
    if (warp < kWarps / 2) take(warp);
    if (warp >= 1 && warp < kWarps / 2) put(warp);
    __syncthreads();
    if (warp == 0) {
#pragma unroll
      for (int w2 = 1; w2 < kWarps / 2; w2++) take(w2);
    }
    __syncthreads();

    const bool partial = b0 > 0 || b1 < nb;
    if (warp == 0) {
#pragma unroll
      for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int c = 0; c < 2; c++) {
          float v = l[nt][c];
          v += __shfl_xor_sync(0xffffffffu, v, 4);
          v += __shfl_xor_sync(0xffffffffu, v, 8);
          v += __shfl_xor_sync(0xffffffffu, v, 16);
          l[nt][c] = v;
        }
      if (partial) {
        float *dst = p.ws + (size_t)(2 * (p.cta_base + blockIdx.x) + (b0 > 0 ? 0 : 1)) * kSlotFloats + lane;
#pragma unroll
        for (int mt = 0; mt < KS; mt++)
#pragma unroll
          for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int i = 0; i < 4; i++)
              dst[((mt * NT + nt) * 4 + i) * 32] = FP8 ? o[mt][nt][i] * v_unscale : o[mt][nt][i];
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
          for (int c = 0; c < 2; c++) {
            dst[(kAcc * NT + nt * 2 + c) * 32] = m[nt][c];
            dst[((kAcc + 2) * NT + nt * 2 + c) * 32] = l[nt][c];
          }
        __threadfence();  // the partial is visible before this CTA counts itself below
      } else {
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
          for (int c = 0; c < 2; c++) {
            const int col = nt * 8 + 2 * tig + c;
            if (col < ncols) {
              const int qj = col / G, g = col - qj * G;
              float inv = l[nt][c] > 0.f ? 1.f / l[nt][c] : 0.f;
              if (FP8) inv *= v_unscale;
              elem16 *op = p.out + (int64_t)(q0 + qj) * p.out_stride +
                                  (int64_t)(h * G + g) * HD;
#pragma unroll
              for (int mt = 0; mt < KS; mt++) {
                op[16 * mt + gid] = to_elem<F16>(o[mt][nt][c] * inv);
                if (HD % 16 == 0 || mt < KS - 1) op[16 * mt + gid + 8] = to_elem<F16>(o[mt][nt][c + 2] * inv);
              }
            }
          }
      }
    }

    // ---- a split item: count this piece; the last piece to arrive combines them ----
    if (partial) {
      const long long U0 = (long long)Hkv * pre[s] + (long long)h * nb, U1 = U0 + nb;
      const int c_first = cta_of(U0), c_last = cta_of(U1 - 1);
      __syncthreads();
      if (tid == 0) {
        // Pieces of the item: one per CTA of [c_first, c_last] that owns anything.
        unsigned pieces = 0;
        for (int c = c_first; c <= c_last; c++) pieces += bnd[c + 1] > bnd[c] ? 1u : 0u;
        // c_first holds the item as its last one, so the word is this item's alone
        const unsigned arrived = atomicAdd(p.sync + p.cta_base + c_first, 1u) + 1u;
        s_last = arrived == pieces;
        if (arrived == pieces) atomicExch(p.sync + p.cta_base + c_first, 0u);
      }
      __syncthreads();
      if (s_last) {
        __threadfence();
        merge_item<NT, F16, HD>(p, bnd, c_first, c_last, q0, h, ncols, tid);
      }
    }

    // ---- next item ---------------------------------------------------------------
    a += seglen;
    b0 = 0;
    if (++h == Hkv) {
      h = 0;
      do { s++; } while (s < S && pre[s + 1] == pre[s]);
    }
    if (s < S) nb = pre[s + 1] - pre[s];
  }
  };
  if (n_local > 0) {
    if constexpr (FP8) {
      if (*p.fp8_special != 0u) main_loop(std::true_type{});
      else main_loop(std::false_type{});
    } else {
      main_loop(std::false_type{});
    }
  }
  // The last CTA of the grid to get here leaves a copy of the error word where the host
  // can read it without a copy of its own: every kernel of this stream that can set a
  // bit in this call has finished by then.
  if (p.err_mirror) {
    __syncthreads();
    if (tid == 0) {
      __threadfence();
      if (atomicAdd(p.sync + kSyncDone - p.lane, 1u) + 1u == gridDim.x) {
        atomicExch(p.sync + kSyncDone - p.lane, 0u);
        *p.err_mirror = *reinterpret_cast<volatile unsigned *>(p.err);
      }
    }
  }
}

// Launch with programmatic stream serialisation: the grid may start while its
// predecessor in the stream drains; it orders itself with griddepcontrol.wait.
template <typename... KArgs, typename... Args>
cudaError_t launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                             cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}

// Head sizes 64 and 256: 16-bit pools with 16-token blocks, attention only.
template <int NT, int HD>
cudaError_t launch_hd(const AttnParams &p, const KvMaps &maps, int num_ctas, cudaStream_t st) {
  cudaError_t e;
  if (p.bs_shift > 0) {  // 32-token blocks: whole blocks per stage, head sizes up to 128
    if constexpr (HD <= kHeadSize)
      e = p.is_f16 ? launch_dependent(splitkv_kernel<NT, true, false, false, false, HD, true>, dim3(num_ctas),
                                      dim3(kThreads), Cfg<NT, false, HD, 2>::kSmemBytes, st, p, maps)
                   : launch_dependent(splitkv_kernel<NT, false, false, false, false, HD, true>, dim3(num_ctas),
                                      dim3(kThreads), Cfg<NT, false, HD, 2>::kSmemBytes, st, p, maps);
    else
      return cudaErrorInvalidValue;
  } else {
    e = p.is_f16 ? launch_dependent(splitkv_kernel<NT, true, false, false, false, HD>, dim3(num_ctas),
                                    dim3(kThreads), Cfg<NT, false, HD>::kSmemBytes, st, p, maps)
                 : launch_dependent(splitkv_kernel<NT, false, false, false, false, HD>, dim3(num_ctas),
                                    dim3(kThreads), Cfg<NT, false, HD>::kSmemBytes, st, p, maps);
  }
  __atomic_fetch_add(&g_launch_count, 1ull, __ATOMIC_RELAXED);
  return e;
}

template <int NT>
cudaError_t launch_nt(const AttnParams &p, const KvMaps &maps, int num_ctas, cudaStream_t st) {
  switch (p.head_size) {
    case kHeadSize: break;
    case 32: return launch_hd<NT, 32>(p, maps, num_ctas, st);
    case 64: return launch_hd<NT, 64>(p, maps, num_ctas, st);
    case 80: return launch_hd<NT, 80>(p, maps, num_ctas, st);
    case 96: return launch_hd<NT, 96>(p, maps, num_ctas, st);
    case 112: return launch_hd<NT, 112>(p, maps, num_ctas, st);
    case 120: return launch_hd<NT, 120>(p, maps, num_ctas, st);
    case 192:  // wider items are cut into pieces by the caller (splitkv_max_cols_for)
      if constexpr (NT <= 2) return launch_hd<NT, 192>(p, maps, num_ctas, st);
      else return cudaErrorInvalidValue;
    case 256:
      if constexpr (NT == 1) return launch_hd<1, 256>(p, maps, num_ctas, st);
      else return cudaErrorInvalidValue;
    default: return cudaErrorInvalidValue;
  }
  cudaError_t e;
  if (p.bs_shift > 0 && !p.is_fp8)  // 16-bit pools of 32-token blocks: whole blocks per stage
    e = p.is_f16 ? launch_dependent(splitkv_kernel<NT, true, false, false, false, kHeadSize, true>,
                                    dim3(num_ctas), dim3(kThreads),
                                    Cfg<NT, false, kHeadSize, 2>::kSmemBytes, st, p, maps)
                 : launch_dependent(splitkv_kernel<NT, false, false, false, false, kHeadSize, true>,
                                    dim3(num_ctas), dim3(kThreads),
                                    Cfg<NT, false, kHeadSize, 2>::kSmemBytes, st, p, maps);
  else if (p.is_fp8)
    e = p.is_f16 ? launch_dependent(splitkv_kernel<NT, true, true>, dim3(num_ctas), dim3(kThreads),
                                    Cfg<NT, true>::kSmemBytes, st, p, maps)
                 : launch_dependent(splitkv_kernel<NT, false, true>, dim3(num_ctas),
                                    dim3(kThreads), Cfg<NT, true>::kSmemBytes, st, p, maps);
  else if (p.bs_shift < 0)
    e = p.is_f16 ? launch_dependent(splitkv_kernel<NT, true, false, true>, dim3(num_ctas),
                                    dim3(kThreads), Cfg<NT>::kSmemBytes, st, p, maps)
                 : launch_dependent(splitkv_kernel<NT, false, false, true>, dim3(num_ctas),
                                    dim3(kThreads), Cfg<NT>::kSmemBytes, st, p, maps);
  else if (NT == 1 && p.k_new)
    e = p.is_f16 ? launch_dependent(splitkv_kernel<1, true, false, false, true>, dim3(num_ctas),
                                    dim3(kThreads), Cfg<1>::kSmemBytes, st, p, maps)
                 : launch_dependent(splitkv_kernel<1, false, false, false, true>, dim3(num_ctas),
                                    dim3(kThreads), Cfg<1>::kSmemBytes, st, p, maps);
  else
    e = p.is_f16 ? launch_dependent(splitkv_kernel<NT, true, false>, dim3(num_ctas), dim3(kThreads),
                                    Cfg<NT>::kSmemBytes, st, p, maps)
                 : launch_dependent(splitkv_kernel<NT, false, false>, dim3(num_ctas),
                                    dim3(kThreads), Cfg<NT>::kSmemBytes, st, p, maps);
  __atomic_fetch_add(&g_launch_count, 1ull, __ATOMIC_RELAXED);
  return e;
}

}  // namespace

// ---- scratch that needs no allocation ----------------------------------------
// Partial-result slots for up to kStaticMaxCtas CTAs, resident in every process
// that loads the library on every GPU it touches (4.2 MiB each) until exit.
constexpr int kStaticMaxCtas = 160;
static __device__ __align__(256) float g_static_scratch[(size_t)kStaticMaxCtas * 2 * kSlotFloats];

int splitkv_static_max_ctas() { return kStaticMaxCtas; }

// Device address of the static scratch on `device`, which must be the current
// device.  In host code the array's name is only a handle, so the address is asked
// of the runtime once per device and remembered.
cudaError_t splitkv_static_scratch(int device, float **out) {
  constexpr int kMaxDevices = 64;
  static float *ptrs[kMaxDevices] = {};
  static std::mutex mu;
  if (device < 0 || device >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(mu);
  if (!ptrs[device]) {
    float *ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void **>(&ptr), g_static_scratch);
    if (e != cudaSuccess) return e;
    ptrs[device] = ptr;
  }
  *out = ptrs[device];
  return cudaSuccess;
}

int splitkv_max_cols() { return 8 * kMaxNT; }
int splitkv_narrow_ctas_per_sm(int head_size, bool fp8) { return (fp8 || head_size <= kTwoCtaMaxHead) ? 2 : 1; }
// Head size 256 leaves registers for one 8-column tile only, 192 for two.
int splitkv_max_cols_for(int head_size) { return head_size == 256 ? 8 : head_size == 192 ? 16 : 8 * kMaxNT; }

size_t splitkv_workspace_bytes(int num_ctas) {
  return (size_t)num_ctas * 2 * kSlotFloats * sizeof(float);
}

template <int NT>
static cudaError_t configure_nt() {
  cudaError_t e = cudaFuncSetAttribute(splitkv_kernel<NT, false, false>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<NT>::kSmemBytes);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(splitkv_kernel<NT, true, false>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<NT>::kSmemBytes);
  if (e == cudaSuccess && NT == 1)
    e = cudaFuncSetAttribute(splitkv_kernel<1, false, false, false, true>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<1>::kSmemBytes);
  if (e == cudaSuccess && NT == 1)
    e = cudaFuncSetAttribute(splitkv_kernel<1, true, false, false, true>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<1>::kSmemBytes);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(splitkv_kernel<NT, false, false, true>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<NT>::kSmemBytes);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(splitkv_kernel<NT, true, false, true>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<NT>::kSmemBytes);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(splitkv_kernel<NT, false, true>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<NT, true>::kSmemBytes);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(splitkv_kernel<NT, true, true>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<NT, true>::kSmemBytes);
  auto head = [&](auto hd_tag) {
    constexpr int HD = decltype(hd_tag)::value;
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(splitkv_kernel<NT, false, false, false, false, HD>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<NT, false, HD>::kSmemBytes);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(splitkv_kernel<NT, true, false, false, false, HD>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<NT, false, HD>::kSmemBytes);
    if constexpr (HD <= kHeadSize) {
      if (e == cudaSuccess)
        e = cudaFuncSetAttribute(splitkv_kernel<NT, false, false, false, false, HD, true>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<NT, false, HD, 2>::kSmemBytes);
      if (e == cudaSuccess)
        e = cudaFuncSetAttribute(splitkv_kernel<NT, true, false, false, false, HD, true>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<NT, false, HD, 2>::kSmemBytes);
    }
  };
  head(std::integral_constant<int, 32>{});
  head(std::integral_constant<int, 64>{});
  head(std::integral_constant<int, 80>{});
  head(std::integral_constant<int, 96>{});
  head(std::integral_constant<int, 112>{});
  head(std::integral_constant<int, 120>{});
  if constexpr (NT <= 2) head(std::integral_constant<int, 192>{});
  if constexpr (NT == 1) head(std::integral_constant<int, 256>{});
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(splitkv_kernel<NT, false, false, false, false, kHeadSize, true>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                             Cfg<NT, false, kHeadSize, 2>::kSmemBytes);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(splitkv_kernel<NT, true, false, false, false, kHeadSize, true>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                             Cfg<NT, false, kHeadSize, 2>::kSmemBytes);
  return e;
}

cudaError_t splitkv_configure() {
  cudaError_t e = configure_nt<1>();
  if (e == cudaSuccess) e = configure_nt<2>();
  if (e == cudaSuccess) e = configure_nt<3>();
  return e;
}

// Tensor maps that fetch one 16-token unit out of a (block, kv head) chunk of `block_size`
// tokens: K as {block_size * 8 elements (16-bit) or block_size * 16 (bytes), D/8 or D/16
// rows, chunk}, box {one unit, every row}; V as {block_size, D, chunk}, box {16, D}.  No
// swizzle: the box arrives in shared memory row after row, which is the layout of a
// 16-token chunk.
cudaError_t encode_unit_maps(UnitMaps *out, const void *k_pool, const void *v_pool,
                             uint64_t num_chunks, int block_size, bool fp8) {
  static_assert(sizeof(CUtensorMap) == sizeof(TensorMapBlob), "tensor map size");
  static_assert(sizeof(KvMaps) == sizeof(UnitMaps), "map pair size");
  using EncodeFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  void *fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
  if (e != cudaSuccess) return e;
  if (!fn || qres != cudaDriverEntryPointSuccess) return cudaErrorNotSupported;
  const uint64_t esz = fp8 ? 1 : 2;
  const uint64_t k_group = fp8 ? 16 : 8;  // elements of one token in a K row
  const cuuint32_t ones[3] = {1, 1, 1};
  const CUtensorMapDataType dt = fp8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_UINT16;
  const uint64_t chunk_bytes = (uint64_t)kHeadSize * block_size * esz;
  {
    const cuuint64_t dims[3] = {(cuuint64_t)block_size * k_group, kHeadSize / k_group, num_chunks};
    const cuuint64_t strides[2] = {(cuuint64_t)block_size * k_group * esz, chunk_bytes};
    const cuuint32_t box[3] = {(cuuint32_t)(kBlockSize * k_group), (cuuint32_t)(kHeadSize / k_group), 1};
    const CUresult r = reinterpret_cast<EncodeFn>(fn)(
        reinterpret_cast<CUtensorMap *>(&out->k), dt, 3, const_cast<void *>(k_pool), dims, strides,
        box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
  }
  {
    const cuuint64_t dims[3] = {(cuuint64_t)block_size, kHeadSize, num_chunks};
    const cuuint64_t strides[2] = {(cuuint64_t)block_size * esz, chunk_bytes};
    const cuuint32_t box[3] = {kBlockSize, kHeadSize, 1};
    const CUresult r = reinterpret_cast<EncodeFn>(fn)(
        reinterpret_cast<CUtensorMap *>(&out->v), dt, 3, const_cast<void *>(v_pool), dims, strides,
        box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
        CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
  }
  return cudaSuccess;
}

cudaError_t launch_splitkv_attention(const AttnParams &p_in, int num_sms_used, cudaStream_t st,
                                     const UnitMaps *unit_maps) {
  if (p_in.bs_shift > 0 && p_in.is_fp8 && !unit_maps) return cudaErrorInvalidValue;
  if (p_in.bs_shift < 0 && p_in.is_fp8) return cudaErrorInvalidValue;
  // (launch_nt refuses a head size that is not built)
  if (p_in.head_size != kHeadSize &&
      (p_in.is_fp8 || p_in.bs_shift < 0 || (p_in.bs_shift > 0 && p_in.head_size > kHeadSize) || p_in.k_new ||
       p_in.max_cols > splitkv_max_cols_for(p_in.head_size)))
    return cudaErrorInvalidValue;
  KvMaps maps;
  if (unit_maps) memcpy(&maps, unit_maps, sizeof(maps));
  else memset(&maps, 0, sizeof(maps));
  // Width of the kernel: enough 8-column tiles for the widest item it may meet.
  const int nt = (p_in.max_cols + 7) / 8;
  // CTAs: one per SM the caller grants, two for the variant built to share an SM, as far
  // as the workspace has partial-result slots for them.
  int num_ctas = num_sms_used;
  if ((p_in.is_fp8 || (p_in.head_size <= kTwoCtaMaxHead && p_in.bs_shift == 0)) && nt <= 1 &&
      p_in.cta_base + 2 * num_sms_used <= p_in.ws_ctas)
    num_ctas = 2 * num_sms_used;
  if (num_ctas < 1 || num_ctas > kMaxSplitCtas || !p_in.sync || p_in.cta_base < 0 ||
      p_in.cta_base + num_ctas > p_in.ws_ctas || p_in.cta_base + num_ctas > kSyncDone - kMaxLanes ||
      p_in.lane < 0 || p_in.lane >= kMaxLanes)
    return cudaErrorInvalidValue;
  for (int base = 0; base < p_in.S; base += kMaxSeqsPerLaunch) {
    AttnParams p = p_in;
    p.seq_base = p_in.seq_base + base;
    p.S = min(kMaxSeqsPerLaunch, p_in.S - base);
    p.item_cost = p.is_fp8 ? kItemCostUnitsFp8 : (p.bs_shift > 0 ? kItemCostUnits / 2 : kItemCostUnits);
    cudaError_t e;
    if (nt <= 1) e = launch_nt<1>(p, maps, num_ctas, st);
    else if (nt == 2) e = launch_nt<2>(p, maps, num_ctas, st);
    else e = launch_nt<3>(p, maps, num_ctas, st);
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
}

}  // namespace pa
