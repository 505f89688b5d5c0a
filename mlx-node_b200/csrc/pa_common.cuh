// Shared device helpers and kernel-launch declarations for the sm_100a
// paged-attention kernels.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace pa {

// One 16-bit element: a bf16 or an f16 bit pattern (cache dtype 1 or 0).  The copies
// never interpret it; the attention kernels are compiled for both formats.
using elem16 = uint16_t;

// Fixed geometry of the tuned path: head size 128, 16-bit elements, and a working unit of
// 16 tokens.  One (block, kv head) pair of the pool is a contiguous K chunk laid out
// [D/8][BS][8] and a contiguous V chunk laid out [D][BS]
// (crates/mlx-paged-attn/src/paged_kv_cache.rs:1129-1136: kv_head_stride = D*BS).
// With BS = 16 a chunk is one unit (4 KB of K, 4 KB of V, each contiguous); with BS = 32 it
// holds two units interleaved (tokens 0-15 and 16-31 of every row) and the kernels fetch
// a unit with a tensor-map copy; with BS = 8 a unit is two chunks of 2 KB.  `bs_shift`
// below is log2(BS / 16).
constexpr int kHeadSize = 128;
constexpr int kBlockSize = 16;                           // tokens of a unit
constexpr int kChunkBytes = kHeadSize * kBlockSize * 2;  // 4096: K (or V) bytes of a unit
constexpr int kChunkElems = kHeadSize * kBlockSize;      // 2048

// Error word bits written by kernels instead of trapping.
constexpr unsigned kErrBlockRange = 1u;  // block-table entry >= num_blocks
constexpr unsigned kErrSlotRange = 2u;   // slot >= num_blocks*block_size
constexpr unsigned kErrTimeout = 4u;     // a bounded wait ran out
constexpr unsigned kErrStepSlot = 8u;    // fused decode step: a slot is not its sequence's last position

constexpr int kSyncWords = 1024;         // arrival counters of a cache handle (AttnParams::sync)
constexpr int kSyncDone = 1023;          // index of the finished-CTA counter (launch lane 0; lane i uses kSyncDone - i)
constexpr int kMaxLanes = 3;             // split-KV launches of one call that may run at the same time
constexpr int kMaxSplitCtas = 320;       // CTAs of one split-KV launch (each has a counter word and a boundary in shared memory)

constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier + bulk async copy (TMA, untiled) -----------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      " selp.b32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after ~2^31 clocks (about a second), returns false.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (clock64() - t0 > (1ll << 31)) return false;
  }
  return true;
}
// 1-D bulk copy global -> shared of `bytes` (multiple of 16; both addresses
// 16-byte aligned), completion counted on `bar`.  Delivered to this CTA only.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes,
                                         uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}

// The same with an L2 eviction policy for the lines it brings in (see l2_evict_first).
__device__ __forceinline__ void bulk_g2s_hint(uint32_t dst, const void *src, uint32_t bytes,
                                              uint32_t bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1], %2, [%3], %4;" ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(policy)
      : "memory");
}
// Policy "evict these lines first": for data that is read once and not again soon.
__device__ __forceinline__ uint64_t l2_evict_first() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
  return policy;
}

// ---- warp-level tensor-core pieces ------------------------------------------
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
// D(16x8,f32) += A(16x16,row) * B(16x8,col), operands bf16 or f16
template <bool F16>
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                          uint32_t b1) {
  if (F16)
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  else
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// Transpose an 8x8 matrix of 16-bit elements held one 32-bit register per lane.
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
  return d;
}
// Pack two floats to a 16-bit pair (lo in the low half), round to nearest even.
template <bool F16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  uint32_t r;
  if (F16) asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  else asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
template <bool F16>
__device__ __forceinline__ elem16 to_elem(float x) {
  return (elem16)(pack2<F16>(x, 0.f) & 0xffffu);
}
__device__ __forceinline__ elem16 to_elem_rt(float x, bool f16) {
  return f16 ? to_elem<true>(x) : to_elem<false>(x);
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// ---- FP8 (E4M3) cache bytes -> f16 ---------------------------------------------
// Four cache bytes -> two f16x2 registers (bytes 0,1 and bytes 2,3) holding value / 256,
// by integer operations only: with the byte in the high half of a 16-bit lane, sign
// stays at bit 15 and the seven exponent/mantissa bits move down one place, which reads
// as an f16 with the E4M3 exponent field taken at bias 15 instead of 7 (subnormals
// included); the factor 2^8 is folded into the scales.  (The conversion instruction
// cvt.rn.f16x2.e4m3x2 measured about four times slower than this in the split-KV kernel.)
// The cache format (crates/mlx-paged-attn/metal/float8.metal:11-33) reads exponent
// field 15 as infinity (mantissa 0) or NaN; EXACT restores that by raising the f16
// exponent field from 15 to 31.  The fast variant is used while the cache is known to
// hold no such byte.
template <bool EXACT>
__device__ __forceinline__ void fp8x4_to_f16(uint32_t w, uint32_t &lo, uint32_t &hi) {
  const uint32_t xa = __byte_perm(w, 0u, 0x1404u);  // b1 << 24 | b0 << 8
  const uint32_t xb = __byte_perm(w, 0u, 0x3424u);  // b3 << 24 | b2 << 8
  lo = ((xa & 0x7F007F00u) >> 1) | (xa & 0x80008000u);
  hi = ((xb & 0x7F007F00u) >> 1) | (xb & 0x80008000u);
  if (EXACT) {
    lo |= ((lo & 0x3C003C00u) + 0x04000400u) & 0x40004000u;
    hi |= ((hi & 0x3C003C00u) + 0x04000400u) & 0x40004000u;
  }
}
constexpr float kFp8Unbias = 256.f;  // the factor the conversion above leaves out

__device__ __forceinline__ uint32_t bf16x2_to_f16x2(uint32_t w) {
  return pack2<true>(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}

// ---- launch parameter blocks --------------------------------------------------
struct AttnParams {
  const elem16 *q;
  elem16 *out;
  const elem16 *k_pool;
  const elem16 *v_pool;
  const int32_t *block_tables;  // [S, MB]
  const int32_t *context_lens;  // [S]
  const int32_t *cu_q_lens;     // [S+1] device copy, or null: one query per sequence
  const int32_t *seq_row;       // null, or [S]: block-table row of each sequence (when a long
                                // chunk is served as several shorter sequences)
  int S, Hq, Hkv, G, MB;
  int head_size;  // 128; 64 and 256 for 16-bit pools with 16-token blocks (split-KV kernel only)
  int bs_shift;  // log2(pool block size / 16): 0, 1 (32 tokens) or -1 (8 tokens); MB counts pool blocks
  int is_f16;  // element format: 1 = f16, 0 = bf16
  int is_fp8;  // pools hold E4M3 bytes; is_f16 is then the q/out format
  float k_scale, v_scale;  // FP8 dequantisation factors; 1 otherwise
  const unsigned *fp8_special;  // FP8: non-zero once the pools may hold an exponent-15 byte
  int early_trigger;  // split-KV: let the merge grid become resident at once
  uint32_t num_blocks;  // pool size, for range checks
  int64_t q_stride, out_stride;
  float scale;    // logits multiplier
  float softcap;  // 1.0f = off
  float *ws;      // partial results, two slots per CTA (layout: splitkv_attention.cu)
  int ws_ctas;    // CTAs the workspace has slots for
  unsigned *err;  // error word
  unsigned *err_mirror;  // null, or a host-visible word the last CTA to finish copies `err` to
  // Arrival counters of the cache handle, all zero between launches: word c counts the
  // CTAs that have stored their partial of the split item whose first piece CTA c holds;
  // word kSyncDone counts finished CTAs.  The last arriver does the work and clears the word.
  unsigned *sync;
  // Decode step in one launch (null = attention only): the new token of every sequence,
  // [S, Hkv, 128] with these row strides in elements, is written to its pool slot
  // (slot_mapping[s] must be position context_len - 1 of sequence s, or negative for
  // "no write") by the warp that attends the sequence's last block.
  const elem16 *k_new;
  const elem16 *v_new;
  const int64_t *slot_mapping;
  int64_t k_new_stride, v_new_stride;
  int seq_base;   // first sequence this launch covers
  // Several split-KV launches of one call may run at the same time (one per width class):
  // launch lane i keeps its partial slots and arrival counters from CTA index cta_base on
  // and counts its finished CTAs on word kSyncDone - lane.
  int cta_base, lane;
  int item_cost;  // split-KV partition: what starting an item costs a CTA, in units (set by the launcher)
  int min_cols;   // a sequence is taken by the split-KV launch iff min_cols <= q_len*G <= max_cols
  int max_cols;
};

// Producer (QK norm + rotary embedding + KV write) launch parameters.
struct ProducerParams {
  const elem16 *q_in;      // [T, Hq, 128] projected queries
  elem16 *q_out;           // rotated queries; may alias q_in
  const elem16 *k;         // [T, Hkv, 128] projected keys
  const elem16 *v;         // [T, Hkv, 128] projected values
  const elem16 *q_norm_w;  // [128] or null: no query norm
  const elem16 *k_norm_w;  // [128] or null: no key norm
  const int32_t *positions;     // [T] rotary position of each token
  const int64_t *slot_mapping;  // [T] pool slot of each token (< 0: not written)
  elem16 *k_pool, *v_pool;
  int64_t num_tokens, q_stride, q_out_stride, k_stride, v_stride;
  int tok_per_cta;         // 1..16, chosen by the launcher
  int bs_shift;            // log2(pool block size / 16): -1, 0 or 1
  int Hq, Hkv, rope_dims;  // rope_dims even, <= 128; elements beyond pass through
  uint32_t num_blocks;
  float eps;
  unsigned *err;
  float inv_freq[kHeadSize / 2];  // base^(-i/(rope_dims/2)), computed on the host
};

// Host-side launchers (defined next to their kernels).
cudaError_t launch_qk_norm_rope_cache(const ProducerParams &p, bool f16, int num_sms,
                                      cudaStream_t st);
cudaError_t launch_reshape_and_cache(const elem16 *key, const elem16 *value,
                                     elem16 *k_pool, elem16 *v_pool,
                                     const int64_t *slot_mapping, int64_t num_tokens,
                                     int64_t key_stride, int64_t value_stride, int Hkv,
                                     uint32_t num_blocks, int bs_shift, unsigned *err,
                                     cudaStream_t st, int head_size = kHeadSize);
cudaError_t launch_reshape_and_cache_fp8(const elem16 *key, const elem16 *value, uint8_t *k_pool,
                                         uint8_t *v_pool, const int64_t *slot_mapping,
                                         int64_t num_tokens, int64_t key_stride,
                                         int64_t value_stride, int Hkv, uint32_t num_blocks,
                                         int bs_shift, float k_scale, float v_scale, bool f16,
                                         unsigned *err, unsigned *special_flag, cudaStream_t st);
cudaError_t launch_copy_blocks(elem16 *k_pool, elem16 *v_pool,
                               const int64_t *mapping, int64_t num_pairs, int64_t bytes_per_block,
                               uint32_t num_blocks, unsigned *err, cudaStream_t st);
// Block moves between the pools and per-block host (pinned, device-mapped) buffers.
// to_host != 0: pool -> host.  ids/host_k/host_v are readable by the device.
cudaError_t launch_swap_blocks(elem16 *k_pool, elem16 *v_pool, const uint32_t *ids,
                               char *const *host_k, char *const *host_v, int num, int64_t bytes_per_block,
                               int to_host, uint32_t num_blocks, unsigned *err, cudaStream_t st);
// Up to three host->device (or any) copies in one launch; sizes multiples of 4 bytes,
// sources and destinations 16-byte aligned.
struct StageCopy {
  const void *src[3];
  void *dst[3];
  size_t bytes[3];
};
cudaError_t launch_stage_copy(const StageCopy &a, cudaStream_t st);
// Head gather over peer memory (cache_kernels.cu).
constexpr int kMaxPeers = 8;
struct PeerGather {
  const void *local_out;          // [num_tokens, row_bytes_local] contiguous
  void *peer_out[kMaxPeers];      // every rank's [num_tokens, world * row_bytes_local] buffer
  unsigned *peer_flags[kMaxPeers];  // every rank's flag words, one per writer
  unsigned *counter;              // zero-initialised device word of the caller
  int64_t num_tokens;
  int32_t row_bytes_local;        // heads_local * head_size * 2, a multiple of 16
  int32_t world, rank;
  unsigned epoch;
};
cudaError_t launch_peer_gather(const PeerGather &a, cudaStream_t st);
cudaError_t launch_peer_wait(const unsigned *my_flags, int world, unsigned epoch, unsigned *err,
                             cudaStream_t st);
// An encoded tensor map (opaque 128 bytes; what the driver calls CUtensorMap).
struct alignas(64) TensorMapBlob {
  unsigned char bytes[128];
};
// Maps over the K and the V pool of one layer that fetch one 16-token unit of a
// (block, kv head) chunk; what the split-KV kernel needs when bs_shift != 0.
struct alignas(64) UnitMaps {
  TensorMapBlob k, v;
};
cudaError_t encode_unit_maps(UnitMaps *out, const void *k_pool, const void *v_pool,
                             uint64_t num_chunks, int block_size, bool fp8);
// Split-KV kernel over every sequence whose q_len*G <= p.max_cols, then the merge.
// `maps` may be null when p.bs_shift == 0.
cudaError_t launch_splitkv_attention(const AttnParams &p, int num_ctas, cudaStream_t st,
                                     const UnitMaps *maps = nullptr);
size_t splitkv_workspace_bytes(int num_ctas);
int splitkv_max_cols();
// CTAs per SM of the narrow (8-column) kernel: 2 on an FP8 cache and on small heads
int splitkv_narrow_ctas_per_sm(int head_size, bool fp8);
int splitkv_max_cols_for(int head_size);
cudaError_t splitkv_configure();  // opt-in shared memory sizes, once per device
// Library-resident scratch for callers that cannot allocate (see splitkv_attention.cu).
int splitkv_static_max_ctas();
cudaError_t splitkv_static_scratch(int device, float **out);
// Tile kernel for long-query sequences; work list built by the caller.
struct TileWork {
  int32_t seq;       // sequence index
  int32_t kv_head;   // kv head
  int32_t q_begin;   // first query (within the sequence) of this tile
  int32_t q_count;   // queries in this tile
};
cudaError_t tile_encode_v_map(TensorMapBlob *out, const void *v_pool, uint64_t num_chunks,
                              int block_size);
cudaError_t launch_tile_attention(const AttnParams &p, const TileWork *work_dev, int num_work,
                                  const TensorMapBlob *v_map, cudaStream_t st);
cudaError_t tile_configure();
int tile_queries_per_cta(int G);
// The same for 16-bit pools of 16-token blocks with every KV operand fetched by TMA
// (tile_attention_tc64.cu); same work list, same rows per CTA.
cudaError_t tile64_encode_k_map(TensorMapBlob *out, const void *k_pool, uint64_t num_chunks);
cudaError_t launch_tile64_attention(const AttnParams &p, const TileWork *work_dev, int num_work,
                                    const TensorMapBlob *k_map, const TensorMapBlob *v_map, cudaStream_t st);
cudaError_t tile64_configure();
int tile64_queries_per_cta(int G);

extern unsigned long long g_launch_count;  // host counter of kernel launches

}  // namespace pa
