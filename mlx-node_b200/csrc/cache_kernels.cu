// KV block write (reshape_and_cache) and block copy (copy_blocks) for sm_100a.
//
// Semantics: crates/mlx-paged-attn/metal/cache/reshape_and_cache.metal:58-97 and
// crates/mlx-paged-attn/metal/cache/copy_blocks.metal:6-36.  Both are pure
// index arithmetic over 16-bit patterns, so results are bit-exact.
#include <algorithm>

#include "pa_common.cuh"

namespace pa {

unsigned long long g_launch_count = 0;

// One CTA stages up to 16 consecutive tokens of one KV head in shared memory and
// writes them out with the token index fastest across threads.  For a prefill
// chunk (consecutive slots of one block) the 16-byte K pieces of neighbouring
// tokens and the 2-byte V elements of neighbouring tokens are adjacent in the
// pool, so a warp's stores fill whole 32-byte sectors; for decode (one token per
// sequence) the stores are scattered, as the layout dictates.
constexpr int kTokPerCta = 16;
constexpr int kVPad = 2;  // bf16 elements of row padding: 65-word rows, conflict-free

template <int HD>
__global__ void __launch_bounds__(256)
reshape_and_cache_kernel(const elem16 *__restrict__ key,
                         const elem16 *__restrict__ value,
                         elem16 *__restrict__ k_pool, elem16 *__restrict__ v_pool,
                         const int64_t *__restrict__ slot_mapping, int64_t num_tokens,
                         int64_t key_stride, int64_t value_stride, int Hkv, uint32_t num_blocks,
                         int bs_shift, unsigned *err) {
  constexpr int kPieces = HD / 8;  // 16-byte pieces of one token's row of one head
  __shared__ uint4 k_s[kTokPerCta][kPieces];
  __shared__ __align__(16) uint16_t v_s[kTokPerCta][HD + kVPad];
  __shared__ int64_t slot_s[kTokPerCta];

  // the attention kernel that follows may set up (it reads no pool data before its
  // own griddepcontrol.wait)
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int h = blockIdx.y;
  const int64_t t0 = (int64_t)blockIdx.x * kTokPerCta;
  const int tid = threadIdx.x;
  const int bs_log = 4 + bs_shift, bs = 1 << bs_log;  // tokens of a pool block
  const int64_t n_slots = (int64_t)num_blocks << bs_log;

  if (tid < kTokPerCta) {
    int64_t s = -1;
    if (t0 + tid < num_tokens) {
      s = slot_mapping[t0 + tid];
      if (s >= n_slots) {
        atomicOr(err, kErrSlotRange);
        s = -1;
      }
    }
    slot_s[tid] = s;
  }
  // Stage: 16 tokens x HD/8 pieces of 16 B for K and for V; thread -> (token, piece).
  for (int i = tid; i < kTokPerCta * kPieces; i += 256) {
    const int tok = i / kPieces, piece = i % kPieces;
    if (t0 + tok < num_tokens) {
      const uint4 kv = *reinterpret_cast<const uint4 *>(key + (t0 + tok) * key_stride +
                                                        (int64_t)h * HD + piece * 8);
      const uint4 vv = *reinterpret_cast<const uint4 *>(value + (t0 + tok) * value_stride +
                                                        (int64_t)h * HD + piece * 8);
      k_s[tok][piece] = kv;
      uint32_t *vd = reinterpret_cast<uint32_t *>(&v_s[tok][piece * 8]);
      vd[0] = vv.x; vd[1] = vv.y; vd[2] = vv.z; vd[3] = vv.w;
    }
  }
  __syncthreads();

  // K: piece c of token `tok` goes to chunk offset c*BS*8 + off*8 (elements).
  for (int i = tid; i < kTokPerCta * kPieces; i += 256) {
    const int tok = i & 15, c = i >> 4;
    const int64_t slot = slot_s[tok];
    if (slot >= 0) {
      const int64_t blk = slot >> bs_log;
      const int off = (int)(slot & (bs - 1));
      elem16 *dst = k_pool + (((blk * Hkv + h) * (int64_t)HD) << bs_log) + c * (bs * 8) + off * 8;
      *reinterpret_cast<uint4 *>(dst) = k_s[tok][c];
    }
  }
  // V: element d of token `tok` goes to chunk offset d*BS + off.
  for (int e = tid; e < kTokPerCta * HD; e += 256) {
    const int tok = e & 15, d = e >> 4;
    const int64_t slot = slot_s[tok];
    if (slot >= 0) {
      const int64_t blk = slot >> bs_log;
      const int off = (int)(slot & (bs - 1));
      reinterpret_cast<uint16_t *>(v_pool)[(((blk * Hkv + h) * (int64_t)HD) << bs_log) + d * bs + off] =
          v_s[tok][d];
    }
  }
}

cudaError_t launch_reshape_and_cache(const elem16 *key, const elem16 *value,
                                     elem16 *k_pool, elem16 *v_pool,
                                     const int64_t *slot_mapping, int64_t num_tokens,
                                     int64_t key_stride, int64_t value_stride, int Hkv,
                                     uint32_t num_blocks, int bs_shift, unsigned *err,
                                     cudaStream_t st, int head_size) {
  if (num_tokens <= 0) return cudaSuccess;
  const int64_t groups = (num_tokens + kTokPerCta - 1) / kTokPerCta;
  // grid.x is 31-bit; a write of more than 2^31*16 tokens is not a real call.
  dim3 grid((unsigned)groups, (unsigned)Hkv);
  auto go = [&](auto kernel) {
    kernel<<<grid, 256, 0, st>>>(key, value, k_pool, v_pool, slot_mapping, num_tokens, key_stride,
                                 value_stride, Hkv, num_blocks, bs_shift, err);
  };
  switch (head_size) {
    case 32: go(reshape_and_cache_kernel<32>); break;
    case 64: go(reshape_and_cache_kernel<64>); break;
    case 80: go(reshape_and_cache_kernel<80>); break;
    case 96: go(reshape_and_cache_kernel<96>); break;
    case 112: go(reshape_and_cache_kernel<112>); break;
    case 120: go(reshape_and_cache_kernel<120>); break;
    case kHeadSize: go(reshape_and_cache_kernel<kHeadSize>); break;
    case 192: go(reshape_and_cache_kernel<192>); break;
    case 256: go(reshape_and_cache_kernel<256>); break;
    default: return cudaErrorInvalidValue;
  }
  __atomic_fetch_add(&g_launch_count, 1ull, __ATOMIC_RELAXED);
  return cudaGetLastError();
}

// ---- FP8 (E4M3) cache write -----------------------------------------------------
// Encoder of the reference's byte format, crates/mlx-paged-attn/metal/float8.metal:63-121:
// bias 7, exponent field 15 is infinity / NaN (largest finite value 240).  Normal range:
// round to nearest even, overflow to the infinity code.  Below it: magnitudes under 2^-9
// become zero, the rest round half up, and a
// value that would round up to the smallest normal number comes out as zero (the result is
// masked to the three mantissa bits).  Inputs of magnitude 256 and above miss the normal
// range test and take the below-normal branch as well; for magnitudes below 16384 that
// yields the low three bits of a shifted mantissa, which is kept as is so that the bytes
// match; above, where the reference's shift count turns negative, the infinity code.
__device__ __forceinline__ uint32_t fp8_e4m3_encode_ref(float f) {
  const uint32_t bits = __float_as_uint(f);
  const uint32_t s = (bits >> 31) << 7, a = bits & 0x7FFFFFFFu;
  if (a >= 0x7F800000u) return s | 0x78u | (a != 0x7F800000u);
  const int e8 = (int)(a >> 23) - 120;
  const uint32_t m = a & 0x7FFFFFu;
  if (e8 >= 1 && e8 <= 14) {
    uint32_t mant = m >> 20;
    mant += ((m >> 19) & 1u) & (((m & 0x7FFFFu) != 0u) | (mant & 1u));
    uint32_t e = (uint32_t)e8;
    if (mant >> 3) {
      mant = 0;
      if (++e > 14u) return s | 0x78u;
    }
    return s | (e << 3) | mant;
  }
  if (e8 < -2) return s;
  const int rshift = 21 - e8;
  if (rshift < 1) return s | 0x78u;
  return s | ((((0x800000u | m) + (1u << (rshift - 1))) >> rshift) & 7u);
}

// Eight 16-bit elements (one uint4) -> eight bytes: x / scale in fp32 (IEEE division),
// rounded to the input type, then encoded
// (crates/mlx-paged-attn/metal/cache/reshape_and_cache.metal:88-92).
template <bool F16>
__device__ __forceinline__ uint2 quantise8(uint4 v, float scale) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  uint32_t out[2] = {0u, 0u};
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const uint32_t bits16 = (w[i >> 1] >> ((i & 1) * 16)) & 0xffffu;
    float x;
    if (F16) asm("cvt.f32.f16 %0, %1;" : "=f"(x) : "h"((uint16_t)bits16));
    else x = __uint_as_float(bits16 << 16);
    const uint32_t r16 = to_elem<F16>(__fdiv_rn(x, scale));
    float y;
    if (F16) asm("cvt.f32.f16 %0, %1;" : "=f"(y) : "h"((uint16_t)r16));
    else y = __uint_as_float(r16 << 16);
    out[i >> 2] |= fp8_e4m3_encode_ref(y) << ((i & 3) * 8);
  }
  return make_uint2(out[0], out[1]);
}

// Same decomposition as reshape_and_cache_kernel; the pools hold bytes, K as
// [block][head][D/16][BS][16] and V as [block][head][D][BS]
// (crates/mlx-paged-attn/src/cache_engine.rs:66-90).
template <bool F16>
__global__ void __launch_bounds__(256)
reshape_and_cache_fp8_kernel(const elem16 *__restrict__ key, const elem16 *__restrict__ value,
                             uint8_t *__restrict__ k_pool, uint8_t *__restrict__ v_pool,
                             const int64_t *__restrict__ slot_mapping, int64_t num_tokens,
                             int64_t key_stride, int64_t value_stride, int Hkv,
                             uint32_t num_blocks, int bs_shift, float k_scale, float v_scale,
                             unsigned *err, unsigned *special_flag) {
  __shared__ uint2 k_s[kTokPerCta][kHeadSize / 8];                   // 16 x 128 B
  __shared__ __align__(8) uint8_t v_s[kTokPerCta][kHeadSize + 8];    // padded rows
  __shared__ int64_t slot_s[kTokPerCta];

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int h = blockIdx.y;
  const int64_t t0 = (int64_t)blockIdx.x * kTokPerCta;
  const int tid = threadIdx.x;
  const int bs_log = 4 + bs_shift, bs = 1 << bs_log;  // tokens of a pool block
  const int64_t n_slots = (int64_t)num_blocks << bs_log;
  if (tid < kTokPerCta) {
    int64_t s = -1;
    if (t0 + tid < num_tokens) {
      s = slot_mapping[t0 + tid];
      if (s >= n_slots) {
        atomicOr(err, kErrSlotRange);
        s = -1;
      }
    }
    slot_s[tid] = s;
  }
  {
    const int tok = tid >> 4, piece = tid & 15;
    if (t0 + tok < num_tokens) {
      const uint4 kv = *reinterpret_cast<const uint4 *>(key + (t0 + tok) * key_stride +
                                                        (int64_t)h * kHeadSize + piece * 8);
      const uint4 vv = *reinterpret_cast<const uint4 *>(value + (t0 + tok) * value_stride +
                                                        (int64_t)h * kHeadSize + piece * 8);
      const uint2 kq = quantise8<F16>(kv, k_scale), vq = quantise8<F16>(vv, v_scale);
      k_s[tok][piece] = kq;
      *reinterpret_cast<uint2 *>(&v_s[tok][piece * 8]) = vq;
      // An exponent-15 byte (overflow, infinity or NaN going in) switches the attention
      // kernels of this cache to their exact decoding variant.  Tokens whose slot is
      // skipped count too; the flag only ever errs on the slow side.
      auto has15 = [](uint32_t w) { return (((w & 0x78787878u) + 0x08080808u) & 0x80808080u) != 0u; };
      if (has15(kq.x) | has15(kq.y) | has15(vq.x) | has15(vq.y)) atomicOr(special_flag, 1u);
    }
  }
  __syncthreads();
  // a (block, head) chunk is kHeadSize * bs bytes
  if (tid < 128) {  // K: 16 bytes of (token, d/16)
    const int tok = tid & 15, c = tid >> 4;
    const int64_t slot = slot_s[tok];
    if (slot >= 0) {
      const int64_t blk = slot >> bs_log;
      const int off = (int)(slot & (bs - 1));
      uint8_t *dst = k_pool + (((blk * Hkv + h) * (int64_t)kHeadSize) << bs_log) + c * (bs * 16) +
                     off * 16;
      *reinterpret_cast<uint4 *>(dst) = make_uint4(k_s[tok][2 * c].x, k_s[tok][2 * c].y,
                                                   k_s[tok][2 * c + 1].x, k_s[tok][2 * c + 1].y);
    }
  }
  for (int e = tid; e < kTokPerCta * kHeadSize; e += 256) {
    const int tok = e & 15, d = e >> 4;
    const int64_t slot = slot_s[tok];
    if (slot >= 0) {
      const int64_t blk = slot >> bs_log;
      const int off = (int)(slot & (bs - 1));
      v_pool[(((blk * Hkv + h) * (int64_t)kHeadSize) << bs_log) + d * bs + off] = v_s[tok][d];
    }
  }
}

cudaError_t launch_reshape_and_cache_fp8(const elem16 *key, const elem16 *value, uint8_t *k_pool,
                                         uint8_t *v_pool, const int64_t *slot_mapping,
                                         int64_t num_tokens, int64_t key_stride,
                                         int64_t value_stride, int Hkv, uint32_t num_blocks,
                                         int bs_shift, float k_scale, float v_scale, bool f16,
                                         unsigned *err, unsigned *special_flag, cudaStream_t st) {
  if (num_tokens <= 0) return cudaSuccess;
  const int64_t groups = (num_tokens + kTokPerCta - 1) / kTokPerCta;
  dim3 grid((unsigned)groups, (unsigned)Hkv);
  if (f16)
    reshape_and_cache_fp8_kernel<true><<<grid, 256, 0, st>>>(
        key, value, k_pool, v_pool, slot_mapping, num_tokens, key_stride, value_stride, Hkv,
        num_blocks, bs_shift, k_scale, v_scale, err, special_flag);
  else
    reshape_and_cache_fp8_kernel<false><<<grid, 256, 0, st>>>(
        key, value, k_pool, v_pool, slot_mapping, num_tokens, key_stride, value_stride, Hkv,
        num_blocks, bs_shift, k_scale, v_scale, err, special_flag);
  __atomic_fetch_add(&g_launch_count, 1ull, __ATOMIC_RELAXED);
  return cudaGetLastError();
}

// One CTA per (pair, 4 KB piece): K piece then V piece, 16 bytes per thread.
// Pairs are independent unless a destination is also a source of a later pair;
// the reference processes pairs in parallel as well (one threadgroup per pair).
__global__ void __launch_bounds__(256)
copy_blocks_kernel(elem16 *__restrict__ k_pool, elem16 *__restrict__ v_pool,
                   const int64_t *__restrict__ mapping, int64_t bytes_per_block,
                   uint32_t num_blocks, unsigned *err) {
  const int64_t pair = blockIdx.x;
  const int64_t src = mapping[2 * pair], dst = mapping[2 * pair + 1];
  if (src < 0 || dst < 0 || src >= (int64_t)num_blocks || dst >= (int64_t)num_blocks) {
    if (threadIdx.x == 0) atomicOr(err, kErrBlockRange);
    return;
  }
  const int64_t piece = (int64_t)blockIdx.y * 4096 + threadIdx.x * 16;
  if (piece >= bytes_per_block) return;
  const char *ks = reinterpret_cast<const char *>(k_pool) + src * bytes_per_block + piece;
  char *kd = reinterpret_cast<char *>(k_pool) + dst * bytes_per_block + piece;
  const char *vs = reinterpret_cast<const char *>(v_pool) + src * bytes_per_block + piece;
  char *vd = reinterpret_cast<char *>(v_pool) + dst * bytes_per_block + piece;
  *reinterpret_cast<uint4 *>(kd) = *reinterpret_cast<const uint4 *>(ks);
  *reinterpret_cast<uint4 *>(vd) = *reinterpret_cast<const uint4 *>(vs);
}

cudaError_t launch_copy_blocks(elem16 *k_pool, elem16 *v_pool,
                               const int64_t *mapping, int64_t num_pairs, int64_t bytes_per_block,
                               uint32_t num_blocks, unsigned *err, cudaStream_t st) {
  if (num_pairs <= 0) return cudaSuccess;
  dim3 grid((unsigned)num_pairs, (unsigned)((bytes_per_block + 4095) / 4096));
  copy_blocks_kernel<<<grid, 256, 0, st>>>(k_pool, v_pool, mapping, bytes_per_block, num_blocks,
                                           err);
  __atomic_fetch_add(&g_launch_count, 1ull, __ATOMIC_RELAXED);
  return cudaGetLastError();
}

// Ingest of a step's small inputs from pinned host memory: up to three segments copied
// by one launch, the device reading the host pages over PCIe itself (one launch instead
// of one DMA operation per buffer).  Segment sizes are multiples of 4 bytes.
__global__ void __launch_bounds__(256)
stage_copy_kernel(StageCopy a) {
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t nthreads = (size_t)gridDim.x * blockDim.x;
#pragma unroll
  for (int k = 0; k < 3; k++) {
    const size_t n16 = a.bytes[k] / 16, tail = (a.bytes[k] % 16) / 4;
    const uint4 *s16 = static_cast<const uint4 *>(a.src[k]);
    uint4 *d16 = static_cast<uint4 *>(a.dst[k]);
    for (size_t i = tid; i < n16; i += nthreads) d16[i] = s16[i];
    if (tid < tail)
      static_cast<uint32_t *>(a.dst[k])[n16 * 4 + tid] =
          static_cast<const uint32_t *>(a.src[k])[n16 * 4 + tid];
  }
}

cudaError_t launch_stage_copy(const StageCopy &a, cudaStream_t st) {
  size_t total = 0;
  for (int k = 0; k < 3; k++) total += a.bytes[k] / 16 + 1;
  const unsigned blocks = (unsigned)std::min<size_t>((total + 255) / 256, 1024);
  stage_copy_kernel<<<blocks, 256, 0, st>>>(a);
  __atomic_fetch_add(&g_launch_count, 1ull, __ATOMIC_RELAXED);
  return cudaGetLastError();
}

// ---- head gather over peer memory ------------------------------------------------
// With the KV heads sharded over the GPUs of a box, rank r holds out[:, r*hl:(r+1)*hl, :].
// A consumer that wants every head on every rank gets them by plain 16-byte stores into
// each rank's full-width buffer (peer pointers: NVLink through NVSwitch), followed by one
// flag per (writer, reader) pair written with release semantics at system scope once all
// of the writer's stores are out.  No library collective, no multicast.
__global__ void __launch_bounds__(256)
scatter_heads_kernel(PeerGather a) {
  const size_t vec_local = (size_t)a.row_bytes_local / 16;   // 16-byte vectors per local row
  const size_t vec_full = vec_local * a.world;
  const size_t total = (size_t)a.num_tokens * vec_local * a.world;
  const uint4 *src = static_cast<const uint4 *>(a.local_out);
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    const size_t per_peer = (size_t)a.num_tokens * vec_local;
    const int w = (int)(i / per_peer);
    const size_t r = i - (size_t)w * per_peer;
    const size_t t = r / vec_local, v = r - t * vec_local;
    static_cast<uint4 *>(a.peer_out[w])[t * vec_full + (size_t)a.rank * vec_local + v] = src[r];
  }
  // last block out publishes: every block fences its stores, then counts itself
  __threadfence_system();
  __syncthreads();
  __shared__ unsigned last;
  if (threadIdx.x == 0) last = atomicAdd(a.counter, 1u) == gridDim.x - 1 ? 1u : 0u;
  __syncthreads();
  if (last) {
    if (threadIdx.x < (unsigned)a.world) {
      __threadfence_system();
      asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(a.peer_flags[threadIdx.x] + a.rank),
                   "r"(a.epoch)
                   : "memory");
    }
    if (threadIdx.x == 0) *a.counter = 0u;
  }
}

// Reader side: until every writer's flag has reached `epoch`, for about a second at most;
// a flag that never comes sets the time-out bit instead of hanging the stream.
__global__ void wait_heads_kernel(const unsigned *my_flags, int world, unsigned epoch, unsigned *err) {
  const int w = threadIdx.x;
  if (w >= world) return;
  const long long t0 = clock64();
  for (;;) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(my_flags + w) : "memory");
    if ((int)(v - epoch) >= 0) return;
    if (clock64() - t0 > (1ll << 31)) {
      atomicOr(err, kErrTimeout);
      return;
    }
  }
}

cudaError_t launch_peer_wait(const unsigned *my_flags, int world, unsigned epoch, unsigned *err,
                             cudaStream_t st) {
  wait_heads_kernel<<<1, 32, 0, st>>>(my_flags, world, epoch, err);
  __atomic_fetch_add(&g_launch_count, 1ull, __ATOMIC_RELAXED);
  return cudaGetLastError();
}

cudaError_t launch_peer_gather(const PeerGather &a, cudaStream_t st) {
  const size_t total = (size_t)a.num_tokens * (a.row_bytes_local / 16) * a.world;
  // An empty step still publishes this rank's flags (one block with nothing to store):
  // the other ranks wait for every writer's epoch.
  const unsigned blocks = (unsigned)std::max<size_t>(1, std::min<size_t>((total + 255) / 256, 296));
  scatter_heads_kernel<<<blocks, 256, 0, st>>>(a);
  __atomic_fetch_add(&g_launch_count, 1ull, __ATOMIC_RELAXED);
  return cudaGetLastError();
}

// Swap: one CTA per (block, 4 KB piece), 16 bytes per thread, K then V.  The host side
// of each block is pinned memory mapped into the device's address space, so the kernel
// itself moves the bytes over PCIe (one launch for any number of blocks).
__global__ void __launch_bounds__(256)
swap_blocks_kernel(elem16 *__restrict__ k_pool, elem16 *__restrict__ v_pool,
                   const uint32_t *__restrict__ ids, char *const *__restrict__ host_k,
                   char *const *__restrict__ host_v, int64_t bytes_per_block, int to_host,
                   uint32_t num_blocks, unsigned *err) {
  const uint32_t id = ids[blockIdx.x];
  if (id >= num_blocks) {
    if (threadIdx.x == 0) atomicOr(err, kErrBlockRange);
    return;
  }
  const int64_t piece = (int64_t)blockIdx.y * 4096 + threadIdx.x * 16;
  if (piece >= bytes_per_block) return;
  char *kd = reinterpret_cast<char *>(k_pool) + (int64_t)id * bytes_per_block + piece;
  char *vd = reinterpret_cast<char *>(v_pool) + (int64_t)id * bytes_per_block + piece;
  char *kh = host_k[blockIdx.x] + piece, *vh = host_v[blockIdx.x] + piece;
  if (to_host) {
    *reinterpret_cast<uint4 *>(kh) = *reinterpret_cast<const uint4 *>(kd);
    *reinterpret_cast<uint4 *>(vh) = *reinterpret_cast<const uint4 *>(vd);
  } else {
    *reinterpret_cast<uint4 *>(kd) = *reinterpret_cast<const uint4 *>(kh);
    *reinterpret_cast<uint4 *>(vd) = *reinterpret_cast<const uint4 *>(vh);
  }
}

cudaError_t launch_swap_blocks(elem16 *k_pool, elem16 *v_pool, const uint32_t *ids,
                               char *const *host_k, char *const *host_v, int num, int64_t bytes_per_block,
                               int to_host, uint32_t num_blocks, unsigned *err, cudaStream_t st) {
  if (num <= 0) return cudaSuccess;
  dim3 grid((unsigned)num, (unsigned)((bytes_per_block + 4095) / 4096));
  swap_blocks_kernel<<<grid, 256, 0, st>>>(k_pool, v_pool, ids, host_k, host_v, bytes_per_block, to_host,
                                           num_blocks, err);
  __atomic_fetch_add(&g_launch_count, 1ull, __ATOMIC_RELAXED);
  return cudaGetLastError();
}

}  // namespace pa
