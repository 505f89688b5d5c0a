/*
 * paged_attn_b200 — C ABI of the B200 (sm_100a) paged-attention library.
 *
 * Two tiers.
 *
 * Tier 1 keeps the seven entry points of the reference's own FFI for this
 * path, with the same names, argument order and ownership rules
 * (crates/mlx-sys/src/lib.rs:689-803, implemented by
 * crates/mlx-sys/src/mlx.cpp:3796-4258).  The opaque `mlx_array` the reference
 * passes across that boundary is, in this library, a small descriptor of a
 * tensor in device memory (pa_array_* below build and inspect one).
 *
 * Tier 2 (`pa_*`) is what tier 1 is built on: plain device pointers, explicit
 * sizes and strides, an explicit cudaStream_t (passed as void*), a status code
 * from every call.  It is what a CUDA port of the crate's `metal` module
 * (crates/mlx-paged-attn/src/metal/mod.rs:29-44) binds.
 *
 * Tensors are f16 (dtype code 0, the reference's default) or bf16 (code 1); q,
 * k, v and out of a call have the cache's dtype.  f32 (code 2) is not built.
 * Pool layout is the
 * reference's (crates/mlx-paged-attn/src/cache_engine.rs:58-106):
 *   key   [num_blocks, num_kv_heads, head_size/8, block_size, 8]
 *   value [num_blocks, num_kv_heads, head_size, block_size]
 *
 * Threading: the library keeps no global mutable state except a per-thread
 * error string and a per-thread current device/stream for tier 1.  One cache
 * handle is used by one stream at a time; different handles may be used
 * concurrently.  Every launch is asynchronous on the given stream.
 * No entry point aborts, traps or throws across the boundary.
 */
#ifndef PAGED_ATTN_B200_H_
#define PAGED_ATTN_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status ------------------------------------------------------------- */
typedef int32_t pa_status;
enum {
  PA_OK = 0,
  PA_ERR_INVALID_ARG = 1,  /* null pointer, bad size/stride/alignment          */
  PA_ERR_UNSUPPORTED = 2,  /* f32, or a combination of head size, block size and FP8 that is not built */
  PA_ERR_OOM = 3,          /* device allocation failed                         */
  PA_ERR_OUT_OF_RANGE = 4, /* a block id or slot outside the pool was seen     */
  PA_ERR_TIMEOUT = 5,      /* a bounded device-side wait ran out               */
  PA_ERR_CUDA = 6,         /* a CUDA runtime call failed                       */
  PA_ERR_NCCL = 7
};
/* Text of the last error raised on the calling thread ("" if none).  The
 * reference reports errors as Result<_, String> (crate) or null / silent
 * return (crates/mlx-sys/src/mlx.cpp:3824, 3907-3908, 4051-4053).             */
const char *pa_last_error_string(void);
/* Library version: major*10000 + minor*100 + patch. */
int32_t pa_version(void);

/* ---- configuration and cache handle -------------------------------------- */
/* Same six u32 fields as the reference (crates/mlx-sys/src/lib.rs:690-705,
 * crates/mlx-sys/src/mlx.cpp:3796-3803). dtype: 0 f16, 1 bf16, 2 f32.
 * Built: head_size 128 with every block size the reference accepts (8, 16, 32;
 * crates/mlx-paged-attn/src/config.rs:40-45) and dtype 0 or 1; the other head
 * sizes of config.rs:47-50 (32, 64, 80, 96, 112, 120, 192, 256) with block_size
 * 16 - and, up to head size 120, with the reference's default block_size 32 -
 * dtype 0 or 1, no FP8 cache (KV write, decode and multi-token attention;
 * chunks of more than 24 / G query tokens - 16 / G with head size 192, 8 / G with
 * 256 - are served in pieces and need context_lens_host, the fused producer
 * launch is refused, pa_decode_step runs its two kernels).  dtype 2 returns
 * PA_ERR_UNSUPPORTED.  An FP8 cache needs block_size 16 or 32, as in the
 * reference (config.rs:71-76).                                                 */
typedef struct PagedAttnConfig {
  uint32_t block_size;
  uint32_t num_blocks;
  uint32_t head_size;
  uint32_t num_kv_heads;
  uint32_t num_layers;
  uint32_t dtype;
} PagedAttnConfig;

typedef struct PagedAttnCache PagedAttnCache; /* opaque */
typedef struct mlx_array mlx_array;           /* opaque device-tensor view */

/* ---- tier 1: the reference's FFI names ----------------------------------- */
/* crates/mlx-sys/src/lib.rs:721, mlx.cpp:3823-3867.  Allocates zero-filled
 * per-layer K and V pools on the calling thread's current device
 * (pa_set_device).  Null on failure (see pa_last_error_string).              */
PagedAttnCache *mlx_paged_attn_create_cache(const PagedAttnConfig *config);
/* crates/mlx-sys/src/lib.rs:724, mlx.cpp:3870-3872. */
void mlx_paged_attn_free_cache(PagedAttnCache *cache);
/* crates/mlx-sys/src/lib.rs:734-750, mlx.cpp:3875-3884.  Returns a NEW handle
 * that views the layer's pool; the caller deletes it with mlx_array_delete
 * (as crates/mlx-core/src/transformer/paged_attention.rs:182-186 does).       */
mlx_array *mlx_paged_attn_get_key_cache(PagedAttnCache *cache, uint32_t layer_idx);
mlx_array *mlx_paged_attn_get_value_cache(PagedAttnCache *cache, uint32_t layer_idx);
/* crates/mlx-sys/src/lib.rs:760-766, mlx.cpp:3900-4012.
 * keys/values [num_tokens, num_kv_heads, head_size] in the cache dtype, slot_mapping
 * [num_tokens] int64 (a negative slot is skipped).  Silent no-op on null or
 * bad layer, like the reference; the reason is left in the error string.      */
void mlx_paged_attn_reshape_and_cache(PagedAttnCache *cache, uint32_t layer_idx,
                                      mlx_array *keys, mlx_array *values,
                                      mlx_array *slot_mapping);
/* crates/mlx-sys/src/lib.rs:782-791, mlx.cpp:4041-4162.
 * queries [num_seqs, num_heads, head_size]; block_tables int32
 * [num_seqs, max_blocks]; context_lens int32 [num_seqs].  Returns a new
 * [num_seqs, num_heads, head_size] array that owns its device memory, or null. */
mlx_array *mlx_paged_attn_forward(mlx_array *queries, mlx_array *key_cache,
                                  mlx_array *value_cache, mlx_array *block_tables,
                                  mlx_array *context_lens, float scale,
                                  uint32_t block_size, uint32_t max_context_len);
/* crates/mlx-sys/src/lib.rs:799-803, mlx.cpp:4170-4258.  block_mapping int64,
 * [num_pairs, 2] or flat [2*num_pairs], pairs are (src, dst).                 */
void mlx_paged_attn_copy_blocks(PagedAttnCache *cache, uint32_t layer_idx,
                                mlx_array *block_mapping);

/* The array shim standing in for the reference's mlx_array on this path.
 * dtype codes: 0 f16, 1 bf16, 2 f32, 3 int32, 4 int64, 5 uint32.
 * (crates/mlx-sys/src/lib.rs:332-355 declares the shape/dtype/delete calls.)  */
mlx_array *pa_array_from_device(void *device_ptr, int32_t dtype, const int64_t *shape,
                                size_t ndim);
/* Copies host data into a new device array the handle owns
 * (the role of crates/mlx-sys/src/lib.rs:19-28 mlx_array_from_int32/int64/...). */
mlx_array *pa_array_from_host(const void *host_ptr, int32_t dtype, const int64_t *shape,
                              size_t ndim);
void *pa_array_data(mlx_array *a);
size_t mlx_array_ndim(mlx_array *handle);
void mlx_array_shape(mlx_array *handle, int64_t *out);
int32_t mlx_array_dtype(mlx_array *handle);
void mlx_array_delete(mlx_array *arr);
/* Device and stream tier 1 runs on, per calling thread (default: device 0,
 * the legacy default stream).                                                 */
pa_status pa_set_device(int32_t device);
pa_status pa_set_stream(void *cuda_stream);

/* ---- tier 2: raw device pointers ------------------------------------------ */
/* Allocate (and zero) the pools on `device`.  Replaces
 * CacheEngine::initialize (crates/mlx-paged-attn/src/cache_engine.rs:58-106). */
pa_status pa_cache_create(const PagedAttnConfig *config, int32_t device,
                          PagedAttnCache **out_cache);
/* Wrap pools the caller owns: key_ptrs/value_ptrs are num_layers device
 * pointers, each 128-byte aligned, laid out as above.  Nothing is copied or
 * freed by the library.                                                       */
pa_status pa_cache_wrap(const PagedAttnConfig *config, int32_t device,
                        void *const *key_ptrs, void *const *value_ptrs,
                        PagedAttnCache **out_cache);
pa_status pa_cache_free(PagedAttnCache *cache);
/* Borrowed pointers into the pools (crates/mlx-paged-attn/src/cache_engine.rs
 * key_cache()/value_cache() accessors). Null on bad arguments.                */
void *pa_cache_key_ptr(PagedAttnCache *cache, uint32_t layer_idx);
void *pa_cache_value_ptr(PagedAttnCache *cache, uint32_t layer_idx);
pa_status pa_cache_get_config(const PagedAttnCache *cache, PagedAttnConfig *out);
/* FP8 (E4M3) KV cache: PagedAttentionConfig::use_fp8_cache
 * (crates/mlx-paged-attn/src/config.rs:23-26, 87-88) as CacheEngine::initialize lays
 * it out (crates/mlx-paged-attn/src/cache_engine.rs:66-90): one byte per element,
 * key pool [num_blocks, num_kv_heads, head_size/16, block_size, 16], value pool
 * [num_blocks, num_kv_heads, head_size, block_size].  config->dtype (0 f16, 1 bf16)
 * is then the type of the queries, outputs and of the keys/values given to
 * pa_reshape_and_cache.  The byte format is the reference's
 * (crates/mlx-paged-attn/metal/float8.metal:11-33, 63-121; largest finite value
 * 240).  The write stores encode(T(x / scale)) (reshape_and_cache.metal:88-92), the
 * attention reads decode(byte) * scale (paged_attention.metal:569-571, 920-929,
 * 1063-1071) with the per-layer scales below (KvScaleManager::k_scale / v_scale,
 * crates/mlx-paged-attn/src/metal/kv_scale.rs:90-97; default 1).  Decode, verify
 * and prefill chunks are all served, as with a 16-bit cache.                      */
pa_status pa_cache_create_fp8(const PagedAttnConfig *config, int32_t device,
                              PagedAttnCache **out_cache);
pa_status pa_cache_wrap_fp8(const PagedAttnConfig *config, int32_t device,
                            void *const *key_ptrs, void *const *value_ptrs,
                            PagedAttnCache **out_cache);
int32_t pa_cache_is_fp8(const PagedAttnCache *cache);
pa_status pa_cache_set_kv_scales(PagedAttnCache *cache, uint32_t layer_idx, float k_scale,
                                 float v_scale);
pa_status pa_cache_get_kv_scales(const PagedAttnCache *cache, uint32_t layer_idx,
                                 float *k_scale, float *v_scale);
/* The attention kernels decode FP8 bytes in one of two ways.  The exact one reads a
 * byte with exponent field 15 as infinity or NaN, as the cache format defines; the
 * fast one is valid while the pools hold no such byte.  A cache made by
 * pa_cache_create_fp8 starts fast (zero-filled pools) and switches to exact by
 * itself when a write produces such a byte (overflow of x/scale, infinity or NaN
 * going in).  A cache made by pa_cache_wrap_fp8 starts exact, because the contents
 * of the caller's memory are unknown; on = 0 is the caller's statement that the
 * pools hold no exponent-15 byte, on = 1 forces the exact variant.  Synchronous
 * (one 4-byte copy); no reference counterpart.                                   */
pa_status pa_cache_fp8_set_exact_decode(PagedAttnCache *cache, int32_t on);

/* Synchronises `stream` and reports, then clears, the error word the kernels
 * of this cache write instead of trapping (out-of-range block id or slot,
 * a bounded wait that ran out).                                               */
pa_status pa_cache_check_errors(PagedAttnCache *cache, void *cuda_stream);
/* The same without a device round trip when nothing is wrong: the attention kernels
 * leave a copy of the error word in host-visible memory as their last act, and this
 * call reads that copy.  Valid once the stream the attention call ran on has been
 * synchronised; falls through to pa_cache_check_errors when the copy is non-zero.   */
pa_status pa_cache_check_errors_fast(PagedAttnCache *cache, void *cuda_stream);

/* KV block write.  dispatch_reshape_and_cache_raw
 * (crates/mlx-paged-attn/src/metal/reshape_and_cache.rs:177-270) over the
 * kernel crates/mlx-paged-attn/metal/cache/reshape_and_cache.metal:33-98.
 * key/value: [num_tokens, num_kv_heads, head_size] in the cache dtype, row strides
 * key_stride/value_stride in elements; slot_mapping: int64 [num_tokens] on
 * the device, slot < 0 skipped, slot >= num_blocks*block_size skipped and
 * reported through pa_cache_check_errors.                                     */
pa_status pa_reshape_and_cache(PagedAttnCache *cache, uint32_t layer_idx,
                               const void *key, const void *value,
                               const int64_t *slot_mapping, int64_t num_tokens,
                               int64_t key_stride, int64_t value_stride,
                               void *cuda_stream);

/* Producer of the write + attend pair: per-head RMS norm of the projected queries
 * and keys, rotary embedding at each token's own position, and the KV block write,
 * one launch for all tokens.  Replaces the per-sequence loop of
 * Attention::compute_qkv_paged_decode
 * (crates/mlx-core/src/transformer/attention.rs:637-691), which runs steps 3-5 of
 * mlx_fused_attention_qkv (crates/mlx-sys/src/mlx.cpp:1343-1365: fast::rms_norm per
 * head, then fast::rope with traditional = false, scale 1, offset = the sequence's
 * position) once per sequence and stacks the results, followed by
 * PagedAttentionLayer::update_cache
 * (crates/mlx-core/src/transformer/block.rs:224-226).
 * q, k, v: the projection outputs [num_tokens, heads, head_size] in the cache dtype
 * (row strides in elements); q_out receives the normalised, rotated queries and may
 * be q itself; the normalised, rotated keys and the values go to the pool at
 * slot_mapping (same skipping and reporting as pa_reshape_and_cache) and nowhere
 * else.  q_norm_weight / k_norm_weight: [head_size] in the cache dtype, or null for
 * no norm.  positions: int32 [num_tokens] on the device.  rope_dims: even, <=
 * head_size; elements beyond it pass through.  The angle of frequency i is
 * float(position) * float(pow(rope_base, -i / (rope_dims/2))).                    */
pa_status pa_qk_norm_rope_and_cache(PagedAttnCache *cache, uint32_t layer_idx,
                                    void *q_out, const void *q, const void *k,
                                    const void *v, const void *q_norm_weight,
                                    const void *k_norm_weight, float eps,
                                    const int32_t *positions, float rope_base,
                                    uint32_t rope_dims, const int64_t *slot_mapping,
                                    int64_t num_tokens, int32_t num_q_heads,
                                    int64_t q_stride, int64_t q_out_stride,
                                    int64_t k_stride, int64_t v_stride,
                                    void *cuda_stream);

/* Copy-on-write block copy.  dispatch_copy_blocks_raw
 * (crates/mlx-paged-attn/src/metal/copy_blocks.rs:96-99) over
 * crates/mlx-paged-attn/metal/cache/copy_blocks.metal:6-36.
 * block_mapping: int64 [num_pairs, 2] (src, dst) on the device.               */
pa_status pa_copy_blocks(PagedAttnCache *cache, uint32_t layer_idx,
                         const int64_t *block_mapping, int64_t num_pairs,
                         void *cuda_stream);

/* ---- swapping blocks to host memory ------------------------------------------
 * CpuBlockCache + swap_out / swap_in of crates/mlx-paged-attn/src/metal/
 * swap_blocks.rs:15-252 (PagedKVCache::swap_out / swap_in / create_cpu_cache,
 * paged_kv_cache.rs:1542-1648).  The host copies live in pinned, device-mapped
 * memory owned by the PaCpuBlockCache; one kernel moves all requested blocks of a
 * layer over PCIe in each direction.  Like the reference, both calls return when the
 * copy has completed, swap_out skips blocks that are already swapped, swap_in fails
 * on a block that is not in the host cache ("Block N not found in CPU cache") and
 * drops the host copies it restored.                                              */
typedef struct PaCpuBlockCache PaCpuBlockCache;
PaCpuBlockCache *pa_cpu_cache_create(const PagedAttnCache *cache);
void pa_cpu_cache_free(PaCpuBlockCache *cpu);
/* One host cache serves every layer of the device cache: copies are kept per (layer,
 * block id), so swapping the same block ids out of several layers keeps every layer's
 * bytes apart (the reference's CpuBlockCache is keyed by block id alone and would
 * skip the second layer as "already swapped").
 * is_swapped: some layer of the block has a host copy; num_swapped: such block ids.    */
int32_t pa_cpu_cache_is_swapped(const PaCpuBlockCache *cpu, uint32_t block_id);
int32_t pa_cpu_cache_is_swapped_layer(const PaCpuBlockCache *cpu, uint32_t layer_idx,
                                      uint32_t block_id);
size_t pa_cpu_cache_num_swapped(const PaCpuBlockCache *cpu);
/* Host addresses of a swapped block's K and V bytes of one layer (borrowed), or
 * PA_ERR_INVALID_ARG.                                                                  */
pa_status pa_cpu_cache_block_ptrs(const PaCpuBlockCache *cpu, uint32_t layer_idx,
                                  uint32_t block_id, void **key, void **value);
pa_status pa_swap_out(PagedAttnCache *cache, uint32_t layer_idx, const uint32_t *block_ids,
                      size_t num_blocks, PaCpuBlockCache *cpu, void *cuda_stream);
pa_status pa_swap_in(PagedAttnCache *cache, uint32_t layer_idx, const uint32_t *block_ids,
                     size_t num_blocks, PaCpuBlockCache *cpu, void *cuda_stream);
/* All-gather of head outputs over peer memory, for KV-head sharding across the GPUs
 * of one box when a consumer needs every head on every rank (no counterpart in the
 * reference, which runs on one device).  Rank `rank` holds local_out
 * [num_tokens, heads_local, head_size]; peer_out[w] is rank w's
 * [num_tokens, world * heads_local, head_size] buffer and peer_flags[w] its `world`
 * flag words (zero before the first call), both addressable from this GPU (peer access
 * in one process, or symmetric-memory / IPC mappings across processes).  The call
 * stores this rank's heads into every buffer with plain 16-byte stores, publishes
 * flag[rank] = epoch in every rank's flag words, and then, if `wait` is non-zero, waits
 * on `stream` (about a second at most; a missing writer is reported as PA_ERR_TIMEOUT by
 * pa_cache_check_errors) until all `world` flags of this rank have reached `epoch`;
 * pa_gather_heads_wait is that wait on its own, for a caller that wants to put work
 * between the two.
 * Use epoch = 1, 2, 3, ... for successive calls; every rank must make the same calls.
 * A step with num_tokens = 0 moves nothing and still publishes its flag (local_out and the
 * entries of peer_out may then be null).
 * Before an output buffer is reused as a peer_out target, all ranks must have consumed
 * its previous contents (alternate two buffers, or separate the steps by a barrier). */
pa_status pa_gather_heads_peer_store(PagedAttnCache *cache, const void *local_out,
                                     int64_t num_tokens, int32_t heads_local, int32_t world,
                                     int32_t rank, void *const *peer_out,
                                     uint32_t *const *peer_flags, uint32_t epoch,
                                     int32_t wait, void *cuda_stream);
pa_status pa_gather_heads_wait(PagedAttnCache *cache, const uint32_t *my_flags, int32_t world,
                               uint32_t epoch, void *cuda_stream);

/* SwapBlocksParams::key_block_size / value_block_size (swap_blocks.rs:53-108):
 * bytes of one block of one layer; use_fp8 halves them.                           */
void pa_swap_block_bytes(uint32_t num_kv_heads, uint32_t head_size, uint32_t block_size,
                         int32_t use_fp8, uint64_t *key_bytes, uint64_t *value_bytes);

/* Scratch the attention calls need, for any batch on this cache's device (it
 * depends only on the device's SM count, the head size and whether the cache is
 * FP8: partial-result slots for one CTA per SM, two where the decode kernel shares
 * an SM - FP8 caches and head sizes up to 80).  A call given less, but at least the
 * slots of one CTA per SM, still runs, on fewer CTAs.                           */
size_t pa_attention_workspace_bytes(const PagedAttnCache *cache);

/* Single-token decode attention: one query per sequence, all query heads of a
 * GQA group served from one read of the KV blocks.  Replaces
 * dispatch_paged_attention_auto (crates/mlx-paged-attn/src/metal/
 * paged_attention.rs:954-991; kernels crates/mlx-paged-attn/metal/attention/
 * paged_attention.metal:760-1260) and mlx_paged_attn_forward
 * (crates/mlx-sys/src/mlx.cpp:4041-4162).
 *   num_q_heads   a multiple of the cache's num_kv_heads, at most 24 times it (16 with
 *                 head size 192, 8 with 256; else PA_ERR_UNSUPPORTED)
 *   out, q        [num_seqs, num_q_heads, head_size] in the cache dtype; row strides
 *                 q_stride / out_stride in elements
 *   block_tables  int32 [num_seqs, max_blocks_per_seq], device
 *   context_lens  int32 [num_seqs], device; counts the token written this step
 *   softcap       1.0f = off (crates/.../paged_attention.metal:937-940)
 *   workspace     >= pa_attention_workspace_bytes(), 256-byte aligned, device
 * context_len 0 gives a zero row (mlx.cpp:4084-4088).                         */
pa_status pa_paged_attention_decode(PagedAttnCache *cache, uint32_t layer_idx,
                                    void *out, const void *q,
                                    const int32_t *block_tables,
                                    const int32_t *context_lens, int32_t num_seqs,
                                    int32_t num_q_heads, int32_t max_blocks_per_seq,
                                    int64_t q_stride, int64_t out_stride, float scale,
                                    float softcap, void *workspace,
                                    size_t workspace_bytes, void *cuda_stream);

/* One decode step of one layer in ONE launch: the step's new token of every
 * sequence is written to the pool and attention runs over the cache that
 * already holds it - the order TransformerBlock::forward_paged keeps with two
 * calls (crates/mlx-core/src/transformer/block.rs:223-232: update_cache, then
 * forward).  The warp that attends the last block of a (sequence, kv head)
 * stores that head's new key and value rows into the pool itself, so no write
 * kernel runs before the attention kernel and no reduce kernel after it.
 *   key, value     [num_seqs, num_kv_heads, head_size] in the cache dtype, row
 *                  strides key_stride / value_stride in elements, device
 *   slot_mapping   int64 [num_seqs], device: slot of sequence s's new token,
 *                  which must be position context_lens[s] - 1 of that sequence
 *                  (what get_slot_mapping_decode returns,
 *                  crates/mlx-paged-attn/src/paged_kv_cache.rs:539-552); negative
 *                  = no write.  Any other value is not written and
 *                  pa_cache_check_errors reports PA_ERR_INVALID_ARG.
 * The other arguments are those of pa_paged_attention_decode.  The pool bytes
 * after the call equal those pa_reshape_and_cache would have produced.  On an
 * FP8 cache, with 8- or 32-token blocks, more than 8 query heads per kv head, or
 * more than 2 x (SM count) (sequence, kv head) pairs in the batch (the in-kernel
 * write costs its CTA a few microseconds per pair, a launch of its own about
 * four in total) the call runs the write kernel and then the attention kernel.
 *   context_lens and block_tables (and, for pa_paged_attention_varlen, the query
 * offsets) are read as soon as the launch is scheduled, which may be before
 * earlier kernels of the stream have finished when those were launched with
 * programmatic dependent launch and trigger early (this library's own write
 * and attention kernels do; they write none of these): produce them with
 * ordinary launches or copies, before such a trigger, or on the host.  Queries,
 * keys, values and the pools are read after the predecessor has completed.    */
pa_status pa_decode_step(PagedAttnCache *cache, uint32_t layer_idx, void *out, const void *q,
                         const void *key, const void *value, const int64_t *slot_mapping,
                         const int32_t *block_tables, const int32_t *context_lens,
                         int32_t num_seqs, int32_t num_q_heads, int32_t max_blocks_per_seq,
                         int64_t q_stride, int64_t out_stride, int64_t key_stride,
                         int64_t value_stride, float scale, float softcap, void *workspace,
                         size_t workspace_bytes, void *cuda_stream);

/* pa_paged_attention_decode / pa_decode_step over a RESIDENT block table: block_tables
 * is [rows, max_blocks_per_seq] with one row per live sequence, kept on the device
 * across steps, and seq_rows int32 [num_seqs] (device) names the row of each sequence
 * of this batch.  The reference has no such form: it rebuilds and re-sends the batch's
 * table on every call (crates/mlx-paged-attn/src/paged_kv_cache.rs:1081-1125,
 * crates/mlx-core/src/models/qwen3/model.rs:879-891).  Used by the bound-cache calls of
 * paged_attn_b200_host.h.                                                         */
pa_status pa_paged_attention_decode_rows(PagedAttnCache *cache, uint32_t layer_idx, void *out,
                                         const void *q, const int32_t *block_tables,
                                         const int32_t *seq_rows, const int32_t *context_lens,
                                         int32_t num_seqs, int32_t num_q_heads,
                                         int32_t max_blocks_per_seq, int64_t q_stride,
                                         int64_t out_stride, float scale, float softcap,
                                         void *workspace, size_t workspace_bytes,
                                         void *cuda_stream);
pa_status pa_decode_step_rows(PagedAttnCache *cache, uint32_t layer_idx, void *out, const void *q,
                              const void *key, const void *value, const int64_t *slot_mapping,
                              const int32_t *block_tables, const int32_t *seq_rows,
                              const int32_t *context_lens, int32_t num_seqs, int32_t num_q_heads,
                              int32_t max_blocks_per_seq, int64_t q_stride, int64_t out_stride,
                              int64_t key_stride, int64_t value_stride, float scale,
                              float softcap, void *workspace, size_t workspace_bytes,
                              void *cuda_stream);

/* Decode attention for callers that cannot allocate device memory.
 * No counterpart in the reference.  Some hosts of this library are handed
 * their buffers by someone else and have no way to ask for more: a plugin
 * running inside another runtime's memory pool, a caller whose allocator is
 * locked down once serving has started, code that runs where a cudaMalloc
 * would stall every stream of the process.  For them this entry computes
 * exactly what pa_paged_attention_decode computes, but keeps the split-KV
 * partial results in an array that is part of the library image instead of a
 * caller workspace; a call that succeeds calls no allocator, the CUDA one or any
 * other (a refused call builds its error message in a host string).
 *   Limit: the array holds partials for 160 CTAs (one per SM), 4.2 MiB.  It is
 * resident on every GPU this process uses the library on, from load to exit,
 * whether or not this entry is ever called.  On a GPU with more than 160 SMs
 * the call is refused with PA_ERR_UNSUPPORTED and a message saying so.  An FP8
 * cache runs its narrow kernel on one CTA per SM here instead of two (the array
 * has slots for 160).
 *   The first call on each device looks up the array's device address (one
 * runtime query, remembered afterwards); make that first call outside any
 * stream capture.
 *   All calls on a device share the one array.  Nothing in it has to start at
 * zero - every slot is written before it is read within a call - but two calls
 * whose kernels overlap on the GPU (different streams, no ordering between
 * them) would overwrite each other's partials: keep calls to this entry
 * ordered on a device.  Arguments are those of pa_paged_attention_decode minus
 * the workspace.                                                              */
pa_status pa_paged_attention_decode_static(PagedAttnCache *cache, uint32_t layer_idx,
                                           void *out, const void *q,
                                           const int32_t *block_tables,
                                           const int32_t *context_lens, int32_t num_seqs,
                                           int32_t num_q_heads, int32_t max_blocks_per_seq,
                                           int64_t q_stride, int64_t out_stride, float scale,
                                           float softcap, void *cuda_stream);

/* Variable-length paged attention: decode, speculative-verify and
 * chunked-prefill sequences mixed in one call.  The reference has no such
 * entry (its scheduler says so, crates/mlx-paged-attn/src/scheduler.rs:237-242);
 * the semantics extend its decode (above) and its dense causal prefill
 * (crates/mlx-core/src/transformer/block.rs:279-317):
 * sequence s has context_lens[s] tokens in the pool after this step's write
 * and q_len_s = cu_q_lens[s+1]-cu_q_lens[s] >= 0 queries that occupy the last
 * q_len_s positions; query j attends keys [0, context_lens[s]-q_len_s+j].
 *   out, q        [total_q, num_q_heads, head_size] in the cache dtype, packed by sequence
 *   cu_q_lens_host      int32 [num_seqs+1] in HOST memory (the scheduler has it);
 *                       the library uploads what its kernels need
 *   context_lens_host   optional host copy of context_lens (may be null).  With
 *                       it, a batch that mixes long-query and short-query sequences
 *                       runs its two kernels side by side on SM shares sized by
 *                       their estimated work; without it they run back to back.
 *                       Required with 8-token blocks when a sequence has more than
 *                       24 / (query heads per kv head) queries (PA_ERR_INVALID_ARG
 *                       otherwise): such chunks are served in pieces of that size.
 *   max_context_len     upper bound of context_lens (0 = unknown)              */
pa_status pa_paged_attention_varlen(PagedAttnCache *cache, uint32_t layer_idx,
                                    void *out, const void *q,
                                    const int32_t *block_tables,
                                    const int32_t *context_lens,
                                    const int32_t *cu_q_lens_host,
                                    const int32_t *context_lens_host, int32_t num_seqs,
                                    int32_t num_q_heads, int32_t max_blocks_per_seq,
                                    int64_t q_stride, int64_t out_stride, float scale,
                                    float softcap, int32_t max_context_len,
                                    void *workspace, size_t workspace_bytes,
                                    void *cuda_stream);

/* One decode step of one layer from HOST buffers, the order
 * TransformerBlock::forward_paged keeps (crates/mlx-core/src/transformer/
 * block.rs:223-232): write the new tokens' K/V, then attend with context
 * lengths that already count them.  Brings q/k/v/slots/tables/lens to the
 * device, runs pa_decode_step, copies `out` back and synchronises.  Staging
 * buffers are kept in the cache handle and grow on demand.  Everything is
 * queued on a stream the handle owns, NOT on a stream of the caller: earlier
 * work on the same pools (a prefill write, copy_blocks, swap_in) must have
 * completed - be synchronised - before this call.                             */
pa_status pa_decode_step_host(PagedAttnCache *cache, uint32_t layer_idx,
                              void *out_host, const void *q_host, const void *k_host,
                              const void *v_host, const int64_t *slot_mapping_host,
                              const int32_t *block_tables_host,
                              const int32_t *context_lens_host, int32_t num_seqs,
                              int32_t num_q_heads, int32_t max_blocks_per_seq,
                              float scale, float softcap);

/* The same for a mixed batch (decode, verify and prefill-chunk sequences, the
 * semantics of pa_paged_attention_varlen) from HOST buffers: copies the
 * total_q = cu_q_lens_host[num_seqs] new tokens' q/k/v and slots, the tables and
 * the lengths to the device, writes the K/V, attends, copies `out`
 * [total_q, num_q_heads, head_size] back and synchronises.  Runs on the handle's
 * own stream like pa_decode_step_host: work the caller queued elsewhere on the
 * same pools must have completed before either call.                          */
pa_status pa_varlen_step_host(PagedAttnCache *cache, uint32_t layer_idx, void *out_host,
                              const void *q_host, const void *k_host, const void *v_host,
                              const int64_t *slot_mapping_host,
                              const int32_t *block_tables_host,
                              const int32_t *context_lens_host,
                              const int32_t *cu_q_lens_host, int32_t num_seqs,
                              int32_t num_q_heads, int32_t max_blocks_per_seq, float scale,
                              float softcap);

/* Number of kernels this library has launched from the calling process
 * (all threads), for launch accounting in benchmarks.                         */
uint64_t pa_kernel_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* PAGED_ATTN_B200_H_ */
