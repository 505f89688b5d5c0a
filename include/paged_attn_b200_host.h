/*
 * paged_attn_b200 — C ABI of the host-side pool management that feeds the
 * paged-attention kernels: block allocator, block tables, slot mapping and
 * kernel-argument metadata, token tracker, continuous-batching scheduler.
 * No CUDA is involved; every function runs on the host.
 *
 * It mirrors, name for name, the host API of the reference crate
 * (crates/mlx-paged-attn/src/lib.rs:21-51).  Where the reference hands out
 * Arc<PhysicalBlock>, this ABI identifies a block by its block id.  Functions
 * that can fail return pa_status (paged_attn_b200.h) and leave the reference's
 * error text in pa_last_error_string().
 */
#ifndef PAGED_ATTN_B200_HOST_H_
#define PAGED_ATTN_B200_HOST_H_

#include <stddef.h>
#include <stdint.h>

#include "paged_attn_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* PagedAttentionConfig, crates/mlx-paged-attn/src/config.rs:5-34.  max_seq_len and
 * max_batch_size 0 mean the reference defaults (8192, 256).                      */
typedef struct PaHostConfig {
  uint32_t block_size, gpu_memory_mb, head_size, num_kv_heads, num_layers;
  uint32_t use_fp8_cache, max_seq_len, max_batch_size;
} PaHostConfig;
/* PagedAttentionConfig::default(), config.rs:125-138. */
void pa_host_config_default(PaHostConfig *out);
/* PagedAttentionConfig::validate(), config.rs:36-75. */
pa_status pa_host_config_validate(const PaHostConfig *cfg);
/* PagedAttentionConfig::calculate_num_blocks(), config.rs:86-102. */
uint32_t pa_host_config_num_blocks(const PaHostConfig *cfg);

/* hash_tokens (SipHash-1-3, zero key), block_allocator.rs:239-249. */
uint64_t pa_hash_tokens(const uint32_t *tokens, size_t n, uint64_t parent_hash);
/* compute_token_hash (FNV-1a), token_tracker.rs:388-402. */
uint64_t pa_compute_token_hash(const uint32_t *tokens, size_t n);
/* KvScaleManager::compute_scale, metal/kv_scale.rs:165-174. */
float pa_kv_compute_scale(float max_abs);

/* KV-head sharding over the GPUs of one box (no counterpart in the reference, which
 * runs on one device): rank r of `world` owns kv heads [kv_begin, kv_end) and the
 * query heads [q_begin, q_end) that map onto them (kv_head = q_head / G,
 * crates/mlx-paged-attn/metal/attention/paged_attention.metal:837-840).  Its pools
 * are [num_blocks, kv_end - kv_begin, ...] with the same block ids on every rank;
 * pointing `out` of an attention call at column q_begin * head_size of a
 * [tokens, num_q_heads, head_size] buffer with out_stride = num_q_heads * head_size
 * places the rank's heads where a gathered result has them.
 * PA_ERR_INVALID_ARG when the heads do not split `world` ways.                      */
pa_status pa_shard_head_ranges(int32_t rank, int32_t world, int32_t num_q_heads,
                               int32_t num_kv_heads, int32_t *kv_begin, int32_t *kv_end,
                               int32_t *q_begin, int32_t *q_end);

/* ---- BlockAllocator, block_allocator.rs:62-236 ---------------------------------- */
typedef struct PaAllocator PaAllocator;
PaAllocator *pa_alloc_create(uint32_t num_blocks, uint32_t block_size);
void pa_alloc_destroy(PaAllocator *a);
int64_t pa_alloc_allocate(PaAllocator *a);                    /* block id, -1 when exhausted   */
pa_status pa_alloc_release(PaAllocator *a, uint32_t block_id); /* BlockAllocator::free          */
pa_status pa_alloc_incref(PaAllocator *a, uint32_t block_id);  /* PhysicalBlock::incref         */
int64_t pa_alloc_ref_count(PaAllocator *a, uint32_t block_id); /* -1 if not allocated           */
int64_t pa_alloc_copy_on_write(PaAllocator *a, uint32_t block_id); /* new id, -1 = no copy     */
pa_status pa_alloc_register_prefix(PaAllocator *a, uint32_t block_id, uint64_t hash);
int64_t pa_alloc_lookup_prefix(PaAllocator *a, uint64_t hash);     /* block id or -1            */
uint32_t pa_alloc_num_free(const PaAllocator *a);
uint32_t pa_alloc_num_allocated(const PaAllocator *a);
uint32_t pa_alloc_total(const PaAllocator *a);
int32_t pa_alloc_can_allocate(const PaAllocator *a, uint32_t n);
void pa_alloc_set_max_prefix_entries(PaAllocator *a, uint32_t n);
uint32_t pa_alloc_prefix_cache_len(const PaAllocator *a);
int32_t pa_alloc_has_block_hash(const PaAllocator *a, uint32_t block_id);
void pa_alloc_clear_lru_order(PaAllocator *a); /* what block_allocator.rs:413-434 does by hand */

/* ---- TokenTracker, token_tracker.rs:29-361 ---------------------------------------- */
typedef struct PaTracker PaTracker;
PaTracker *pa_tracker_create(uint32_t block_size, int32_t enabled);
void pa_tracker_destroy(PaTracker *t);
int32_t pa_tracker_is_enabled(const PaTracker *t);
uint64_t pa_tracker_track_tokens(PaTracker *t, uint32_t block_id, const uint32_t *tokens, size_t n,
                                 uint32_t start_offset);
/* copies up to cap tokens, returns the block's token count */
uint32_t pa_tracker_get_block_tokens(const PaTracker *t, uint32_t block_id, uint32_t *out, size_t cap);
void pa_tracker_remove_block(PaTracker *t, uint32_t block_id);
void pa_tracker_copy_block(PaTracker *t, uint32_t src, uint32_t dst);
/* pairs (block id, matched tokens); returns the number of matches */
size_t pa_tracker_find_prefix_matches(const PaTracker *t, const uint32_t *tokens, size_t n,
                                      uint32_t *out_pairs, size_t cap_pairs);
/* block ids of the longest cached prefix; *matched_tokens receives the token count */
size_t pa_tracker_find_longest_prefix(const PaTracker *t, const uint32_t *tokens, size_t n,
                                      uint32_t *out_blocks, size_t cap, uint32_t *matched_tokens);
typedef struct PaTrackerStats {
  uint32_t num_tracked_blocks, total_tracked_tokens;
  float avg_tokens_per_block;
  uint32_t prefix_index_size;
} PaTrackerStats;
void pa_tracker_stats(const PaTracker *t, PaTrackerStats *out);
void pa_tracker_clear(PaTracker *t);
size_t pa_tracker_memory_usage(const PaTracker *t);

/* ---- SequenceBlockTable arithmetic, block_table.rs:95-143 -------------------------- */
/* free_slots_in_last_block / blocks_needed / is_last_block_full for a table that holds
 * num_blocks blocks and num_tokens tokens                                             */
uint32_t pa_table_free_slots_in_last_block(uint32_t num_blocks, uint32_t num_tokens, uint32_t block_size);
uint32_t pa_table_blocks_needed(uint32_t num_blocks, uint32_t num_tokens, uint32_t block_size,
                                uint32_t new_tokens);
int32_t pa_table_is_last_block_full(uint32_t num_tokens, uint32_t block_size);
void pa_table_slot_index(uint32_t token_pos, uint32_t block_size, uint32_t *block_idx, uint32_t *offset);

/* ---- PagedKVCache host methods, paged_kv_cache.rs ------------------------------------ */
typedef struct PaKvHost PaKvHost;
pa_status pa_kv_create(const PaHostConfig *cfg, PaKvHost **out);      /* PagedKVCache::new      */
void pa_kv_destroy(PaKvHost *kv);
pa_status pa_kv_add_sequence(PaKvHost *kv, uint32_t prompt_len, uint32_t *seq_id);   /* :97-125 */
pa_status pa_kv_remove_sequence(PaKvHost *kv, uint32_t seq_id);                      /* :127-151 */
pa_status pa_kv_extend_sequence(PaKvHost *kv, uint32_t seq_id, uint32_t num_new);    /* :458-479 */
/* extend_sequence for every sequence of a batch, what process_outputs does once per
 * sampled token (scheduler.rs:354-358), in one call.  Stops at the first failure.       */
pa_status pa_kv_extend_sequences(PaKvHost *kv, const uint32_t *seq_ids, size_t n, uint32_t num_tokens);
pa_status pa_kv_fork_sequence(PaKvHost *kv, uint32_t parent, uint32_t *child);       /* :1437-1465 */
/* handle_cow (:1476-1523): *copied = 0 when the block is not shared; otherwise the
 * caller issues pa_copy_blocks for the (src, dst) pair on every layer.                */
pa_status pa_kv_handle_cow(PaKvHost *kv, uint32_t seq_id, uint32_t block_idx, int32_t *copied,
                           uint32_t *src_block, uint32_t *dst_block);
int32_t pa_kv_can_allocate(const PaKvHost *kv, uint32_t num_blocks);
uint32_t pa_kv_num_sequences(const PaKvHost *kv);
uint32_t pa_kv_num_free_blocks(const PaKvHost *kv);
uint32_t pa_kv_total_blocks(const PaKvHost *kv);
uint32_t pa_kv_block_size(const PaKvHost *kv);
uint32_t pa_kv_max_blocks_per_seq(const PaKvHost *kv);               /* :196-199 */
size_t pa_kv_get_context_lens(const PaKvHost *kv, uint32_t *out, size_t cap);
size_t pa_kv_get_seq_ids(const PaKvHost *kv, uint32_t *out, size_t cap);
/* build_block_tables (:203-208): [num_sequences, max_blocks_per_seq], zero padded;
 * returns the element count                                                           */
size_t pa_kv_build_block_tables(const PaKvHost *kv, uint32_t *out, size_t cap);
/* block ids of one sequence; returns the count */
pa_status pa_kv_sequence_blocks(const PaKvHost *kv, uint32_t seq_id, uint32_t *out, size_t cap, size_t *count);
pa_status pa_kv_get_slot_mapping(const PaKvHost *kv, uint32_t seq_id, uint32_t start_pos,
                                 uint32_t num_tokens, int64_t *out);                  /* :483-507 */
/* get_slot_mapping_batch (:509-561); out needs sum(prefill input_lens) + #decode slots */
pa_status pa_kv_get_slot_mapping_batch(const PaKvHost *kv, const uint32_t *seq_ids,
                                       const uint32_t *context_lens, const uint8_t *is_prefill,
                                       const uint32_t *input_lens, size_t n, int64_t *out, size_t cap,
                                       size_t *count);
/* build_input_metadata (:646-704): the three arrays the kernels take, in their device
 * types (int32 tables [n, max_blocks_per_seq], int32 lens [n], int64 slots).  The
 * capacities are in elements; a buffer that is too small is an error, never an
 * overflow (the table needs n * pa_kv_max_blocks_per_seq(kv) entries).                */
pa_status pa_kv_build_input_metadata(const PaKvHost *kv, const uint32_t *seq_ids,
                                     const uint32_t *input_lens, const uint8_t *is_prefill, size_t n,
                                     int32_t *block_tables_out, size_t tables_cap,
                                     int32_t *context_lens_out, size_t lens_cap,
                                     int64_t *slots_out, size_t slots_cap, size_t *num_slots,
                                     uint32_t *max_context_len, int32_t *batch_is_prefill);
typedef struct PaMemoryStats {
  uint32_t total_blocks, free_blocks, allocated_blocks, total_memory_mb, used_memory_mb;
  double utilization_percent;
} PaMemoryStats;
void pa_kv_memory_stats(const PaKvHost *kv, PaMemoryStats *out);                      /* :598-622 */
pa_status pa_kv_track_sequence_tokens(PaKvHost *kv, uint32_t seq_id, const uint32_t *tokens, size_t n,
                                      uint32_t start_pos);
pa_status pa_kv_get_sequence_tokens(const PaKvHost *kv, uint32_t seq_id, uint32_t *out, size_t cap,
                                    size_t *count);
size_t pa_kv_find_prefix_matches(const PaKvHost *kv, const uint32_t *tokens, size_t n, uint32_t *out_pairs,
                                 size_t cap_pairs);
size_t pa_kv_find_longest_prefix(const PaKvHost *kv, const uint32_t *tokens, size_t n, uint32_t *out_blocks,
                                 size_t cap, uint32_t *matched_tokens);
uint32_t pa_kv_get_block_tokens(const PaKvHost *kv, uint32_t block_id, uint32_t *out, size_t cap);
void pa_kv_tracker_stats(const PaKvHost *kv, PaTrackerStats *out);
size_t pa_kv_tracker_memory(const PaKvHost *kv);

/* ---- ContinuousBatchingScheduler, scheduler.rs:114-483 ------------------------------ */
typedef struct PaSchedulerConfig {
  uint32_t max_batch_size, max_tokens_per_step, max_prefill_per_step, prioritize_decode, eos_token_id;
} PaSchedulerConfig;
void pa_sched_config_default(PaSchedulerConfig *out);                                /* :127-137 */
typedef struct PaScheduler PaScheduler;
PaScheduler *pa_sched_create(uint32_t block_size, const PaSchedulerConfig *cfg_or_null);
void pa_sched_destroy(PaScheduler *s);
void pa_sched_add_request(PaScheduler *s, const char *request_id, const uint32_t *prompt_tokens, size_t n,
                          uint32_t max_new_tokens, int32_t priority);
/* schedule_step (:195-330): returns the number of sequences in the batch (0 = none).
 * The batch is kept until the next call and read with the accessors below.            */
uint32_t pa_sched_schedule_step(PaScheduler *s, PaKvHost *kv);
typedef struct PaBatchTotals {
  uint32_t total_tokens, num_prefill, num_decode;
} PaBatchTotals;
void pa_sched_batch_totals(const PaScheduler *s, PaBatchTotals *out);
/* per sequence i: seq id, prefill flag, context length, number of input tokens */
pa_status pa_sched_batch_entry(const PaScheduler *s, uint32_t i, uint32_t *seq_id, int32_t *is_prefill,
                               uint32_t *context_len, uint32_t *num_input_tokens);
uint32_t pa_sched_batch_tokens(const PaScheduler *s, uint32_t i, uint32_t *out, size_t cap);
const char *pa_sched_batch_request_id(const PaScheduler *s, uint32_t i);
/* process_outputs (:339-389) */
pa_status pa_sched_process_outputs(PaScheduler *s, PaKvHost *kv, const uint32_t *seq_ids,
                                   const uint32_t *tokens, const uint8_t *is_eos, size_t n);
/* get_completed (:392-394): moves the finished sequences into a list read below */
uint32_t pa_sched_take_completed(PaScheduler *s);
const char *pa_sched_completed_request_id(const PaScheduler *s, uint32_t i);
const char *pa_sched_completed_finish_reason(const PaScheduler *s, uint32_t i);
uint32_t pa_sched_completed_tokens(const PaScheduler *s, uint32_t i, uint32_t *out, size_t cap,
                                   uint32_t *total_tokens);
pa_status pa_sched_abort_request(PaScheduler *s, PaKvHost *kv, const char *request_id, int32_t *found);
int32_t pa_sched_is_empty(const PaScheduler *s);
typedef struct PaSchedulerStats {
  uint32_t num_waiting, num_running, num_completed, num_prefill, num_decode, total_running_tokens;
} PaSchedulerStats;
void pa_sched_stats(const PaScheduler *s, PaSchedulerStats *out);
/* 1 / 0 for a running sequence's prefill flag, -1 if it is not running */
int32_t pa_sched_running_is_prefill(const PaScheduler *s, uint32_t seq_id);

/* ---- hybrid scheduler: chunked prefill + speculative verify + decode in one batch ----
 * No counterpart in the reference: its scheduler runs a whole prompt in one step and
 * says chunked prefill is future work (scheduler.rs:237-242).  This one emits the mixed
 * batches pa_paged_attention_varlen takes.  Per step and sequence: kind 0 = prefill
 * chunk, 1 = decode (one token), 2 = verify (last token + draft tokens); q_len new
 * tokens whose K/V the step writes at positions [kv_len - q_len, kv_len).           */
typedef struct PaHybridConfig {
  uint32_t max_batch_size, max_tokens_per_step, prefill_chunk_size, max_prefill_per_step;
  uint32_t prioritize_decode, eos_token_id;
} PaHybridConfig;
void pa_hybrid_config_default(PaHybridConfig *out);
typedef struct PaHybridScheduler PaHybridScheduler;
PaHybridScheduler *pa_hybrid_create(uint32_t block_size, const PaHybridConfig *cfg_or_null);
void pa_hybrid_destroy(PaHybridScheduler *s);
void pa_hybrid_add_request(PaHybridScheduler *s, const char *request_id, const uint32_t *prompt_tokens,
                           size_t n, uint32_t max_new_tokens, int32_t priority);
/* draft tokens to verify at the sequence's next decode step */
pa_status pa_hybrid_set_draft_tokens(PaHybridScheduler *s, uint32_t seq_id, const uint32_t *tokens, size_t n);
/* returns the number of sequences in the batch (0 = nothing to run); the batch stays
 * readable until the next call                                                       */
uint32_t pa_hybrid_schedule_step(PaHybridScheduler *s, PaKvHost *kv);
typedef struct PaHybridTotals {
  uint32_t total_tokens, num_prefill, num_decode, num_verify;
} PaHybridTotals;
void pa_hybrid_batch_totals(const PaHybridScheduler *s, PaHybridTotals *out);
pa_status pa_hybrid_batch_entry(const PaHybridScheduler *s, uint32_t i, uint32_t *seq_id, int32_t *kind,
                                uint32_t *q_len, uint32_t *kv_len, int32_t *needs_sample);
uint32_t pa_hybrid_batch_tokens(const PaHybridScheduler *s, uint32_t i, uint32_t *out, size_t cap);
const char *pa_hybrid_batch_request_id(const PaHybridScheduler *s, uint32_t i);
/* kernel arguments of the current batch: int32 tables [n, max_blocks_per_seq] zero
 * padded, int32 context lens [n] (counting this step's tokens), int32 cu_q_lens [n+1],
 * int64 slots [total_tokens].  Capacities in elements: tables_cap for block_tables,
 * seqs_cap = sequences context_lens has room for (cu_q_lens then has seqs_cap + 1),
 * slots_cap for slots; too small is an error, never an overflow.                      */
pa_status pa_hybrid_batch_metadata(const PaHybridScheduler *s, const PaKvHost *kv, int32_t *block_tables,
                                   size_t tables_cap, int32_t *context_lens, int32_t *cu_q_lens,
                                   size_t seqs_cap, int64_t *slots, size_t slots_cap,
                                   uint32_t *max_context_len);
/* one record per entry with needs_sample: accepted draft tokens and the token sampled
 * after them                                                                          */
pa_status pa_hybrid_process_outputs(PaHybridScheduler *s, PaKvHost *kv, const uint32_t *seq_ids,
                                    const uint32_t *num_accepted, const uint32_t *next_tokens,
                                    const uint8_t *is_eos, size_t n);
uint32_t pa_hybrid_take_completed(PaHybridScheduler *s);
const char *pa_hybrid_completed_request_id(const PaHybridScheduler *s, uint32_t i);
const char *pa_hybrid_completed_finish_reason(const PaHybridScheduler *s, uint32_t i);
uint32_t pa_hybrid_completed_tokens(const PaHybridScheduler *s, uint32_t i, uint32_t *out, size_t cap,
                                    uint32_t *total_tokens);
int32_t pa_hybrid_is_empty(const PaHybridScheduler *s);
uint32_t pa_hybrid_num_waiting(const PaHybridScheduler *s);
uint32_t pa_hybrid_num_running(const PaHybridScheduler *s);
/* truncate_sequence: drop the tail of a sequence, releasing emptied blocks (used for
 * rejected draft tokens)                                                              */
pa_status pa_kv_truncate_sequence(PaKvHost *kv, uint32_t seq_id, uint32_t new_num_tokens);

/* ==== The host cache bound to a device cache ========================================
 * In the reference PagedKVCache is one object: block tables and allocator on the host,
 * per-layer pools on the device behind its CacheEngineManager.  Here the host side is
 * PaKvHost and the pools are PagedAttnCache; a binding joins the two so that the
 * reference's device-touching methods exist with their own argument lists
 * (sequence ids in, no tables or lengths to build by hand).
 *
 * The binding keeps the block tables RESIDENT on the device, one row per live
 * sequence, and sends per call only the table entries that changed since the last call
 * (a decode step appends one entry per sequence every block_size steps), the batch's
 * row indices and its context lengths - one small pinned staging area read by one
 * launch.  The reference rebuilds and re-uploads the whole [num_seqs,
 * max_blocks_per_seq] table on every call (paged_kv_cache.rs:1081-1125).
 * One binding is used by one thread and one stream at a time.                         */
typedef struct PaKvBinding PaKvBinding;
pa_status pa_kv_bind(PaKvHost *kv, PagedAttnCache *cache, PaKvBinding **out);
void pa_kv_unbind(PaKvBinding *b);
/* PagedKVCache::update (paged_kv_cache.rs:753-870): keys, values [num_tokens,
 * num_kv_heads, head_size] and slot_mapping int64 [num_tokens], all on the device.     */
pa_status pa_kv_update(PaKvBinding *b, uint32_t layer_idx, const void *keys, const void *values,
                       const int64_t *slot_mapping_dev, int64_t num_tokens, void *cuda_stream);
/* PagedKVCache::update_with_slots (:887-1012): the slot mapping is a host slice.        */
pa_status pa_kv_update_with_slots(PaKvBinding *b, uint32_t layer_idx, const void *keys,
                                  const void *values, const int64_t *slot_mapping_host,
                                  int64_t num_tokens, void *cuda_stream);
/* PagedKVCache::attention (:1034-1193): decode attention for the sequences `seq_ids`,
 * context lengths taken from the block tables; q, out [n, num_query_heads, head_size] on
 * the device.  An id that is not in the cache fails with the reference's message.
 * FP8 caches take their per-layer scales from the binding's scale manager.              */
pa_status pa_kv_attention(PaKvBinding *b, uint32_t layer_idx, void *out, const void *queries,
                          const uint32_t *seq_ids, size_t n, uint32_t num_query_heads, float scale,
                          void *cuda_stream);
/* PagedKVCache::attention_with_context (:1205-1347): context lengths given.             */
pa_status pa_kv_attention_with_context(PaKvBinding *b, uint32_t layer_idx, void *out,
                                       const void *queries, const uint32_t *seq_ids,
                                       const uint32_t *context_lens, size_t n,
                                       uint32_t num_query_heads, float scale, void *cuda_stream);
/* update_with_slots for the batch's newest tokens followed by attention, as one call
 * and (where pa_decode_step can) one launch: the slot of sequence i is position
 * num_tokens - 1 of its table (get_slot_mapping_decode, :539-552); keys, values
 * [n, num_kv_heads, head_size], q, out [n, num_query_heads, head_size] on the device.   */
pa_status pa_kv_decode_step(PaKvBinding *b, uint32_t layer_idx, void *out, const void *queries,
                            const void *keys, const void *values, const uint32_t *seq_ids, size_t n,
                            uint32_t num_query_heads, float scale, void *cuda_stream);
/* The same from HOST buffers (pinned buffers are read in place by the ingest launch,
 * pageable ones are copied first), result copied back to out_host, synchronous.  Runs
 * on a stream the binding owns: earlier work on the same pools must have completed.     */
pa_status pa_kv_decode_step_host(PaKvBinding *b, uint32_t layer_idx, void *out_host,
                                 const void *q_host, const void *k_host, const void *v_host,
                                 const uint32_t *seq_ids, size_t n, uint32_t num_query_heads,
                                 float scale);
/* Counters of the resident tables: block-table entries sent to the device so far, calls
 * that sent metadata, rows in use.                                                      */
void pa_kv_binding_stats(const PaKvBinding *b, uint64_t *table_entries_sent, uint64_t *calls,
                         uint32_t *rows_in_use);

/* ---- KvScaleManager, metal/kv_scale.rs:36-300 -------------------------------------------
 * alpha is clamped to [0, 1] (with_alpha); KvScaleManager::new uses 0.1.                 */
typedef struct PaKvScaleManager PaKvScaleManager;
typedef struct PaKvScaleStats {
  uint32_t num_layers_calibrated;
  float k_scale_min, k_scale_max, k_scale_mean, v_scale_min, v_scale_max, v_scale_mean;
} PaKvScaleStats;
PaKvScaleManager *pa_scale_create(uint32_t num_layers, float alpha);
void pa_scale_destroy(PaKvScaleManager *m);
uint32_t pa_scale_num_layers(const PaKvScaleManager *m);
float pa_scale_alpha(const PaKvScaleManager *m);
void pa_scale_init_default_scales(PaKvScaleManager *m);
float pa_scale_k(const PaKvScaleManager *m, uint32_t layer_idx);
float pa_scale_v(const PaKvScaleManager *m, uint32_t layer_idx);
int32_t pa_scale_is_calibrated(const PaKvScaleManager *m);
/* calibrate_layer / update_layer_ema on observed maxima of |x| (the host arithmetic)     */
void pa_scale_calibrate_layer_max(PaKvScaleManager *m, uint32_t layer_idx, float k_max_abs,
                                  float v_max_abs, float *k_scale, float *v_scale);
void pa_scale_update_layer_ema_max(PaKvScaleManager *m, uint32_t layer_idx, float k_max_abs,
                                   float v_max_abs, float *k_scale, float *v_scale);
/* calibrate_layer / update_layer_ema on device tensors of the cache dtype (any shape,
 * `count` elements each): max |x| by a reduction kernel, then the above.  dtype 0 = f16,
 * 1 = bf16.  Synchronises the stream (the reference evaluates the reduction too).        */
pa_status pa_scale_calibrate_layer(PaKvScaleManager *m, uint32_t layer_idx, const void *keys,
                                   const void *values, size_t count, int32_t dtype, int32_t ema,
                                   float *k_scale, float *v_scale, void *cuda_stream);
void pa_scale_set_scales(PaKvScaleManager *m, uint32_t layer_idx, float k_scale, float v_scale);
/* get_all_scales / load_scales: num_layers floats each (serialisation)                   */
void pa_scale_get_all_scales(const PaKvScaleManager *m, float *k_out, float *v_out);
void pa_scale_load_scales(PaKvScaleManager *m, const float *k, size_t nk, const float *v, size_t nv);
void pa_scale_reset(PaKvScaleManager *m);
void pa_scale_stats(const PaKvScaleManager *m, PaKvScaleStats *out);
/* The manager of a binding whose device cache is FP8 (paged_kv_cache.rs:226-309: the
 * cache owns one iff use_fp8); NULL otherwise.  Owned by the binding.  Its scales are
 * handed to the kernels as they are on every update / attention call of the binding,
 * which is what the reference does (paged_kv_cache.rs:826-834).                          */
PaKvScaleManager *pa_kv_scale_manager(PaKvBinding *b);

/* ---- PagedAttentionInputMetadata (+ builder), input_metadata.rs:29-278 ------------------- */
typedef struct PaInputMetadata PaInputMetadata;
PaInputMetadata *pa_metadata_create(const int32_t *block_tables, size_t num_table_entries,
                                    const int32_t *context_lens, size_t num_seqs,
                                    const int64_t *slot_mappings, size_t num_tokens,
                                    uint32_t max_context_len, int32_t is_prefill,
                                    uint32_t max_blocks_per_seq);
PaInputMetadata *pa_metadata_dummy(void);                         /* :88-104 */
void pa_metadata_destroy(PaInputMetadata *m);
uint32_t pa_metadata_num_seqs(const PaInputMetadata *m);
size_t pa_metadata_num_tokens(const PaInputMetadata *m);
int32_t pa_metadata_is_prefill(const PaInputMetadata *m);
uint32_t pa_metadata_max_context_len(const PaInputMetadata *m);
uint32_t pa_metadata_max_blocks_per_seq(const PaInputMetadata *m);
/* get_metal_buffers (:157-199): device copies of the three arrays on `device`, made on
 * first use and kept until pa_metadata_invalidate_buffers (:201-206).                    */
pa_status pa_metadata_device_buffers(PaInputMetadata *m, int32_t device, const int32_t **block_tables,
                                     const int32_t **context_lens, const int64_t **slot_mappings);
void pa_metadata_invalidate_buffers(PaInputMetadata *m);

/* ---- PagedAttentionLayer / PagedAttentionLayers, attention_layer.rs:41-478 ---------------
 * scale, softcap, k_scale, v_scale <= 0 in the parameters mean "default": 1/sqrt(head_size),
 * 1.0 (off), 1.0, 1.0 (attention_layer.rs:116-124).                                      */
typedef struct PaLayerParams {
  uint32_t layer_idx, num_heads, num_kv_heads, head_size;
  float scale;
  uint32_t block_size;
  float softcap;
  uint32_t use_fp8;
  float k_scale, v_scale;
} PaLayerParams;
typedef struct PaAttentionLayer PaAttentionLayer;
PaAttentionLayer *pa_layer_create(const PaLayerParams *p);
PaAttentionLayer *pa_layer_from_cache_config(uint32_t layer_idx, uint32_t num_heads,
                                             const PaHostConfig *cfg);
void pa_layer_destroy(PaAttentionLayer *l);
/* the layer's parameters with the defaults filled in */
void pa_layer_get(const PaAttentionLayer *l, PaLayerParams *out);
void pa_layer_set_kv_scales(PaAttentionLayer *l, float k_scale, float v_scale);
/* PagedAttentionLayer::forward (:217-384): writes the K/V of every token of
 * metadata.slot_mappings; a prefill batch then returns with *has_output = 0 (the caller
 * runs dense attention, as the reference's Ok(None)); a decode batch runs paged
 * attention into `out` and sets *has_output = 1.  queries/out [num_seqs, num_heads,
 * head_size], keys/values [num_tokens, num_kv_heads, head_size], on the device.          */
pa_status pa_layer_forward(const PaAttentionLayer *l, PaKvBinding *cache, void *out,
                           const void *queries, const void *keys, const void *values,
                           PaInputMetadata *metadata, int32_t *has_output, void *cuda_stream);
/* forward_decode (:399-416): an error for a prefill batch.                               */
pa_status pa_layer_forward_decode(const PaAttentionLayer *l, PaKvBinding *cache, void *out,
                                  const void *queries, const void *keys, const void *values,
                                  PaInputMetadata *metadata, void *cuda_stream);
typedef struct PaAttentionLayers PaAttentionLayers;
PaAttentionLayers *pa_layers_create(uint32_t num_layers, uint32_t num_heads, uint32_t num_kv_heads,
                                    uint32_t head_size, uint32_t block_size, int32_t use_fp8);
PaAttentionLayers *pa_layers_from_cache_config(uint32_t num_heads, const PaHostConfig *cfg);
void pa_layers_destroy(PaAttentionLayers *ls);
const PaAttentionLayer *pa_layers_get(const PaAttentionLayers *ls, uint32_t layer_idx); /* NULL past the end */
uint32_t pa_layers_num_layers(const PaAttentionLayers *ls);

/* CacheEngineManager::new (cache_engine.rs:137-216) as one call: validates the host
 * configuration, sizes the pool with calculate_num_blocks and creates host cache, device
 * cache (all layers; dtype 0 = f16, 1 = bf16; FP8 if the configuration says so) and the
 * binding.  The three handles are freed with their own destroy / free / unbind calls,
 * binding first.                                                                         */
pa_status pa_kv_create_bound(const PaHostConfig *cfg, int32_t device, uint32_t dtype, PaKvHost **kv_out,
                             PagedAttnCache **cache_out, PaKvBinding **binding_out);

#ifdef __cplusplus
}
#endif
#endif /* PAGED_ATTN_B200_HOST_H_ */
