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
 * types (int32 tables [n, max_blocks_per_seq], int32 lens [n], int64 slots).          */
pa_status pa_kv_build_input_metadata(const PaKvHost *kv, const uint32_t *seq_ids,
                                     const uint32_t *input_lens, const uint8_t *is_prefill, size_t n,
                                     int32_t *block_tables_out, int32_t *context_lens_out,
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
 * int64 slots [total_tokens]                                                          */
pa_status pa_hybrid_batch_metadata(const PaHybridScheduler *s, const PaKvHost *kv, int32_t *block_tables,
                                   int32_t *context_lens, int32_t *cu_q_lens, int64_t *slots,
                                   size_t slots_cap, uint32_t *max_context_len);
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

#ifdef __cplusplus
}
#endif
#endif /* PAGED_ATTN_B200_HOST_H_ */
