// C ABI over the host-side pool management (include/paged_attn_b200_host.h).
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "../../include/paged_attn_b200_host.h"
#include "host_logic.hpp"

namespace pa {
int32_t set_error(int32_t code, const std::string &msg);
}
using namespace pa_host;

struct PaAllocator { BlockAllocator a; PaAllocator(uint32_t n, uint32_t bs) : a(n, bs) {} };
struct PaTracker { TokenTracker t; explicit PaTracker(TokenTracker tt) : t(std::move(tt)) {} };
struct PaScheduler {
  ContinuousBatchingScheduler s;
  ScheduledBatch batch;
  std::vector<CompletedSequence> done;
  PaScheduler(uint32_t bs, const SchedulerConfig &c) : s(bs, c) {}
};

struct PaHybridScheduler {
  HybridScheduler s;
  HybridBatch batch;
  std::vector<CompletedSequence> done;
  PaHybridScheduler(uint32_t bs, const HybridConfig &c) : s(bs, c) {}
};

namespace {
pa_status err(const std::string &msg, pa_status code = PA_ERR_INVALID_ARG) { return pa::set_error(code, msg); }
PagedAttentionConfig to_cfg(const PaHostConfig &c) {
  PagedAttentionConfig r;
  r.block_size = c.block_size;
  r.gpu_memory_mb = c.gpu_memory_mb;
  r.head_size = c.head_size;
  r.num_kv_heads = c.num_kv_heads;
  r.num_layers = c.num_layers;
  r.use_fp8_cache = c.use_fp8_cache != 0;
  r.max_seq_len = c.max_seq_len ? c.max_seq_len : 8192;
  r.max_batch_size = c.max_batch_size ? c.max_batch_size : 256;
  return r;
}
template <typename T>
size_t copy_out(const std::vector<T> &v, T *out, size_t cap) {
  if (out) std::memcpy(out, v.data(), sizeof(T) * (v.size() < cap ? v.size() : cap));
  return v.size();
}
}  // namespace

extern "C" {

void pa_host_config_default(PaHostConfig *out) {
  if (!out) return;
  const PagedAttentionConfig d;
  *out = PaHostConfig{d.block_size, d.gpu_memory_mb, d.head_size, d.num_kv_heads, d.num_layers, 0,
                      d.max_seq_len, d.max_batch_size};
}
pa_status pa_host_config_validate(const PaHostConfig *cfg) {
  if (!cfg) return err("config is null");
  const std::string msg = to_cfg(*cfg).validate();
  return msg.empty() ? PA_OK : err(msg);
}
uint32_t pa_host_config_num_blocks(const PaHostConfig *cfg) { return cfg ? to_cfg(*cfg).calculate_num_blocks() : 0; }
uint64_t pa_hash_tokens(const uint32_t *tokens, size_t n, uint64_t parent) { return hash_tokens(tokens, n, parent); }
uint64_t pa_compute_token_hash(const uint32_t *tokens, size_t n) { return compute_token_hash(tokens, n); }
float pa_kv_compute_scale(float max_abs) { return kv_compute_scale(max_abs); }
pa_status pa_shard_head_ranges(int32_t rank, int32_t world, int32_t num_q_heads, int32_t num_kv_heads,
                               int32_t *kv_begin, int32_t *kv_end, int32_t *q_begin, int32_t *q_end) {
  if (!kv_begin || !kv_end || !q_begin || !q_end) return err("null output pointer");
  if (world < 1 || rank < 0 || rank >= world) return err("bad rank/world");
  if (num_kv_heads < 1 || num_q_heads < 1 || num_q_heads % num_kv_heads)
    return err("query heads must be a positive multiple of kv heads");
  if (num_kv_heads % world) return err("kv heads do not split this many ways");
  const int32_t n = num_kv_heads / world, g = num_q_heads / num_kv_heads;
  *kv_begin = rank * n;
  *kv_end = (rank + 1) * n;
  *q_begin = *kv_begin * g;
  *q_end = *kv_end * g;
  return PA_OK;
}

/* ---- allocator ---- */
PaAllocator *pa_alloc_create(uint32_t num_blocks, uint32_t block_size) { return new PaAllocator(num_blocks, block_size); }
void pa_alloc_destroy(PaAllocator *a) { delete a; }
int64_t pa_alloc_allocate(PaAllocator *a) {
  if (!a) return -1;
  BlockRef b = a->a.allocate();
  return b ? (int64_t)b->block_id : -1;
}
pa_status pa_alloc_release(PaAllocator *a, uint32_t id) {
  BlockRef b = a ? a->a.get(id) : nullptr;
  if (!b) return err("block is not allocated");
  a->a.free(b);
  return PA_OK;
}
pa_status pa_alloc_incref(PaAllocator *a, uint32_t id) {
  BlockRef b = a ? a->a.get(id) : nullptr;
  if (!b) return err("block is not allocated");
  b->incref();
  return PA_OK;
}
int64_t pa_alloc_ref_count(PaAllocator *a, uint32_t id) {
  BlockRef b = a ? a->a.get(id) : nullptr;
  return b ? (int64_t)b->ref_count : -1;
}
int64_t pa_alloc_copy_on_write(PaAllocator *a, uint32_t id) {
  BlockRef b = a ? a->a.get(id) : nullptr;
  if (!b) return -1;
  BlockRef f = a->a.copy_on_write(b);
  return f ? (int64_t)f->block_id : -1;
}
pa_status pa_alloc_register_prefix(PaAllocator *a, uint32_t id, uint64_t hash) {
  BlockRef b = a ? a->a.get(id) : nullptr;
  if (!b) return err("block is not allocated");
  a->a.register_prefix(b, hash);
  return PA_OK;
}
int64_t pa_alloc_lookup_prefix(PaAllocator *a, uint64_t hash) {
  if (!a) return -1;
  BlockRef b = a->a.lookup_prefix(hash);
  return b ? (int64_t)b->block_id : -1;
}
uint32_t pa_alloc_num_free(const PaAllocator *a) { return a ? a->a.num_free_blocks() : 0; }
uint32_t pa_alloc_num_allocated(const PaAllocator *a) { return a ? a->a.num_allocated_blocks() : 0; }
uint32_t pa_alloc_total(const PaAllocator *a) { return a ? a->a.total_blocks() : 0; }
int32_t pa_alloc_can_allocate(const PaAllocator *a, uint32_t n) { return a && a->a.can_allocate(n); }
void pa_alloc_set_max_prefix_entries(PaAllocator *a, uint32_t n) { if (a) a->a.max_prefix_cache_entries = n; }
uint32_t pa_alloc_prefix_cache_len(const PaAllocator *a) { return a ? (uint32_t)a->a.prefix_cache_len() : 0; }
int32_t pa_alloc_has_block_hash(const PaAllocator *a, uint32_t id) { return a && a->a.has_block_hash(id); }
void pa_alloc_clear_lru_order(PaAllocator *a) { if (a) a->a.clear_lru_order(); }

/* ---- tracker ---- */
PaTracker *pa_tracker_create(uint32_t block_size, int32_t enabled) {
  return new PaTracker(enabled ? TokenTracker(block_size) : TokenTracker::disabled());
}
void pa_tracker_destroy(PaTracker *t) { delete t; }
int32_t pa_tracker_is_enabled(const PaTracker *t) { return t && t->t.is_enabled(); }
uint64_t pa_tracker_track_tokens(PaTracker *t, uint32_t block_id, const uint32_t *tokens, size_t n, uint32_t off) {
  return t ? t->t.track_tokens(block_id, tokens, n, off) : 0;
}
static uint32_t block_tokens_out(const TokenTracker &t, uint32_t block_id, uint32_t *out, size_t cap) {
  return (uint32_t)copy_out(t.get_block_tokens(block_id), out, cap);
}
uint32_t pa_tracker_get_block_tokens(const PaTracker *t, uint32_t block_id, uint32_t *out, size_t cap) {
  return t ? block_tokens_out(t->t, block_id, out, cap) : 0;
}
void pa_tracker_remove_block(PaTracker *t, uint32_t id) { if (t) t->t.remove_block(id); }
void pa_tracker_copy_block(PaTracker *t, uint32_t src, uint32_t dst) { if (t) t->t.copy_block(src, dst); }
static size_t matches_out(const TokenTracker &t, const uint32_t *tokens, size_t n, uint32_t *out, size_t cap) {
  const auto m = t.find_prefix_matches(tokens, n);
  for (size_t i = 0; i < m.size() && i < cap && out; i++) {
    out[2 * i] = m[i].first;
    out[2 * i + 1] = m[i].second;
  }
  return m.size();
}
static size_t longest_out(const TokenTracker &t, const uint32_t *tokens, size_t n, uint32_t *out, size_t cap,
                          uint32_t *matched) {
  const auto r = t.find_longest_prefix(tokens, n);
  if (matched) *matched = r.second;
  return copy_out(r.first, out, cap);
}
size_t pa_tracker_find_prefix_matches(const PaTracker *t, const uint32_t *tokens, size_t n, uint32_t *out, size_t cap) {
  return t ? matches_out(t->t, tokens, n, out, cap) : 0;
}
size_t pa_tracker_find_longest_prefix(const PaTracker *t, const uint32_t *tokens, size_t n, uint32_t *out,
                                      size_t cap, uint32_t *matched) {
  if (!t) { if (matched) *matched = 0; return 0; }
  return longest_out(t->t, tokens, n, out, cap, matched);
}
static void stats_out(const TokenTracker &t, PaTrackerStats *out) {
  const TokenTrackerStats s = t.stats();
  *out = PaTrackerStats{s.num_tracked_blocks, s.total_tracked_tokens, s.avg_tokens_per_block, s.prefix_index_size};
}
void pa_tracker_stats(const PaTracker *t, PaTrackerStats *out) { if (t && out) stats_out(t->t, out); }
void pa_tracker_clear(PaTracker *t) { if (t) t->t.clear(); }
size_t pa_tracker_memory_usage(const PaTracker *t) { return t ? t->t.memory_usage() : 0; }

/* ---- block table arithmetic ---- */
static SequenceBlockTable fake_table(uint32_t num_blocks, uint32_t num_tokens, uint32_t bs) {
  SequenceBlockTable t(0, bs);
  for (uint32_t i = 0; i < num_blocks; i++) t.add_block(std::make_shared<PhysicalBlock>(i));
  t.set_num_tokens(num_tokens);
  return t;
}
uint32_t pa_table_free_slots_in_last_block(uint32_t nb, uint32_t nt, uint32_t bs) {
  return bs ? fake_table(nb, nt, bs).free_slots_in_last_block() : 0;
}
uint32_t pa_table_blocks_needed(uint32_t nb, uint32_t nt, uint32_t bs, uint32_t new_tokens) {
  return bs ? fake_table(nb, nt, bs).blocks_needed(new_tokens) : 0;
}
int32_t pa_table_is_last_block_full(uint32_t nt, uint32_t bs) { return bs && fake_table(0, nt, bs).is_last_block_full(); }
void pa_table_slot_index(uint32_t pos, uint32_t bs, uint32_t *blk, uint32_t *off) {
  if (!bs || !blk || !off) return;
  const auto r = SequenceBlockTable(0, bs).slot_index(pos);
  *blk = r.first;
  *off = r.second;
}

/* ---- kv cache host ---- */
pa_status pa_kv_create(const PaHostConfig *cfg, PaKvHost **out) {
  if (!cfg || !out) return err("null argument");
  *out = nullptr;
  std::string e;
  auto kv = PagedKVCache::create(to_cfg(*cfg), &e);
  if (!kv) return err(e);
  *out = new PaKvHost{std::move(kv)};
  return PA_OK;
}
void pa_kv_destroy(PaKvHost *kv) { delete kv; }
#define KV_CALL(expr)                      \
  do {                                     \
    if (!kv) return err("cache is null");  \
    std::string e;                         \
    if (!(expr)) return err(e);            \
    return PA_OK;                          \
  } while (0)
pa_status pa_kv_add_sequence(PaKvHost *kv, uint32_t prompt_len, uint32_t *seq_id) {
  if (!seq_id) return err("seq_id is null");
  KV_CALL(kv->kv->add_sequence(prompt_len, seq_id, &e));
}
pa_status pa_kv_remove_sequence(PaKvHost *kv, uint32_t seq_id) { KV_CALL(kv->kv->remove_sequence(seq_id, &e)); }
pa_status pa_kv_extend_sequence(PaKvHost *kv, uint32_t seq_id, uint32_t n) { KV_CALL(kv->kv->extend_sequence(seq_id, n, &e)); }
pa_status pa_kv_extend_sequences(PaKvHost *kv, const uint32_t *seq_ids, size_t n, uint32_t num_tokens) {
  if (!kv || (!seq_ids && n)) return err("null argument");
  std::string e;
  for (size_t i = 0; i < n; i++)
    if (!kv->kv->extend_sequence(seq_ids[i], num_tokens, &e)) return err(e);
  return PA_OK;
}
pa_status pa_kv_fork_sequence(PaKvHost *kv, uint32_t parent, uint32_t *child) {
  if (!child) return err("child is null");
  KV_CALL(kv->kv->fork_sequence(parent, child, &e));
}
pa_status pa_kv_handle_cow(PaKvHost *kv, uint32_t seq_id, uint32_t block_idx, int32_t *copied, uint32_t *src,
                           uint32_t *dst) {
  if (!kv || !copied || !src || !dst) return err("null argument");
  std::string e;
  bool c = false;
  if (!kv->kv->handle_cow(seq_id, block_idx, &c, src, dst, &e)) return err(e);
  *copied = c ? 1 : 0;
  return PA_OK;
}
int32_t pa_kv_can_allocate(const PaKvHost *kv, uint32_t n) { return kv && kv->kv->can_allocate(n); }
uint32_t pa_kv_num_sequences(const PaKvHost *kv) { return kv ? kv->kv->num_sequences() : 0; }
uint32_t pa_kv_num_free_blocks(const PaKvHost *kv) { return kv ? kv->kv->num_free_blocks() : 0; }
uint32_t pa_kv_total_blocks(const PaKvHost *kv) { return kv ? kv->kv->total_blocks() : 0; }
uint32_t pa_kv_block_size(const PaKvHost *kv) { return kv ? kv->kv->block_size() : 0; }
uint32_t pa_kv_max_blocks_per_seq(const PaKvHost *kv) { return kv ? kv->kv->max_blocks_per_seq() : 0; }
size_t pa_kv_get_context_lens(const PaKvHost *kv, uint32_t *out, size_t cap) {
  return kv ? copy_out(kv->kv->get_context_lens(), out, cap) : 0;
}
size_t pa_kv_get_seq_ids(const PaKvHost *kv, uint32_t *out, size_t cap) {
  return kv ? copy_out(kv->kv->get_seq_ids(), out, cap) : 0;
}
size_t pa_kv_build_block_tables(const PaKvHost *kv, uint32_t *out, size_t cap) {
  return kv ? copy_out(kv->kv->build_block_tables(), out, cap) : 0;
}
pa_status pa_kv_sequence_blocks(const PaKvHost *kv, uint32_t seq_id, uint32_t *out, size_t cap, size_t *count) {
  if (!kv || !count) return err("null argument");
  std::string e;
  std::vector<std::vector<uint32_t>> t;
  if (!kv->kv->build_block_tables_batch(&seq_id, 1, &t, &e)) return err(e);
  *count = copy_out(t[0], out, cap);
  return PA_OK;
}
pa_status pa_kv_get_slot_mapping(const PaKvHost *kv, uint32_t seq_id, uint32_t start, uint32_t n, int64_t *out) {
  if (!kv || (!out && n)) return err("null argument");
  std::string e;
  std::vector<int64_t> v;
  if (!kv->kv->get_slot_mapping(seq_id, start, n, &v, &e)) return err(e);
  copy_out(v, out, n);
  return PA_OK;
}
pa_status pa_kv_get_slot_mapping_batch(const PaKvHost *kv, const uint32_t *seq_ids, const uint32_t *ctx,
                                       const uint8_t *is_prefill, const uint32_t *input_lens, size_t n,
                                       int64_t *out, size_t cap, size_t *count) {
  if (!kv || !seq_ids || !count) return err("null argument");
  std::string e;
  std::vector<int64_t> v;
  if (!kv->kv->get_slot_mapping_batch(seq_ids, ctx, is_prefill, input_lens, n, &v, &e)) return err(e);
  if (v.size() > cap) return err("slot buffer too small");
  *count = copy_out(v, out, cap);
  return PA_OK;
}
pa_status pa_kv_build_input_metadata(const PaKvHost *kv, const uint32_t *seq_ids, const uint32_t *input_lens,
                                     const uint8_t *is_prefill, size_t n, int32_t *tables, size_t tables_cap,
                                     int32_t *lens, size_t lens_cap, int64_t *slots, size_t slots_cap,
                                     size_t *num_slots, uint32_t *max_ctx, int32_t *batch_is_prefill) {
  if (!kv || !seq_ids || !tables || !lens || !slots || !num_slots) return err("null argument");
  std::string e;
  InputMetadata m;
  if (!kv->kv->build_input_metadata(seq_ids, input_lens, is_prefill, n, &m, &e)) return err(e);
  if (m.block_tables.size() > tables_cap)
    return err("block table buffer too small: need " + std::to_string(m.block_tables.size()) + " entries (" +
               std::to_string(n) + " x max_blocks_per_seq " + std::to_string(m.max_blocks_per_seq) + ")");
  if (m.context_lens.size() > lens_cap) return err("context length buffer too small");
  if (m.slot_mappings.size() > slots_cap) return err("slot buffer too small");
  copy_out(m.block_tables, tables, m.block_tables.size());
  copy_out(m.context_lens, lens, m.context_lens.size());
  *num_slots = copy_out(m.slot_mappings, slots, slots_cap);
  if (max_ctx) *max_ctx = m.max_context_len;
  if (batch_is_prefill) *batch_is_prefill = m.is_prefill ? 1 : 0;
  return PA_OK;
}
void pa_kv_memory_stats(const PaKvHost *kv, PaMemoryStats *out) {
  if (!kv || !out) return;
  const MemoryStats s = kv->kv->get_memory_stats();
  *out = PaMemoryStats{s.total_blocks, s.free_blocks, s.allocated_blocks, s.total_memory_mb, s.used_memory_mb,
                       s.utilization_percent};
}
pa_status pa_kv_track_sequence_tokens(PaKvHost *kv, uint32_t seq_id, const uint32_t *tokens, size_t n, uint32_t start) {
  KV_CALL(kv->kv->track_sequence_tokens(seq_id, tokens, n, start, &e));
}
pa_status pa_kv_get_sequence_tokens(const PaKvHost *kv, uint32_t seq_id, uint32_t *out, size_t cap, size_t *count) {
  if (!kv || !count) return err("null argument");
  std::string e;
  std::vector<uint32_t> v;
  if (!kv->kv->get_sequence_tokens(seq_id, &v, &e)) return err(e);
  *count = copy_out(v, out, cap);
  return PA_OK;
}
size_t pa_kv_find_prefix_matches(const PaKvHost *kv, const uint32_t *tokens, size_t n, uint32_t *out, size_t cap) {
  return kv ? matches_out(kv->kv->tracker(), tokens, n, out, cap) : 0;
}
size_t pa_kv_find_longest_prefix(const PaKvHost *kv, const uint32_t *tokens, size_t n, uint32_t *out, size_t cap,
                                 uint32_t *matched) {
  if (!kv) { if (matched) *matched = 0; return 0; }
  return longest_out(kv->kv->tracker(), tokens, n, out, cap, matched);
}
uint32_t pa_kv_get_block_tokens(const PaKvHost *kv, uint32_t block_id, uint32_t *out, size_t cap) {
  return kv ? block_tokens_out(kv->kv->tracker(), block_id, out, cap) : 0;
}
void pa_kv_tracker_stats(const PaKvHost *kv, PaTrackerStats *out) { if (kv && out) stats_out(kv->kv->tracker(), out); }
size_t pa_kv_tracker_memory(const PaKvHost *kv) { return kv ? kv->kv->tracker().memory_usage() : 0; }

/* ---- scheduler ---- */
void pa_sched_config_default(PaSchedulerConfig *out) {
  if (!out) return;
  const SchedulerConfig d;
  *out = PaSchedulerConfig{d.max_batch_size, d.max_tokens_per_step, d.max_prefill_per_step,
                           d.prioritize_decode ? 1u : 0u, d.eos_token_id};
}
PaScheduler *pa_sched_create(uint32_t block_size, const PaSchedulerConfig *c) {
  SchedulerConfig cfg;
  if (c) {
    cfg.max_batch_size = c->max_batch_size;
    cfg.max_tokens_per_step = c->max_tokens_per_step;
    cfg.max_prefill_per_step = c->max_prefill_per_step;
    cfg.prioritize_decode = c->prioritize_decode != 0;
    cfg.eos_token_id = c->eos_token_id;
  }
  return new PaScheduler(block_size, cfg);
}
void pa_sched_destroy(PaScheduler *s) { delete s; }
void pa_sched_add_request(PaScheduler *s, const char *request_id, const uint32_t *tokens, size_t n,
                          uint32_t max_new_tokens, int32_t priority) {
  if (!s || !request_id) return;
  PendingRequest r;
  r.request_id = request_id;
  if (tokens) r.prompt_tokens.assign(tokens, tokens + n);
  r.max_new_tokens = max_new_tokens;
  r.priority = priority;
  s->s.add_request(std::move(r));
}
uint32_t pa_sched_schedule_step(PaScheduler *s, PaKvHost *kv) {
  if (!s || !kv) return 0;
  s->batch = ScheduledBatch();
  if (!s->s.schedule_step(*kv->kv, &s->batch)) return 0;
  return (uint32_t)s->batch.seq_ids.size();
}
void pa_sched_batch_totals(const PaScheduler *s, PaBatchTotals *out) {
  if (s && out) *out = PaBatchTotals{s->batch.total_tokens, s->batch.num_prefill, s->batch.num_decode};
}
pa_status pa_sched_batch_entry(const PaScheduler *s, uint32_t i, uint32_t *seq_id, int32_t *is_prefill,
                               uint32_t *context_len, uint32_t *num_input) {
  if (!s || i >= s->batch.seq_ids.size()) return err("batch index out of range");
  if (seq_id) *seq_id = s->batch.seq_ids[i];
  if (is_prefill) *is_prefill = s->batch.is_prefill[i];
  if (context_len) *context_len = s->batch.context_lens[i];
  if (num_input) *num_input = (uint32_t)s->batch.input_tokens[i].size();
  return PA_OK;
}
uint32_t pa_sched_batch_tokens(const PaScheduler *s, uint32_t i, uint32_t *out, size_t cap) {
  if (!s || i >= s->batch.seq_ids.size()) return 0;
  return (uint32_t)copy_out(s->batch.input_tokens[i], out, cap);
}
const char *pa_sched_batch_request_id(const PaScheduler *s, uint32_t i) {
  return (s && i < s->batch.request_ids.size()) ? s->batch.request_ids[i].c_str() : "";
}
pa_status pa_sched_process_outputs(PaScheduler *s, PaKvHost *kv, const uint32_t *seq_ids, const uint32_t *tokens,
                                   const uint8_t *is_eos, size_t n) {
  if (!s || !kv || (n && (!seq_ids || !tokens))) return err("null argument");
  std::vector<TokenOutput> o;
  for (size_t i = 0; i < n; i++) o.push_back(TokenOutput{seq_ids[i], tokens[i], is_eos && is_eos[i]});
  std::string e;
  if (!s->s.process_outputs(o, *kv->kv, &e)) return err(e);
  return PA_OK;
}
uint32_t pa_sched_take_completed(PaScheduler *s) {
  if (!s) return 0;
  s->done = s->s.get_completed();
  return (uint32_t)s->done.size();
}
const char *pa_sched_completed_request_id(const PaScheduler *s, uint32_t i) {
  return (s && i < s->done.size()) ? s->done[i].request_id.c_str() : "";
}
const char *pa_sched_completed_finish_reason(const PaScheduler *s, uint32_t i) {
  return (s && i < s->done.size()) ? s->done[i].finish_reason.c_str() : "";
}
uint32_t pa_sched_completed_tokens(const PaScheduler *s, uint32_t i, uint32_t *out, size_t cap, uint32_t *total) {
  if (!s || i >= s->done.size()) return 0;
  if (total) *total = s->done[i].total_tokens;
  return (uint32_t)copy_out(s->done[i].generated_tokens, out, cap);
}
pa_status pa_sched_abort_request(PaScheduler *s, PaKvHost *kv, const char *request_id, int32_t *found) {
  if (!s || !kv || !request_id || !found) return err("null argument");
  bool f = false;
  std::string e;
  if (!s->s.abort_request(request_id, *kv->kv, &f, &e)) return err(e);
  *found = f ? 1 : 0;
  return PA_OK;
}
int32_t pa_sched_is_empty(const PaScheduler *s) { return !s || s->s.is_empty(); }
void pa_sched_stats(const PaScheduler *s, PaSchedulerStats *out) {
  if (!s || !out) return;
  const SchedulerStats st = s->s.get_stats();
  *out = PaSchedulerStats{st.num_waiting, st.num_running, st.num_completed, st.num_prefill, st.num_decode,
                          st.total_running_tokens};
}
int32_t pa_sched_running_is_prefill(const PaScheduler *s, uint32_t seq_id) {
  const ActiveSequence *a = s ? s->s.running(seq_id) : nullptr;
  return a ? (a->is_prefill ? 1 : 0) : -1;
}

/* ---- hybrid scheduler ---- */
void pa_hybrid_config_default(PaHybridConfig *out) {
  if (!out) return;
  const HybridConfig d;
  *out = PaHybridConfig{d.max_batch_size, d.max_tokens_per_step, d.prefill_chunk_size, d.max_prefill_per_step,
                        d.prioritize_decode ? 1u : 0u, d.eos_token_id};
}
PaHybridScheduler *pa_hybrid_create(uint32_t block_size, const PaHybridConfig *c) {
  HybridConfig cfg;
  if (c) {
    cfg.max_batch_size = c->max_batch_size;
    cfg.max_tokens_per_step = c->max_tokens_per_step;
    cfg.prefill_chunk_size = c->prefill_chunk_size;
    cfg.max_prefill_per_step = c->max_prefill_per_step;
    cfg.prioritize_decode = c->prioritize_decode != 0;
    cfg.eos_token_id = c->eos_token_id;
  }
  return new PaHybridScheduler(block_size, cfg);
}
void pa_hybrid_destroy(PaHybridScheduler *s) { delete s; }
void pa_hybrid_add_request(PaHybridScheduler *s, const char *request_id, const uint32_t *tokens, size_t n,
                           uint32_t max_new_tokens, int32_t priority) {
  if (!s || !request_id) return;
  PendingRequest r;
  r.request_id = request_id;
  if (tokens) r.prompt_tokens.assign(tokens, tokens + n);
  r.max_new_tokens = max_new_tokens;
  r.priority = priority;
  s->s.add_request(std::move(r));
}
pa_status pa_hybrid_set_draft_tokens(PaHybridScheduler *s, uint32_t seq_id, const uint32_t *tokens, size_t n) {
  if (!s || (n && !tokens)) return err("null argument");
  return s->s.set_draft_tokens(seq_id, tokens, n) ? PA_OK : err("sequence is not running in decode");
}
uint32_t pa_hybrid_schedule_step(PaHybridScheduler *s, PaKvHost *kv) {
  if (!s || !kv) return 0;
  s->batch = HybridBatch();
  std::string e;
  if (!s->s.schedule_step(*kv->kv, &s->batch, &e)) return 0;
  return (uint32_t)s->batch.entries.size();
}
void pa_hybrid_batch_totals(const PaHybridScheduler *s, PaHybridTotals *out) {
  if (s && out)
    *out = PaHybridTotals{s->batch.total_tokens, s->batch.num_prefill, s->batch.num_decode, s->batch.num_verify};
}
pa_status pa_hybrid_batch_entry(const PaHybridScheduler *s, uint32_t i, uint32_t *seq_id, int32_t *kind,
                                uint32_t *q_len, uint32_t *kv_len, int32_t *needs_sample) {
  if (!s || i >= s->batch.entries.size()) return err("batch index out of range");
  const HybridEntry &e = s->batch.entries[i];
  if (seq_id) *seq_id = e.seq_id;
  if (kind) *kind = e.kind;
  if (q_len) *q_len = e.q_len;
  if (kv_len) *kv_len = e.kv_len;
  if (needs_sample) *needs_sample = e.needs_sample ? 1 : 0;
  return PA_OK;
}
uint32_t pa_hybrid_batch_tokens(const PaHybridScheduler *s, uint32_t i, uint32_t *out, size_t cap) {
  if (!s || i >= s->batch.entries.size()) return 0;
  return (uint32_t)copy_out(s->batch.entries[i].tokens, out, cap);
}
const char *pa_hybrid_batch_request_id(const PaHybridScheduler *s, uint32_t i) {
  return (s && i < s->batch.entries.size()) ? s->batch.entries[i].request_id.c_str() : "";
}
pa_status pa_hybrid_batch_metadata(const PaHybridScheduler *s, const PaKvHost *kv, int32_t *tables,
                                   size_t tables_cap, int32_t *lens, int32_t *cu_q, size_t seqs_cap,
                                   int64_t *slots, size_t slots_cap, uint32_t *max_ctx) {
  if (!s || !kv || !tables || !lens || !cu_q || !slots) return err("null argument");
  InputMetadata m;
  std::vector<int32_t> cu;
  std::string e;
  if (!s->s.build_metadata(*kv->kv, s->batch, &m, &cu, &e)) return err(e);
  if (m.block_tables.size() > tables_cap)
    return err("block table buffer too small: need " + std::to_string(m.block_tables.size()) + " entries");
  if (m.context_lens.size() > seqs_cap) return err("context length / cu_q_lens buffers too small");
  if (m.slot_mappings.size() > slots_cap) return err("slot buffer too small");
  copy_out(m.block_tables, tables, m.block_tables.size());
  copy_out(m.context_lens, lens, m.context_lens.size());
  copy_out(cu, cu_q, cu.size());
  copy_out(m.slot_mappings, slots, slots_cap);
  if (max_ctx) *max_ctx = m.max_context_len;
  return PA_OK;
}
pa_status pa_hybrid_process_outputs(PaHybridScheduler *s, PaKvHost *kv, const uint32_t *seq_ids,
                                    const uint32_t *num_accepted, const uint32_t *next_tokens,
                                    const uint8_t *is_eos, size_t n) {
  if (!s || !kv || (n && (!seq_ids || !next_tokens))) return err("null argument");
  std::vector<HybridOutput> o;
  for (size_t i = 0; i < n; i++)
    o.push_back(HybridOutput{seq_ids[i], num_accepted ? num_accepted[i] : 0, next_tokens[i], is_eos && is_eos[i]});
  std::string e;
  if (!s->s.process_outputs(s->batch, o, *kv->kv, &e)) return err(e);
  return PA_OK;
}
uint32_t pa_hybrid_take_completed(PaHybridScheduler *s) {
  if (!s) return 0;
  s->done = s->s.get_completed();
  return (uint32_t)s->done.size();
}
const char *pa_hybrid_completed_request_id(const PaHybridScheduler *s, uint32_t i) {
  return (s && i < s->done.size()) ? s->done[i].request_id.c_str() : "";
}
const char *pa_hybrid_completed_finish_reason(const PaHybridScheduler *s, uint32_t i) {
  return (s && i < s->done.size()) ? s->done[i].finish_reason.c_str() : "";
}
uint32_t pa_hybrid_completed_tokens(const PaHybridScheduler *s, uint32_t i, uint32_t *out, size_t cap,
                                    uint32_t *total) {
  if (!s || i >= s->done.size()) return 0;
  if (total) *total = s->done[i].total_tokens;
  return (uint32_t)copy_out(s->done[i].generated_tokens, out, cap);
}
int32_t pa_hybrid_is_empty(const PaHybridScheduler *s) { return !s || s->s.is_empty(); }
uint32_t pa_hybrid_num_waiting(const PaHybridScheduler *s) { return s ? s->s.num_waiting() : 0; }
uint32_t pa_hybrid_num_running(const PaHybridScheduler *s) { return s ? s->s.num_running() : 0; }
pa_status pa_kv_truncate_sequence(PaKvHost *kv, uint32_t seq_id, uint32_t n) {
  KV_CALL(kv->kv->truncate_sequence(seq_id, n, &e));
}

}  // extern "C"
