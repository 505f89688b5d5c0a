// Host-side pool management of the paged KV cache: block allocator with reference
// counts, copy-on-write and an LRU prefix cache; per-sequence block tables; slot
// mapping and kernel-argument metadata; token tracker; continuous-batching
// scheduler.  Plain C++17, no CUDA.
//
// Behaviour follows the reference crate so that the integer results (block ids,
// slots, table layouts, scheduling decisions) are the ones its unit tests pin:
//   crates/mlx-paged-attn/src/block_allocator.rs   (BlockAllocator, hash_tokens)
//   crates/mlx-paged-attn/src/block_table.rs       (SequenceBlockTable, BlockTable)
//   crates/mlx-paged-attn/src/config.rs            (PagedAttentionConfig)
//   crates/mlx-paged-attn/src/paged_kv_cache.rs    (PagedKVCache host methods)
//   crates/mlx-paged-attn/src/token_tracker.rs     (TokenTracker, FNV-1a)
//   crates/mlx-paged-attn/src/scheduler.rs         (ContinuousBatchingScheduler)
//   crates/mlx-paged-attn/src/metal/kv_scale.rs    (KvScaleManager host maths)
#pragma once
#include <cstdint>
#include <deque>
#include <map>
#include <memory>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

namespace pa_host {

// ---- block_allocator.rs ---------------------------------------------------------
struct PhysicalBlock {
  uint32_t block_id;
  uint32_t ref_count = 1;  // sequences using the block (copy-on-write count)
  uint32_t num_tokens = 0;
  explicit PhysicalBlock(uint32_t id) : block_id(id) {}
  void incref() { ref_count++; }
  bool decref() { return ref_count-- == 1; }
  bool is_shared() const { return ref_count > 1; }
};
using BlockRef = std::shared_ptr<PhysicalBlock>;

class BlockAllocator {
 public:
  BlockAllocator(uint32_t num_blocks, uint32_t block_size);
  BlockRef allocate();                       // FIFO free list; null when exhausted
  void free(const BlockRef &block);          // returns to the pool when the count reaches 0
  BlockRef copy_on_write(const BlockRef &block);  // new block if shared, else null
  void register_prefix(const BlockRef &block, uint64_t hash);
  BlockRef lookup_prefix(uint64_t hash);     // increments the count on a hit
  uint32_t num_free_blocks() const { return (uint32_t)free_.size(); }
  uint32_t num_allocated_blocks() const { return (uint32_t)allocated_.size(); }
  uint32_t total_blocks() const { return num_blocks_; }
  uint32_t block_size() const { return block_size_; }
  bool can_allocate(uint32_t n) const { return num_free_blocks() >= n; }
  size_t max_prefix_cache_entries = 1024;
  size_t prefix_cache_len() const { return prefix_cache_.size(); }
  bool has_block_hash(uint32_t block_id) const { return block_hashes_.count(block_id) != 0; }
  void clear_lru_order() { lru_.clear(); }  // test hook: the reference test desynchronises it
  BlockRef get(uint32_t block_id) const {
    auto it = allocated_.find(block_id);
    return it == allocated_.end() ? nullptr : it->second;
  }

 private:
  std::deque<uint32_t> free_;
  std::unordered_map<uint32_t, BlockRef> allocated_;
  uint32_t num_blocks_, block_size_;
  std::unordered_map<uint64_t, BlockRef> prefix_cache_;
  std::unordered_map<uint32_t, uint64_t> block_hashes_;
  std::deque<uint64_t> lru_;
};

// SipHash-1-3 with a zero key over parent_hash (8 bytes LE) then each token (4 bytes
// LE): what Rust's DefaultHasher computes for block_allocator.rs:239-249.
uint64_t hash_tokens(const uint32_t *tokens, size_t n, uint64_t parent_hash);

// ---- block_table.rs ----------------------------------------------------------------
class SequenceBlockTable {
 public:
  SequenceBlockTable(uint32_t seq_id, uint32_t block_size) : seq_id(seq_id), block_size_(block_size) {}
  uint32_t seq_id;
  void add_block(BlockRef b) {
    blocks_.push_back(std::move(b));
    touch();
  }
  bool replace_block(size_t i, BlockRef b);
  // Changes whenever the list of blocks changes (a process-wide stamp, so a table
  // rebuilt from scratch never repeats an older value): lets a device-side copy of the
  // row tell "nothing to send" from "compare and send" in O(1).
  uint64_t version() const { return version_; }
  size_t num_blocks() const { return blocks_.size(); }
  uint32_t num_tokens() const { return num_tokens_; }
  void set_num_tokens(uint32_t n) { num_tokens_ = n; }
  const std::vector<BlockRef> &blocks() const { return blocks_; }
  bool is_last_block_full() const;
  uint32_t free_slots_in_last_block() const;
  uint32_t blocks_needed(uint32_t new_tokens) const;
  std::pair<uint32_t, uint32_t> slot_index(uint32_t token_pos) const;
  bool absolute_slot_index(uint32_t token_pos, int64_t *slot) const;

 private:
  void touch();
  std::vector<BlockRef> blocks_;
  uint32_t num_tokens_ = 0;
  uint32_t block_size_;
  uint64_t version_ = 0;
};

class BlockTable {
 public:
  explicit BlockTable(uint32_t block_size) : block_size_(block_size) {}
  uint32_t add_sequence();
  bool remove_sequence(uint32_t seq_id, SequenceBlockTable *out);  // swap-remove, as the reference
  SequenceBlockTable *get(uint32_t seq_id);
  const SequenceBlockTable *get(uint32_t seq_id) const;
  std::vector<uint32_t> seq_ids() const;
  size_t num_sequences() const { return tables_.size(); }
  const std::vector<SequenceBlockTable> &all_tables() const { return tables_; }
  std::vector<uint32_t> build_block_tables_array(size_t max_blocks_per_seq) const;
  std::vector<uint32_t> build_context_lens_array() const;

 private:
  std::vector<SequenceBlockTable> tables_;
  std::unordered_map<uint32_t, size_t> idx_;
  uint32_t next_seq_id_ = 0;
  uint32_t block_size_;
};

// ---- config.rs ---------------------------------------------------------------------
struct PagedAttentionConfig {
  uint32_t block_size = 32;
  uint32_t gpu_memory_mb = 4096;
  uint32_t head_size = 128;
  uint32_t num_kv_heads = 4;
  uint32_t num_layers = 28;
  bool use_fp8_cache = false;
  uint32_t max_seq_len = 8192;
  uint32_t max_batch_size = 256;
  std::string validate() const;  // empty = ok, else the reference's message
  uint32_t calculate_num_blocks() const;
  uint64_t max_cached_tokens() const { return (uint64_t)calculate_num_blocks() * block_size; }
};

// ---- token_tracker.rs ---------------------------------------------------------------
uint64_t compute_token_hash(const uint32_t *tokens, size_t n);  // FNV-1a over LE bytes

struct TokenTrackerStats {
  uint32_t num_tracked_blocks, total_tracked_tokens;
  float avg_tokens_per_block;
  uint32_t prefix_index_size;
};

class TokenTracker {
 public:
  explicit TokenTracker(uint32_t block_size) : block_size_(block_size), enabled_(true) {}
  static TokenTracker disabled() { TokenTracker t(0); t.enabled_ = false; return t; }
  bool is_enabled() const { return enabled_; }
  uint64_t track_tokens(uint32_t block_id, const uint32_t *tokens, size_t n, uint32_t start_offset);
  const std::vector<uint32_t> &get_block_tokens(uint32_t block_id) const;
  uint32_t get_block_token_count(uint32_t block_id) const { return (uint32_t)get_block_tokens(block_id).size(); }
  void remove_block(uint32_t block_id);
  void copy_block(uint32_t src, uint32_t dst);
  std::vector<std::pair<uint32_t, uint32_t>> find_prefix_matches(const uint32_t *tokens, size_t n) const;
  std::pair<std::vector<uint32_t>, uint32_t> find_longest_prefix(const uint32_t *tokens, size_t n) const;
  TokenTrackerStats stats() const;
  void clear();
  size_t memory_usage() const;

 private:
  std::unordered_map<uint32_t, std::vector<uint32_t>> block_tokens_;
  std::unordered_map<uint64_t, std::pair<uint32_t, uint32_t>> prefix_index_;
  uint32_t block_size_;
  bool enabled_;
};

// ---- input_metadata.rs ----------------------------------------------------------------
struct InputMetadata {
  std::vector<int32_t> block_tables;  // [num_seqs, max_blocks_per_seq], zero padded
  std::vector<int32_t> context_lens;
  std::vector<int64_t> slot_mappings;
  uint32_t max_context_len = 0;
  bool is_prefill = false;
  uint32_t num_seqs = 0;
  uint32_t max_blocks_per_seq = 0;
};

struct MemoryStats {
  uint32_t total_blocks, free_blocks, allocated_blocks, total_memory_mb, used_memory_mb;
  double utilization_percent;
};

// ---- paged_kv_cache.rs (host bookkeeping) ----------------------------------------------
class PagedKVCache {
 public:
  // error: set on failure (reference returns Err(String))
  static std::unique_ptr<PagedKVCache> create(const PagedAttentionConfig &cfg, std::string *error);
  bool add_sequence(uint32_t prompt_len, uint32_t *seq_id, std::string *error);
  bool remove_sequence(uint32_t seq_id, std::string *error);
  bool extend_sequence(uint32_t seq_id, uint32_t n, std::string *error);
  bool fork_sequence(uint32_t parent, uint32_t *child, std::string *error);
  // copied=false when the block is not shared; else (src,dst) is the device copy to issue
  bool handle_cow(uint32_t seq_id, size_t block_idx, bool *copied, uint32_t *src, uint32_t *dst,
                  std::string *error);
  bool can_allocate(uint32_t n) const { return alloc_.can_allocate(n); }
  uint32_t num_sequences() const { return (uint32_t)table_.num_sequences(); }
  uint32_t num_free_blocks() const { return alloc_.num_free_blocks(); }
  uint32_t total_blocks() const { return alloc_.total_blocks(); }
  uint32_t block_size() const { return cfg_.block_size; }
  uint32_t max_blocks_per_seq() const { return (cfg_.max_seq_len + cfg_.block_size - 1) / cfg_.block_size; }
  std::vector<uint32_t> get_context_lens() const { return table_.build_context_lens_array(); }
  std::vector<uint32_t> get_seq_ids() const { return table_.seq_ids(); }
  std::vector<uint32_t> build_block_tables() const { return table_.build_block_tables_array(max_blocks_per_seq()); }
  bool build_block_tables_batch(const uint32_t *seq_ids, size_t n, std::vector<std::vector<uint32_t>> *out,
                                std::string *error) const;
  bool get_slot_mapping(uint32_t seq_id, uint32_t start, uint32_t n, std::vector<int64_t> *out,
                        std::string *error) const;
  bool get_slot_mapping_batch(const uint32_t *seq_ids, const uint32_t *context_lens, const uint8_t *is_prefill,
                              const uint32_t *input_lens, size_t n, std::vector<int64_t> *out,
                              std::string *error) const;
  bool build_input_metadata(const uint32_t *seq_ids, const uint32_t *input_lens, const uint8_t *is_prefill,
                            size_t n, InputMetadata *out, std::string *error) const;
  MemoryStats get_memory_stats() const;
  const PagedAttentionConfig &config() const { return cfg_; }
  // token tracking
  bool track_sequence_tokens(uint32_t seq_id, const uint32_t *tokens, size_t n, uint32_t start_pos,
                             std::string *error);
  bool get_sequence_tokens(uint32_t seq_id, std::vector<uint32_t> *out, std::string *error) const;
  // Not in the reference: drop the tail of a sequence (rejected speculative tokens),
  // releasing blocks that no longer hold a token.
  bool truncate_sequence(uint32_t seq_id, uint32_t new_num_tokens, std::string *error);
  uint32_t sequence_num_tokens(uint32_t seq_id) const {
    const SequenceBlockTable *t = table_.get(seq_id);
    return t ? t->num_tokens() : 0;
  }
  // the block table of one sequence, or null
  const SequenceBlockTable *sequence(uint32_t seq_id) const { return table_.get(seq_id); }
  TokenTracker &tracker() { return tracker_; }
  const TokenTracker &tracker() const { return tracker_; }
  BlockAllocator &allocator() { return alloc_; }

 private:
  PagedKVCache(const PagedAttentionConfig &cfg, uint32_t num_blocks)
      : table_(cfg.block_size), alloc_(num_blocks, cfg.block_size), cfg_(cfg), tracker_(cfg.block_size) {}
  BlockTable table_;
  BlockAllocator alloc_;
  PagedAttentionConfig cfg_;
  TokenTracker tracker_;
};

// ---- scheduler.rs -------------------------------------------------------------------------
struct PendingRequest {
  std::string request_id;
  std::vector<uint32_t> prompt_tokens;
  uint32_t max_new_tokens = 0;
  int32_t priority = 0;
};
struct ActiveSequence {
  uint32_t seq_id;
  std::string request_id;
  std::vector<uint32_t> generated_tokens;
  uint32_t max_new_tokens, prompt_len;
  bool is_prefill;
  uint32_t position;
};
struct ScheduledBatch {
  std::vector<uint32_t> seq_ids;
  std::vector<std::string> request_ids;
  std::vector<std::vector<uint32_t>> input_tokens;
  std::vector<uint8_t> is_prefill;
  std::vector<uint32_t> context_lens;
  uint32_t total_tokens = 0, num_prefill = 0, num_decode = 0;
};
struct CompletedSequence {
  std::string request_id;
  std::vector<uint32_t> generated_tokens;
  std::string finish_reason;
  uint32_t total_tokens;
};
struct TokenOutput {
  uint32_t seq_id, token;
  bool is_eos;
};
struct SchedulerConfig {
  uint32_t max_batch_size = 32;
  uint32_t max_tokens_per_step = 4096;
  uint32_t max_prefill_per_step = 1;
  bool prioritize_decode = true;
  uint32_t eos_token_id = 151645;
};
struct SchedulerStats {
  uint32_t num_waiting, num_running, num_completed, num_prefill, num_decode, total_running_tokens;
};

class ContinuousBatchingScheduler {
 public:
  ContinuousBatchingScheduler(uint32_t block_size, const SchedulerConfig &cfg) : cfg_(cfg), block_size_(block_size) {}
  void add_request(PendingRequest r);  // higher priority first, FIFO within a priority
  bool schedule_step(PagedKVCache &cache, ScheduledBatch *out);  // false = nothing to run
  bool process_outputs(const std::vector<TokenOutput> &outputs, PagedKVCache &cache, std::string *error);
  std::vector<CompletedSequence> get_completed();
  bool is_empty() const { return waiting_.empty() && running_.empty(); }
  uint32_t num_waiting() const { return (uint32_t)waiting_.size(); }
  uint32_t num_running() const { return (uint32_t)running_.size(); }
  uint32_t num_completed() const { return (uint32_t)completed_.size(); }
  bool abort_request(const std::string &request_id, PagedKVCache &cache, bool *found, std::string *error);
  SchedulerStats get_stats() const;
  const ActiveSequence *running(uint32_t seq_id) const;

 private:
  std::deque<PendingRequest> waiting_;
  std::map<uint32_t, ActiveSequence> running_;  // ordered by seq id: a deterministic batch order
  std::vector<CompletedSequence> completed_;
  SchedulerConfig cfg_;
  uint32_t block_size_;
};

// ---- hybrid scheduler: chunked prefill + speculative verify + decode in one batch ----------
// The reference scheduler runs a whole prompt in one step and has no multi-token decode
// (scheduler.rs:237-242 says so).  This scheduler emits the mixed batches the variable-
// length attention entry takes: per sequence q_len new tokens on top of its cached
// prefix, with the slot mapping, context lengths (counting the new tokens) and
// cu_q_lens the kernels need.  Ordering contract as in the reference: the step's K/V
// are written first, then attention runs with context lengths that include them.
struct HybridConfig {
  uint32_t max_batch_size = 32;
  uint32_t max_tokens_per_step = 4096;
  uint32_t prefill_chunk_size = 1024;  // 0 = whole prompt in one step
  uint32_t max_prefill_per_step = 1;   // sequences in prefill per step
  bool prioritize_decode = true;
  uint32_t eos_token_id = 151645;
};
enum HybridKind : int32_t { kPrefillChunk = 0, kDecode = 1, kVerify = 2 };
struct HybridEntry {
  uint32_t seq_id;
  std::string request_id;
  int32_t kind;
  uint32_t q_len;    // new tokens this step
  uint32_t kv_len;   // tokens in the pool after this step's write
  bool needs_sample; // the caller samples after this step (false for a non-final prefill chunk)
  std::vector<uint32_t> tokens;  // the q_len input tokens
};
struct HybridBatch {
  std::vector<HybridEntry> entries;
  uint32_t total_tokens = 0, num_prefill = 0, num_decode = 0, num_verify = 0;
};
struct HybridOutput {
  uint32_t seq_id;
  uint32_t num_accepted;  // accepted draft tokens (0 for prefill / plain decode)
  uint32_t next_token;    // the token sampled after the accepted ones
  bool is_eos;
};
class HybridScheduler {
 public:
  HybridScheduler(uint32_t block_size, const HybridConfig &cfg) : cfg_(cfg), block_size_(block_size) {}
  void add_request(PendingRequest r);
  // draft tokens to verify at the sequence's next decode step (consumed by it)
  bool set_draft_tokens(uint32_t seq_id, const uint32_t *tokens, size_t n);
  bool schedule_step(PagedKVCache &cache, HybridBatch *out, std::string *error);
  // kernel arguments of the batch: tables [n, max_blocks_per_seq] zero padded, context
  // lens [n], cu_q_lens [n+1], slots [total_tokens]
  bool build_metadata(const PagedKVCache &cache, const HybridBatch &batch, InputMetadata *meta,
                      std::vector<int32_t> *cu_q_lens, std::string *error) const;
  bool process_outputs(const HybridBatch &batch, const std::vector<HybridOutput> &outputs, PagedKVCache &cache,
                       std::string *error);
  std::vector<CompletedSequence> get_completed();
  bool is_empty() const { return waiting_.empty() && running_.empty(); }
  uint32_t num_waiting() const { return (uint32_t)waiting_.size(); }
  uint32_t num_running() const { return (uint32_t)running_.size(); }

 private:
  struct Seq {
    uint32_t seq_id;
    std::string request_id;
    std::vector<uint32_t> prompt, generated, drafts;
    uint32_t max_new_tokens;
    uint32_t num_computed = 0;  // prompt tokens whose K/V are in the pool
  };
  std::deque<PendingRequest> waiting_;
  std::map<uint32_t, Seq> running_;
  std::vector<CompletedSequence> completed_;
  HybridConfig cfg_;
  uint32_t block_size_;
};

// ---- metal/kv_scale.rs -----------------------------------------------------------------------
float kv_compute_scale(float max_abs);  // 448 / max_abs, 1.0 for an all-zero tensor

struct KvScaleStats {
  uint32_t num_layers_calibrated;
  float k_scale_min, k_scale_max, k_scale_mean, v_scale_min, v_scale_max, v_scale_mean;
};

// Per-layer FP8 scales with one-shot and running (exponential moving average)
// calibration, crates/mlx-paged-attn/src/metal/kv_scale.rs:36-300.  The tensor
// reductions (max |x|) are done by the caller (on the device); this class holds the
// arithmetic and the state, the only checkpointable state of the paged cache
// (get_all_scales / load_scales, paged_kv_cache.rs:297-309).
class KvScaleManager {
 public:
  explicit KvScaleManager(uint32_t num_layers, float alpha = 0.1f);
  uint32_t num_layers() const { return num_layers_; }
  float alpha() const { return alpha_; }
  void init_default_scales();
  float k_scale(uint32_t layer) const;
  float v_scale(uint32_t layer) const;
  bool is_calibrated() const { return calibrated_; }
  // scales from the observed maxima of one batch
  std::pair<float, float> calibrate_layer(uint32_t layer, float k_max_abs, float v_max_abs);
  // running maxima: m = alpha * observed + (1 - alpha) * m (first observation: m = observed)
  std::pair<float, float> update_layer_ema(uint32_t layer, float k_max_abs, float v_max_abs);
  void set_scales(uint32_t layer, float k, float v);
  void get_all_scales(std::vector<float> *k, std::vector<float> *v) const;
  void load_scales(const float *k, size_t nk, const float *v, size_t nv);
  void reset();
  KvScaleStats stats() const;

 private:
  std::map<uint32_t, float> k_scales_, v_scales_, k_running_max_, v_running_max_;
  uint32_t num_layers_;
  float alpha_;
  bool calibrated_ = false;
};

// ---- attention_layer.rs (parameters; the dispatch lives next to the device code) ----------------
struct AttentionLayerParams {
  uint32_t layer_idx = 0, num_heads = 0, num_kv_heads = 0, head_size = 0;
  float scale = 0.f;        // <= 0: 1 / sqrt(head_size)
  uint32_t block_size = 16;
  float softcap = 0.f;      // <= 0: 1.0 (off)
  bool use_fp8 = false;
  float k_scale = 0.f, v_scale = 0.f;  // <= 0: 1.0
};
class AttentionLayer {
 public:
  explicit AttentionLayer(const AttentionLayerParams &p);
  static AttentionLayer from_cache_config(uint32_t layer_idx, uint32_t num_heads, const PagedAttentionConfig &cfg);
  uint32_t layer_idx, num_heads, num_kv_heads, head_size, block_size;
  float scale, softcap, k_scale, v_scale;
  bool use_fp8;
};

}  // namespace pa_host

// Handle types of the C ABI that more than one translation unit opens.
struct PaKvHost {
  std::unique_ptr<pa_host::PagedKVCache> kv;
};
struct PaKvScaleManager {
  pa_host::KvScaleManager m;
  explicit PaKvScaleManager(uint32_t num_layers, float alpha) : m(num_layers, alpha) {}
};
struct PaAttentionLayer {
  pa_host::AttentionLayer l;
  explicit PaAttentionLayer(const pa_host::AttentionLayer &x) : l(x) {}
};
