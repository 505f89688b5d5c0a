// Implementation of the host-side pool management (see host_logic.hpp).
#include "host_logic.hpp"

#include <algorithm>
#include <atomic>
#include <cmath>

namespace pa_host {

// ---- BlockAllocator (crates/mlx-paged-attn/src/block_allocator.rs:62-236) ----------
BlockAllocator::BlockAllocator(uint32_t num_blocks, uint32_t block_size)
    : num_blocks_(num_blocks), block_size_(block_size) {
  for (uint32_t i = 0; i < num_blocks; i++) free_.push_back(i);
  allocated_.reserve(num_blocks);
}

BlockRef BlockAllocator::allocate() {
  if (free_.empty()) return nullptr;
  const uint32_t id = free_.front();
  free_.pop_front();
  auto b = std::make_shared<PhysicalBlock>(id);
  allocated_[id] = b;
  return b;
}

void BlockAllocator::free(const BlockRef &block) {
  const uint32_t id = block->block_id;
  if (!block->decref()) return;
  allocated_.erase(id);
  auto it = block_hashes_.find(id);
  if (it != block_hashes_.end()) {
    const uint64_t hash = it->second;
    block_hashes_.erase(it);
    prefix_cache_.erase(hash);
    lru_.erase(std::remove(lru_.begin(), lru_.end(), hash), lru_.end());
  }
  free_.push_back(id);
}

BlockRef BlockAllocator::copy_on_write(const BlockRef &block) {
  if (!block->is_shared()) return nullptr;
  BlockRef fresh = allocate();
  if (!fresh) return nullptr;
  block->decref();
  return fresh;
}

void BlockAllocator::register_prefix(const BlockRef &block, uint64_t hash) {
  if (max_prefix_cache_entries == 0) return;
  while (prefix_cache_.size() >= max_prefix_cache_entries) {
    if (lru_.empty()) break;  // desynchronised: do not spin
    const uint64_t old = lru_.front();
    lru_.pop_front();
    auto it = prefix_cache_.find(old);
    if (it != prefix_cache_.end()) {
      block_hashes_.erase(it->second->block_id);
      prefix_cache_.erase(it);
    }
  }
  lru_.erase(std::remove(lru_.begin(), lru_.end(), hash), lru_.end());
  lru_.push_back(hash);
  block_hashes_[block->block_id] = hash;
  prefix_cache_[hash] = block;
}

BlockRef BlockAllocator::lookup_prefix(uint64_t hash) {
  auto it = prefix_cache_.find(hash);
  if (it == prefix_cache_.end()) return nullptr;
  lru_.erase(std::remove(lru_.begin(), lru_.end(), hash), lru_.end());
  lru_.push_back(hash);
  it->second->incref();
  return it->second;
}

namespace {
inline uint64_t rotl(uint64_t x, int b) { return (x << b) | (x >> (64 - b)); }
struct Sip13 {
  uint64_t v0 = 0x736f6d6570736575ull, v1 = 0x646f72616e646f6dull, v2 = 0x6c7967656e657261ull,
           v3 = 0x7465646279746573ull;  // zero key
  uint64_t tail = 0;
  int ntail = 0;
  uint64_t length = 0;
  void round() {
    v0 += v1; v1 = rotl(v1, 13); v1 ^= v0; v0 = rotl(v0, 32);
    v2 += v3; v3 = rotl(v3, 16); v3 ^= v2;
    v0 += v3; v3 = rotl(v3, 21); v3 ^= v0;
    v2 += v1; v1 = rotl(v1, 17); v1 ^= v2; v2 = rotl(v2, 32);
  }
  void write(const uint8_t *p, size_t n) {
    length += n;
    for (size_t i = 0; i < n; i++) {
      tail |= (uint64_t)p[i] << (8 * ntail);
      if (++ntail == 8) {
        v3 ^= tail; round(); v0 ^= tail;
        tail = 0; ntail = 0;
      }
    }
  }
  uint64_t finish() {
    const uint64_t b = (length << 56) | tail;
    v3 ^= b; round(); v0 ^= b;
    v2 ^= 0xff;
    round(); round(); round();
    return v0 ^ v1 ^ v2 ^ v3;
  }
};
}  // namespace

uint64_t hash_tokens(const uint32_t *tokens, size_t n, uint64_t parent_hash) {
  Sip13 h;
  uint8_t buf[8];
  for (int i = 0; i < 8; i++) buf[i] = (uint8_t)(parent_hash >> (8 * i));
  h.write(buf, 8);
  for (size_t t = 0; t < n; t++) {
    for (int i = 0; i < 4; i++) buf[i] = (uint8_t)(tokens[t] >> (8 * i));
    h.write(buf, 4);
  }
  return h.finish();
}

// ---- block tables (crates/mlx-paged-attn/src/block_table.rs) -----------------------------
void SequenceBlockTable::touch() {
  static std::atomic<uint64_t> stamp{0};
  version_ = stamp.fetch_add(1, std::memory_order_relaxed) + 1;
}

bool SequenceBlockTable::replace_block(size_t i, BlockRef b) {
  if (i >= blocks_.size()) return false;
  touch();
  blocks_[i] = std::move(b);
  return true;
}
bool SequenceBlockTable::is_last_block_full() const {
  return num_tokens_ % block_size_ == 0 && num_tokens_ > 0;
}
uint32_t SequenceBlockTable::free_slots_in_last_block() const {
  if (blocks_.empty()) return 0;
  const uint32_t in_last = num_tokens_ % block_size_;
  if (in_last == 0 && num_tokens_ > 0) return 0;
  return block_size_ - in_last;
}
uint32_t SequenceBlockTable::blocks_needed(uint32_t new_tokens) const {
  const uint32_t free_slots = free_slots_in_last_block();
  if (new_tokens <= free_slots) return 0;
  return (new_tokens - free_slots + block_size_ - 1) / block_size_;
}
std::pair<uint32_t, uint32_t> SequenceBlockTable::slot_index(uint32_t token_pos) const {
  return {token_pos / block_size_, token_pos % block_size_};
}
bool SequenceBlockTable::absolute_slot_index(uint32_t token_pos, int64_t *slot) const {
  const auto [blk, off] = slot_index(token_pos);
  if (blk >= blocks_.size()) return false;
  *slot = (int64_t)blocks_[blk]->block_id * (int64_t)block_size_ + (int64_t)off;
  return true;
}

uint32_t BlockTable::add_sequence() {
  const uint32_t id = next_seq_id_++;
  idx_[id] = tables_.size();
  tables_.emplace_back(id, block_size_);
  return id;
}
bool BlockTable::remove_sequence(uint32_t seq_id, SequenceBlockTable *out) {
  auto it = idx_.find(seq_id);
  if (it == idx_.end()) return false;
  const size_t i = it->second;
  idx_.erase(it);
  if (out) *out = tables_[i];
  if (i + 1 != tables_.size()) {
    tables_[i] = std::move(tables_.back());
    idx_[tables_[i].seq_id] = i;
  }
  tables_.pop_back();
  return true;
}
SequenceBlockTable *BlockTable::get(uint32_t seq_id) {
  auto it = idx_.find(seq_id);
  return it == idx_.end() ? nullptr : &tables_[it->second];
}
const SequenceBlockTable *BlockTable::get(uint32_t seq_id) const {
  auto it = idx_.find(seq_id);
  return it == idx_.end() ? nullptr : &tables_[it->second];
}
std::vector<uint32_t> BlockTable::seq_ids() const {
  std::vector<uint32_t> r;
  for (const auto &t : tables_) r.push_back(t.seq_id);
  return r;
}
std::vector<uint32_t> BlockTable::build_block_tables_array(size_t mb) const {
  std::vector<uint32_t> r(tables_.size() * mb, 0u);
  for (size_t s = 0; s < tables_.size(); s++) {
    const auto &blocks = tables_[s].blocks();
    for (size_t b = 0; b < blocks.size() && b < mb; b++) r[s * mb + b] = blocks[b]->block_id;
  }
  return r;
}
std::vector<uint32_t> BlockTable::build_context_lens_array() const {
  std::vector<uint32_t> r;
  for (const auto &t : tables_) r.push_back(t.num_tokens());
  return r;
}

// ---- config (crates/mlx-paged-attn/src/config.rs:36-123) ------------------------------------
std::string PagedAttentionConfig::validate() const {
  if (block_size != 8 && block_size != 16 && block_size != 32)
    return "Invalid block_size: " + std::to_string(block_size) + ". Must be 8, 16, or 32.";
  static const uint32_t heads[] = {32, 64, 80, 96, 112, 120, 128, 192, 256};
  bool ok = false;
  for (uint32_t h : heads) ok |= h == head_size;
  if (!ok)
    return "Invalid head_size: " + std::to_string(head_size) +
           ". Must be one of [32, 64, 80, 96, 112, 120, 128, 192, 256].";
  if (gpu_memory_mb < 256)
    return "gpu_memory_mb too small: " + std::to_string(gpu_memory_mb) + ". Minimum is 256 MB.";
  if (num_layers == 0) return "num_layers must be > 0";
  if (num_kv_heads == 0) return "num_kv_heads must be > 0";
  if (use_fp8_cache && block_size == 8)
    return "FP8 cache requires block_size 16 or 32 for optimal alignment.";
  return "";
}
uint32_t PagedAttentionConfig::calculate_num_blocks() const {
  const uint64_t elem = use_fp8_cache ? 1 : 2;
  const uint64_t per_block = 2ull * num_kv_heads * head_size * block_size * elem * num_layers;
  return (uint32_t)((uint64_t)gpu_memory_mb * 1024 * 1024 / per_block);
}

// ---- token tracker (crates/mlx-paged-attn/src/token_tracker.rs) -----------------------------
uint64_t compute_token_hash(const uint32_t *tokens, size_t n) {
  uint64_t state = 0xcbf29ce484222325ull;
  for (size_t t = 0; t < n; t++)
    for (int i = 0; i < 4; i++) {
      state ^= (uint8_t)(tokens[t] >> (8 * i));
      state *= 0x100000001b3ull;
    }
  return state;
}

uint64_t TokenTracker::track_tokens(uint32_t block_id, const uint32_t *tokens, size_t n,
                                    uint32_t start_offset) {
  if (!enabled_) return 0;
  bool had_old = false;
  uint64_t old_hash = 0;
  auto it = block_tokens_.find(block_id);
  if (it != block_tokens_.end() && !it->second.empty()) {
    had_old = true;
    old_hash = compute_token_hash(it->second.data(), it->second.size());
  }
  auto &vec = block_tokens_[block_id];
  if (vec.size() < start_offset) vec.resize(start_offset, 0);
  for (size_t i = 0; i < n; i++) {
    const size_t pos = start_offset + i;
    if (pos < vec.size()) vec[pos] = tokens[i];
    else vec.push_back(tokens[i]);
  }
  const uint64_t hash = compute_token_hash(vec.data(), vec.size());
  const uint32_t count = (uint32_t)vec.size();
  if (had_old && old_hash != hash) {
    auto pi = prefix_index_.find(old_hash);
    if (pi != prefix_index_.end() && pi->second.first == block_id) prefix_index_.erase(pi);
  }
  prefix_index_[hash] = {block_id, count};
  return hash;
}

const std::vector<uint32_t> &TokenTracker::get_block_tokens(uint32_t block_id) const {
  static const std::vector<uint32_t> empty;
  auto it = block_tokens_.find(block_id);
  return it == block_tokens_.end() ? empty : it->second;
}

void TokenTracker::remove_block(uint32_t block_id) {
  if (!enabled_) return;
  auto it = block_tokens_.find(block_id);
  if (it != block_tokens_.end()) {
    const uint64_t hash = compute_token_hash(it->second.data(), it->second.size());
    auto pi = prefix_index_.find(hash);
    if (pi != prefix_index_.end() && pi->second.first == block_id) prefix_index_.erase(pi);
    block_tokens_.erase(it);
  }
}

void TokenTracker::copy_block(uint32_t src, uint32_t dst) {
  if (!enabled_) return;
  auto si = block_tokens_.find(src);
  if (si == block_tokens_.end()) return;  // destination untouched
  std::vector<uint32_t> tokens = si->second;
  auto di = block_tokens_.find(dst);
  if (di != block_tokens_.end() && !di->second.empty()) {
    const uint64_t old = compute_token_hash(di->second.data(), di->second.size());
    auto pi = prefix_index_.find(old);
    if (pi != prefix_index_.end() && pi->second.first == dst) prefix_index_.erase(pi);
  }
  const uint64_t hash = compute_token_hash(tokens.data(), tokens.size());
  const uint32_t count = (uint32_t)tokens.size();
  block_tokens_[dst] = std::move(tokens);
  prefix_index_[hash] = {dst, count};
}

std::vector<std::pair<uint32_t, uint32_t>> TokenTracker::find_prefix_matches(const uint32_t *tokens,
                                                                             size_t n) const {
  std::vector<std::pair<uint32_t, uint32_t>> matches;
  if (!enabled_ || n == 0) return matches;
  const size_t full = n / block_size_;
  for (size_t b = 0; b <= full; b++) {
    const size_t start = b * block_size_;
    if (start >= n) break;
    const size_t end = std::min(start + block_size_, n);
    const uint64_t hash = compute_token_hash(tokens + start, end - start);
    auto pi = prefix_index_.find(hash);
    if (pi == prefix_index_.end()) continue;
    auto bt = block_tokens_.find(pi->second.first);
    if (bt != block_tokens_.end() && bt->second.size() >= end - start &&
        std::equal(tokens + start, tokens + end, bt->second.begin()))
      matches.push_back(pi->second);
  }
  return matches;
}

std::pair<std::vector<uint32_t>, uint32_t> TokenTracker::find_longest_prefix(const uint32_t *tokens,
                                                                             size_t n) const {
  std::vector<uint32_t> blocks;
  uint32_t total = 0;
  if (!enabled_ || n == 0) return {blocks, 0};
  size_t pos = 0;
  while (pos < n) {
    const size_t len = std::min<size_t>(block_size_, n - pos);
    const uint64_t hash = compute_token_hash(tokens + pos, len);
    auto pi = prefix_index_.find(hash);
    if (pi == prefix_index_.end()) break;
    auto bt = block_tokens_.find(pi->second.first);
    if (bt == block_tokens_.end() || bt->second.size() < len ||
        !std::equal(tokens + pos, tokens + pos + len, bt->second.begin()))
      break;
    blocks.push_back(pi->second.first);
    total += pi->second.second;
    pos += pi->second.second;
  }
  return {blocks, total};
}

TokenTrackerStats TokenTracker::stats() const {
  size_t total = 0;
  for (const auto &kv : block_tokens_) total += kv.second.size();
  const uint32_t nb = (uint32_t)block_tokens_.size();
  return {nb, (uint32_t)total, nb ? (float)total / (float)nb : 0.f, (uint32_t)prefix_index_.size()};
}
void TokenTracker::clear() {
  block_tokens_.clear();
  prefix_index_.clear();
}
size_t TokenTracker::memory_usage() const {
  size_t bytes = 0;
  for (const auto &kv : block_tokens_) bytes += kv.second.capacity() * sizeof(uint32_t);
  return bytes + prefix_index_.bucket_count() * (sizeof(uint64_t) + 2 * sizeof(uint32_t));
}

// ---- PagedKVCache host methods (crates/mlx-paged-attn/src/paged_kv_cache.rs) ----------------
std::unique_ptr<PagedKVCache> PagedKVCache::create(const PagedAttentionConfig &cfg, std::string *error) {
  const std::string msg = cfg.validate();
  if (!msg.empty()) {
    if (error) *error = msg;
    return nullptr;
  }
  return std::unique_ptr<PagedKVCache>(new PagedKVCache(cfg, cfg.calculate_num_blocks()));
}

bool PagedKVCache::add_sequence(uint32_t prompt_len, uint32_t *seq_id, std::string *error) {
  const uint32_t need = (prompt_len + cfg_.block_size - 1) / cfg_.block_size;
  if (!alloc_.can_allocate(need)) {
    *error = "Not enough memory to allocate " + std::to_string(need) + " blocks for " +
             std::to_string(prompt_len) + " tokens";
    return false;
  }
  const uint32_t id = table_.add_sequence();
  SequenceBlockTable *t = table_.get(id);
  for (uint32_t i = 0; i < need; i++) t->add_block(alloc_.allocate());
  t->set_num_tokens(prompt_len);
  *seq_id = id;
  return true;
}

bool PagedKVCache::remove_sequence(uint32_t seq_id, std::string *error) {
  SequenceBlockTable t(0, cfg_.block_size);
  if (!table_.remove_sequence(seq_id, &t)) {
    *error = "Sequence " + std::to_string(seq_id) + " not found";
    return false;
  }
  for (const auto &b : t.blocks()) {
    if (b->ref_count == 1) tracker_.remove_block(b->block_id);  // last user: drop its tokens
    alloc_.free(b);
  }
  return true;
}

bool PagedKVCache::extend_sequence(uint32_t seq_id, uint32_t n, std::string *error) {
  SequenceBlockTable *t = table_.get(seq_id);
  if (!t) {
    *error = "Sequence " + std::to_string(seq_id) + " not found";
    return false;
  }
  const uint32_t need = t->blocks_needed(n);
  for (uint32_t i = 0; i < need; i++) {
    BlockRef b = alloc_.allocate();
    if (!b) {
      *error = "Block allocation failed";
      return false;
    }
    t->add_block(b);
  }
  t->set_num_tokens(t->num_tokens() + n);
  return true;
}

bool PagedKVCache::fork_sequence(uint32_t parent, uint32_t *child, std::string *error) {
  const SequenceBlockTable *p = table_.get(parent);
  if (!p) {
    *error = "Parent sequence " + std::to_string(parent) + " not found";
    return false;
  }
  const std::vector<BlockRef> blocks = p->blocks();
  const uint32_t tokens = p->num_tokens();
  const uint32_t id = table_.add_sequence();
  SequenceBlockTable *c = table_.get(id);
  for (const auto &b : blocks) {
    b->incref();
    c->add_block(b);
  }
  c->set_num_tokens(tokens);
  *child = id;
  return true;
}

bool PagedKVCache::handle_cow(uint32_t seq_id, size_t block_idx, bool *copied, uint32_t *src, uint32_t *dst,
                              std::string *error) {
  SequenceBlockTable *t = table_.get(seq_id);
  if (!t) {
    *error = "Sequence " + std::to_string(seq_id) + " not found";
    return false;
  }
  if (block_idx >= t->blocks().size()) {
    *error = "Block index " + std::to_string(block_idx) + " out of range";
    return false;
  }
  const BlockRef block = t->blocks()[block_idx];
  *copied = false;
  if (!block->is_shared()) return true;
  BlockRef fresh = alloc_.copy_on_write(block);
  if (!fresh) {
    *error = "Failed to allocate block for copy-on-write";
    return false;
  }
  *src = block->block_id;
  *dst = fresh->block_id;
  *copied = true;
  t->replace_block(block_idx, fresh);
  return true;
}

bool PagedKVCache::build_block_tables_batch(const uint32_t *seq_ids, size_t n,
                                            std::vector<std::vector<uint32_t>> *out, std::string *error) const {
  out->clear();
  for (size_t i = 0; i < n; i++) {
    const SequenceBlockTable *t = table_.get(seq_ids[i]);
    if (!t) {
      *error = "Sequence " + std::to_string(seq_ids[i]) + " not found";
      return false;
    }
    std::vector<uint32_t> ids;
    for (const auto &b : t->blocks()) ids.push_back(b->block_id);
    out->push_back(std::move(ids));
  }
  return true;
}

bool PagedKVCache::get_slot_mapping(uint32_t seq_id, uint32_t start, uint32_t n, std::vector<int64_t> *out,
                                    std::string *error) const {
  const SequenceBlockTable *t = table_.get(seq_id);
  if (!t) {
    *error = "Sequence " + std::to_string(seq_id) + " not found";
    return false;
  }
  for (uint32_t i = 0; i < n; i++) {
    int64_t slot;
    if (!t->absolute_slot_index(start + i, &slot)) {
      *error = "Token position " + std::to_string(start + i) + " out of range for sequence " +
               std::to_string(seq_id);
      return false;
    }
    out->push_back(slot);
  }
  return true;
}

bool PagedKVCache::get_slot_mapping_batch(const uint32_t *seq_ids, const uint32_t *context_lens,
                                          const uint8_t *is_prefill, const uint32_t *input_lens, size_t n,
                                          std::vector<int64_t> *out, std::string *error) const {
  for (size_t i = 0; i < n; i++) {
    if (is_prefill && is_prefill[i]) {
      if (!get_slot_mapping(seq_ids[i], 0, input_lens ? input_lens[i] : 1, out, error)) return false;
    } else {
      // decode: the token being processed sits at position context_len - 1
      const uint32_t ctx = context_lens ? context_lens[i] : 0;
      if (ctx == 0) {
        *error = "Decode sequence " + std::to_string(seq_ids[i]) +
                 " has context_len=0. This indicates prefill was not completed. "
                 "Prefill must run before decode.";
        return false;
      }
      if (!get_slot_mapping(seq_ids[i], ctx - 1, 1, out, error)) return false;
    }
  }
  return true;
}

bool PagedKVCache::build_input_metadata(const uint32_t *seq_ids, const uint32_t *input_lens,
                                        const uint8_t *is_prefill, size_t n, InputMetadata *out,
                                        std::string *error) const {
  InputMetadata m;
  std::vector<uint32_t> ctx(n);
  for (size_t i = 0; i < n; i++) {
    const SequenceBlockTable *t = table_.get(seq_ids[i]);
    ctx[i] = t ? t->num_tokens() : 0;
    m.context_lens.push_back((int32_t)ctx[i]);
    m.max_context_len = std::max(m.max_context_len, ctx[i]);
  }
  if (!get_slot_mapping_batch(seq_ids, ctx.data(), is_prefill, input_lens, n, &m.slot_mappings, error))
    return false;
  std::vector<std::vector<uint32_t>> tables;
  if (!build_block_tables_batch(seq_ids, n, &tables, error)) return false;
  const size_t mb = max_blocks_per_seq();
  for (const auto &t : tables) {
    if (t.size() > mb) {
      *error = "sequence holds more blocks than max_seq_len allows";
      return false;
    }
    for (uint32_t id : t) m.block_tables.push_back((int32_t)id);
    m.block_tables.insert(m.block_tables.end(), mb - t.size(), 0);
  }
  m.is_prefill = true;
  for (size_t i = 0; i < n; i++) m.is_prefill = m.is_prefill && is_prefill && is_prefill[i];
  m.num_seqs = (uint32_t)n;
  m.max_blocks_per_seq = (uint32_t)mb;
  *out = std::move(m);
  return true;
}

MemoryStats PagedKVCache::get_memory_stats() const {
  const uint64_t per_block = 2ull * cfg_.num_kv_heads * cfg_.head_size * cfg_.block_size * cfg_.num_layers *
                             (cfg_.use_fp8_cache ? 1 : 2);
  const uint32_t total = alloc_.total_blocks(), used = alloc_.num_allocated_blocks();
  return {total,
          alloc_.num_free_blocks(),
          used,
          (uint32_t)((uint64_t)total * per_block / 1024 / 1024),
          (uint32_t)((uint64_t)used * per_block / 1024 / 1024),
          total ? (double)used / (double)total * 100.0 : 0.0};
}

bool PagedKVCache::track_sequence_tokens(uint32_t seq_id, const uint32_t *tokens, size_t n, uint32_t start_pos,
                                         std::string *error) {
  const SequenceBlockTable *t = table_.get(seq_id);
  if (!t) {
    *error = "Sequence " + std::to_string(seq_id) + " not found";
    return false;
  }
  for (size_t i = 0; i < n; i++) {
    const uint32_t pos = start_pos + (uint32_t)i;
    const size_t blk = pos / cfg_.block_size;
    if (blk < t->blocks().size())
      tracker_.track_tokens(t->blocks()[blk]->block_id, &tokens[i], 1, pos % cfg_.block_size);
  }
  return true;
}

bool PagedKVCache::get_sequence_tokens(uint32_t seq_id, std::vector<uint32_t> *out, std::string *error) const {
  const SequenceBlockTable *t = table_.get(seq_id);
  if (!t) {
    *error = "Sequence " + std::to_string(seq_id) + " not found";
    return false;
  }
  out->clear();
  for (const auto &b : t->blocks()) {
    const auto &v = tracker_.get_block_tokens(b->block_id);
    out->insert(out->end(), v.begin(), v.end());
  }
  if (out->size() > t->num_tokens()) out->resize(t->num_tokens());
  return true;
}

// ---- scheduler (crates/mlx-paged-attn/src/scheduler.rs:143-466) -----------------------------
void ContinuousBatchingScheduler::add_request(PendingRequest r) {
  auto pos = waiting_.begin();
  while (pos != waiting_.end() && pos->priority >= r.priority) ++pos;
  waiting_.insert(pos, std::move(r));
}

bool ContinuousBatchingScheduler::schedule_step(PagedKVCache &cache, ScheduledBatch *out) {
  if (running_.empty() && waiting_.empty()) return false;
  ScheduledBatch b;
  size_t total = 0;
  auto add_decodes = [&](bool skip_present) {
    for (const auto &kv : running_) {
      if (b.seq_ids.size() >= cfg_.max_batch_size) break;
      const ActiveSequence &s = kv.second;
      if (s.is_prefill || total >= cfg_.max_tokens_per_step) continue;
      if (skip_present && std::find(b.seq_ids.begin(), b.seq_ids.end(), kv.first) != b.seq_ids.end()) continue;
      b.seq_ids.push_back(kv.first);
      b.request_ids.push_back(s.request_id);
      b.input_tokens.push_back({s.generated_tokens.empty() ? 0u : s.generated_tokens.back()});
      b.is_prefill.push_back(0);
      b.context_lens.push_back(s.position);
      total += 1;
      b.num_decode++;
    }
  };
  if (cfg_.prioritize_decode) add_decodes(false);
  // admit waiting requests: prefill = the whole prompt in one step
  while (b.seq_ids.size() < cfg_.max_batch_size && b.num_prefill < cfg_.max_prefill_per_step &&
         !waiting_.empty()) {
    const PendingRequest &front = waiting_.front();
    const uint32_t prompt_len = (uint32_t)front.prompt_tokens.size();
    const uint32_t need = (prompt_len + block_size_ - 1) / block_size_;
    if (total + prompt_len > cfg_.max_tokens_per_step) break;
    if (!cache.can_allocate(need)) break;  // back-pressure: leave it queued
    PendingRequest req = std::move(waiting_.front());
    waiting_.pop_front();
    uint32_t seq_id;
    std::string err;
    if (!cache.add_sequence(prompt_len, &seq_id, &err)) {
      waiting_.push_front(std::move(req));
      break;
    }
    running_[seq_id] = ActiveSequence{seq_id, req.request_id, {}, req.max_new_tokens, prompt_len, true, prompt_len};
    b.seq_ids.push_back(seq_id);
    b.request_ids.push_back(req.request_id);
    b.input_tokens.push_back(std::move(req.prompt_tokens));
    b.is_prefill.push_back(1);
    b.context_lens.push_back(prompt_len);
    total += prompt_len;
    b.num_prefill++;
  }
  if (!cfg_.prioritize_decode) add_decodes(true);
  if (b.seq_ids.empty()) return false;
  b.total_tokens = (uint32_t)total;
  *out = std::move(b);
  return true;
}

bool ContinuousBatchingScheduler::process_outputs(const std::vector<TokenOutput> &outputs, PagedKVCache &cache,
                                                  std::string *error) {
  for (const TokenOutput &o : outputs) {
    auto it = running_.find(o.seq_id);
    if (it == running_.end()) continue;
    ActiveSequence &s = it->second;
    s.is_prefill = false;
    s.generated_tokens.push_back(o.token);
    s.position += 1;
    if (!cache.extend_sequence(o.seq_id, 1, error)) return false;
    const bool eos = o.is_eos || o.token == cfg_.eos_token_id;
    if (eos || s.generated_tokens.size() >= s.max_new_tokens) {
      const uint32_t gen = (uint32_t)s.generated_tokens.size();
      completed_.push_back(
          CompletedSequence{s.request_id, std::move(s.generated_tokens), eos ? "stop" : "length", s.prompt_len + gen});
      running_.erase(it);
      if (!cache.remove_sequence(o.seq_id, error)) return false;
    }
  }
  return true;
}

std::vector<CompletedSequence> ContinuousBatchingScheduler::get_completed() {
  std::vector<CompletedSequence> r;
  r.swap(completed_);
  return r;
}

bool ContinuousBatchingScheduler::abort_request(const std::string &request_id, PagedKVCache &cache, bool *found,
                                                std::string *error) {
  *found = false;
  for (auto it = waiting_.begin(); it != waiting_.end(); ++it)
    if (it->request_id == request_id) {
      waiting_.erase(it);
      *found = true;
      return true;
    }
  for (auto it = running_.begin(); it != running_.end(); ++it)
    if (it->second.request_id == request_id) {
      const uint32_t seq_id = it->first;
      running_.erase(it);
      *found = true;
      return cache.remove_sequence(seq_id, error);
    }
  return true;
}

SchedulerStats ContinuousBatchingScheduler::get_stats() const {
  uint32_t tokens = 0, prefill = 0;
  for (const auto &kv : running_) {
    tokens += kv.second.position;
    prefill += kv.second.is_prefill ? 1 : 0;
  }
  return {(uint32_t)waiting_.size(), (uint32_t)running_.size(), (uint32_t)completed_.size(), prefill,
          (uint32_t)running_.size() - prefill, tokens};
}

const ActiveSequence *ContinuousBatchingScheduler::running(uint32_t seq_id) const {
  auto it = running_.find(seq_id);
  return it == running_.end() ? nullptr : &it->second;
}

bool PagedKVCache::truncate_sequence(uint32_t seq_id, uint32_t new_num_tokens, std::string *error) {
  SequenceBlockTable *t = table_.get(seq_id);
  if (!t) {
    *error = "Sequence " + std::to_string(seq_id) + " not found";
    return false;
  }
  if (new_num_tokens > t->num_tokens()) {
    *error = "truncate_sequence cannot grow a sequence";
    return false;
  }
  const size_t keep = (new_num_tokens + cfg_.block_size - 1) / cfg_.block_size;
  // rebuild the table with the kept blocks; release the rest
  std::vector<BlockRef> blocks = t->blocks();
  SequenceBlockTable fresh(seq_id, cfg_.block_size);
  for (size_t i = 0; i < blocks.size(); i++) {
    if (i < keep) {
      fresh.add_block(blocks[i]);
    } else {
      if (blocks[i]->ref_count == 1) tracker_.remove_block(blocks[i]->block_id);
      alloc_.free(blocks[i]);
    }
  }
  fresh.set_num_tokens(new_num_tokens);
  *t = fresh;
  return true;
}

// ---- hybrid scheduler ------------------------------------------------------------------------------
void HybridScheduler::add_request(PendingRequest r) {
  auto pos = waiting_.begin();
  while (pos != waiting_.end() && pos->priority >= r.priority) ++pos;
  waiting_.insert(pos, std::move(r));
}

bool HybridScheduler::set_draft_tokens(uint32_t seq_id, const uint32_t *tokens, size_t n) {
  auto it = running_.find(seq_id);
  if (it == running_.end() || it->second.num_computed < it->second.prompt.size()) return false;
  it->second.drafts.assign(tokens, tokens + n);
  return true;
}

bool HybridScheduler::schedule_step(PagedKVCache &cache, HybridBatch *out, std::string *error) {
  HybridBatch b;
  size_t budget = cfg_.max_tokens_per_step;
  auto add_decodes = [&]() -> bool {
    for (auto &kv : running_) {
      Seq &s = kv.second;
      if (s.num_computed < s.prompt.size()) continue;  // still in prefill
      if (b.entries.size() >= cfg_.max_batch_size) break;
      uint32_t k = (uint32_t)s.drafts.size();
      if (1 + k > budget) k = budget >= 1 ? (uint32_t)budget - 1 : 0;  // verify fewer drafts
      if (budget < 1) break;
      const uint32_t total = (uint32_t)(s.prompt.size() + s.generated.size());
      if (k && !cache.extend_sequence(s.seq_id, k, error)) {
        // pool exhausted: fall back to a plain decode step for this sequence
        error->clear();
        k = 0;
      }
      HybridEntry e;
      e.seq_id = s.seq_id;
      e.request_id = s.request_id;
      e.kind = k ? kVerify : kDecode;
      e.q_len = 1 + k;
      e.kv_len = total + k;
      e.needs_sample = true;
      e.tokens.push_back(s.generated.back());
      e.tokens.insert(e.tokens.end(), s.drafts.begin(), s.drafts.begin() + k);
      s.drafts.resize(k);
      budget -= e.q_len;
      (k ? b.num_verify : b.num_decode)++;
      b.entries.push_back(std::move(e));
    }
    return true;
  };
  auto add_prefills = [&]() {
    // sequences already admitted and still in prefill, then new admissions
    uint32_t in_prefill = 0;
    auto chunk_for = [&](Seq &s) {
      const uint32_t remaining = (uint32_t)s.prompt.size() - s.num_computed;
      uint32_t chunk = cfg_.prefill_chunk_size ? std::min(remaining, cfg_.prefill_chunk_size) : remaining;
      chunk = (uint32_t)std::min<size_t>(chunk, budget);
      if (chunk == 0) return;
      HybridEntry e;
      e.seq_id = s.seq_id;
      e.request_id = s.request_id;
      e.kind = kPrefillChunk;
      e.q_len = chunk;
      e.kv_len = s.num_computed + chunk;
      e.needs_sample = e.kv_len == s.prompt.size();
      e.tokens.assign(s.prompt.begin() + s.num_computed, s.prompt.begin() + s.num_computed + chunk);
      budget -= chunk;
      b.num_prefill++;
      b.entries.push_back(std::move(e));
    };
    for (auto &kv : running_) {
      Seq &s = kv.second;
      if (s.num_computed >= s.prompt.size()) continue;
      if (b.entries.size() >= cfg_.max_batch_size || in_prefill >= cfg_.max_prefill_per_step || !budget) break;
      chunk_for(s);
      in_prefill++;
    }
    while (b.entries.size() < cfg_.max_batch_size && in_prefill < cfg_.max_prefill_per_step && budget &&
           !waiting_.empty()) {
      const PendingRequest &front = waiting_.front();
      const uint32_t prompt_len = (uint32_t)front.prompt_tokens.size();
      if (prompt_len == 0) {  // nothing to attend to: reject instead of looping
        waiting_.pop_front();
        continue;
      }
      if (!cache.can_allocate((prompt_len + block_size_ - 1) / block_size_)) break;
      PendingRequest req = std::move(waiting_.front());
      waiting_.pop_front();
      uint32_t seq_id;
      std::string err;
      if (!cache.add_sequence(prompt_len, &seq_id, &err)) {
        waiting_.push_front(std::move(req));
        break;
      }
      Seq s;
      s.seq_id = seq_id;
      s.request_id = req.request_id;
      s.prompt = std::move(req.prompt_tokens);
      s.max_new_tokens = req.max_new_tokens;
      auto ins = running_.emplace(seq_id, std::move(s));
      chunk_for(ins.first->second);
      in_prefill++;
    }
  };
  if (cfg_.prioritize_decode) {
    add_decodes();
    add_prefills();
  } else {
    add_prefills();
    add_decodes();
  }
  if (b.entries.empty()) return false;
  b.total_tokens = 0;
  for (const auto &e : b.entries) b.total_tokens += e.q_len;
  *out = std::move(b);
  return true;
}

bool HybridScheduler::build_metadata(const PagedKVCache &cache, const HybridBatch &batch, InputMetadata *meta,
                                     std::vector<int32_t> *cu_q_lens, std::string *error) const {
  InputMetadata m;
  cu_q_lens->assign(1, 0);
  const size_t mb = cache.max_blocks_per_seq();
  bool all_prefill = true;
  for (const HybridEntry &e : batch.entries) {
    m.context_lens.push_back((int32_t)e.kv_len);
    m.max_context_len = std::max(m.max_context_len, e.kv_len);
    cu_q_lens->push_back(cu_q_lens->back() + (int32_t)e.q_len);
    if (!cache.get_slot_mapping(e.seq_id, e.kv_len - e.q_len, e.q_len, &m.slot_mappings, error)) return false;
    std::vector<std::vector<uint32_t>> t;
    if (!cache.build_block_tables_batch(&e.seq_id, 1, &t, error)) return false;
    if (t[0].size() > mb) {
      *error = "sequence holds more blocks than max_seq_len allows";
      return false;
    }
    for (uint32_t id : t[0]) m.block_tables.push_back((int32_t)id);
    m.block_tables.insert(m.block_tables.end(), mb - t[0].size(), 0);
    all_prefill = all_prefill && e.kind == kPrefillChunk;
  }
  m.is_prefill = all_prefill;
  m.num_seqs = (uint32_t)batch.entries.size();
  m.max_blocks_per_seq = (uint32_t)mb;
  *meta = std::move(m);
  return true;
}

bool HybridScheduler::process_outputs(const HybridBatch &batch, const std::vector<HybridOutput> &outputs,
                                      PagedKVCache &cache, std::string *error) {
  std::map<uint32_t, const HybridOutput *> by_seq;
  for (const HybridOutput &o : outputs) by_seq[o.seq_id] = &o;
  for (const HybridEntry &e : batch.entries) {
    auto it = running_.find(e.seq_id);
    if (it == running_.end()) continue;
    Seq &s = it->second;
    if (e.kind == kPrefillChunk) s.num_computed = e.kv_len;
    if (!e.needs_sample) continue;
    auto oi = by_seq.find(e.seq_id);
    if (oi == by_seq.end()) {
      *error = "no output for sequence " + std::to_string(e.seq_id);
      return false;
    }
    const HybridOutput &o = *oi->second;
    const uint32_t k = e.kind == kVerify ? e.q_len - 1 : 0;
    const uint32_t a = std::min(o.num_accepted, k);
    std::vector<uint32_t> fresh(s.drafts.begin(), s.drafts.begin() + a);
    fresh.push_back(o.next_token);
    s.drafts.clear();
    bool stop = false, eos = false;
    for (size_t i = 0; i < fresh.size(); i++) {
      const uint32_t tok = fresh[i];
      s.generated.push_back(tok);
      const bool last = i + 1 == fresh.size();
      if (tok == cfg_.eos_token_id || (last && o.is_eos)) { stop = eos = true; break; }
      if (s.generated.size() >= s.max_new_tokens) { stop = true; break; }
    }
    // the pool must hold one slot per token of the sequence (the newest token's K/V is
    // written by the next step): prompt + generated
    const uint32_t want = (uint32_t)(s.prompt.size() + s.generated.size());
    const uint32_t have = cache.sequence_num_tokens(e.seq_id);
    if (want > have) {
      if (!stop && !cache.extend_sequence(e.seq_id, want - have, error)) return false;
    } else if (want < have) {
      if (!cache.truncate_sequence(e.seq_id, want, error)) return false;
    }
    if (stop) {
      const uint32_t gen = (uint32_t)s.generated.size();
      completed_.push_back(CompletedSequence{s.request_id, std::move(s.generated), eos ? "stop" : "length",
                                             (uint32_t)s.prompt.size() + gen});
      running_.erase(it);
      if (!cache.remove_sequence(e.seq_id, error)) return false;
    }
  }
  return true;
}

std::vector<CompletedSequence> HybridScheduler::get_completed() {
  std::vector<CompletedSequence> r;
  r.swap(completed_);
  return r;
}

// ---- kv_scale.rs:165-174 -------------------------------------------------------------------------
float kv_compute_scale(float max_abs) { return max_abs < 1e-12f ? 1.0f : 448.0f / max_abs; }

// ---- kv_scale.rs:36-300 ----------------------------------------------------------------------------
KvScaleManager::KvScaleManager(uint32_t num_layers, float alpha)
    : num_layers_(num_layers), alpha_(alpha < 0.f ? 0.f : (alpha > 1.f ? 1.f : alpha)) {}

void KvScaleManager::init_default_scales() {
  for (uint32_t i = 0; i < num_layers_; i++) k_scales_[i] = v_scales_[i] = 1.0f;
}
float KvScaleManager::k_scale(uint32_t layer) const {
  auto it = k_scales_.find(layer);
  return it == k_scales_.end() ? 1.0f : it->second;
}
float KvScaleManager::v_scale(uint32_t layer) const {
  auto it = v_scales_.find(layer);
  return it == v_scales_.end() ? 1.0f : it->second;
}
std::pair<float, float> KvScaleManager::calibrate_layer(uint32_t layer, float k_max, float v_max) {
  const float k = kv_compute_scale(k_max), v = kv_compute_scale(v_max);
  k_scales_[layer] = k;
  v_scales_[layer] = v;
  calibrated_ = true;
  return {k, v};
}
std::pair<float, float> KvScaleManager::update_layer_ema(uint32_t layer, float k_max, float v_max) {
  // entry(layer).or_insert(observed), then the update runs on that value as well
  // (kv_scale.rs:167-171)
  auto kr = k_running_max_.emplace(layer, k_max).first;
  kr->second = alpha_ * k_max + (1.0f - alpha_) * kr->second;
  auto vr = v_running_max_.emplace(layer, v_max).first;
  vr->second = alpha_ * v_max + (1.0f - alpha_) * vr->second;
  const float k = kv_compute_scale(kr->second), v = kv_compute_scale(vr->second);
  k_scales_[layer] = k;
  v_scales_[layer] = v;
  calibrated_ = true;
  return {k, v};
}
void KvScaleManager::set_scales(uint32_t layer, float k, float v) {
  k_scales_[layer] = k;
  v_scales_[layer] = v;
  calibrated_ = true;
}
void KvScaleManager::get_all_scales(std::vector<float> *k, std::vector<float> *v) const {
  k->assign(num_layers_, 1.0f);
  v->assign(num_layers_, 1.0f);
  for (const auto &e : k_scales_) if (e.first < num_layers_) (*k)[e.first] = e.second;
  for (const auto &e : v_scales_) if (e.first < num_layers_) (*v)[e.first] = e.second;
}
void KvScaleManager::load_scales(const float *k, size_t nk, const float *v, size_t nv) {
  for (size_t i = 0; i < nk; i++) k_scales_[(uint32_t)i] = k[i];
  for (size_t i = 0; i < nv; i++) v_scales_[(uint32_t)i] = v[i];
  calibrated_ = true;
}
void KvScaleManager::reset() {
  k_scales_.clear();
  v_scales_.clear();
  k_running_max_.clear();
  v_running_max_.clear();
  calibrated_ = false;
}
KvScaleStats KvScaleManager::stats() const {
  KvScaleStats s{};
  s.num_layers_calibrated = (uint32_t)k_scales_.size();
  auto fold = [](const std::map<uint32_t, float> &m, float *mn, float *mx, float *mean) {
    *mn = INFINITY;
    *mx = -INFINITY;
    float sum = 0.f;
    for (const auto &e : m) {
      *mn = std::min(*mn, e.second);
      *mx = std::max(*mx, e.second);
      sum += e.second;
    }
    *mean = m.empty() ? 0.f : sum / (float)m.size();
  };
  fold(k_scales_, &s.k_scale_min, &s.k_scale_max, &s.k_scale_mean);
  fold(v_scales_, &s.v_scale_min, &s.v_scale_max, &s.v_scale_mean);
  return s;
}

// ---- attention_layer.rs:116-161 ----------------------------------------------------------------------
AttentionLayer::AttentionLayer(const AttentionLayerParams &p)
    : layer_idx(p.layer_idx), num_heads(p.num_heads), num_kv_heads(p.num_kv_heads), head_size(p.head_size),
      block_size(p.block_size), scale(p.scale > 0.f ? p.scale : 1.0f / std::sqrt((float)p.head_size)),
      softcap(p.softcap > 0.f ? p.softcap : 1.0f), k_scale(p.k_scale > 0.f ? p.k_scale : 1.0f),
      v_scale(p.v_scale > 0.f ? p.v_scale : 1.0f), use_fp8(p.use_fp8) {}

AttentionLayer AttentionLayer::from_cache_config(uint32_t layer_idx, uint32_t num_heads,
                                                 const PagedAttentionConfig &cfg) {
  AttentionLayerParams p;
  p.layer_idx = layer_idx;
  p.num_heads = num_heads;
  p.num_kv_heads = cfg.num_kv_heads;
  p.head_size = cfg.head_size;
  p.block_size = cfg.block_size;
  p.use_fp8 = cfg.use_fp8_cache;
  return AttentionLayer(p);
}

}  // namespace pa_host
