// The host cache bound to a device cache (include/paged_attn_b200_host.h, last
// section): the reference's device-touching PagedKVCache methods
// (crates/mlx-paged-attn/src/paged_kv_cache.rs:753-1347), its PagedAttentionLayer(s)
// (attention_layer.rs:41-478), the kernel-argument metadata object with its lazily made
// device buffers (input_metadata.rs:29-278) and the FP8 scale manager's device
// reductions (metal/kv_scale.rs:108-226).
//
// Resident block tables.  The binding owns a device table [rows, max_blocks_per_seq]
// with one row per live sequence and remembers, per sequence, which entries it has
// sent.  A call stages the batch's row indices, context lengths, decode slots and the
// (row, column, block id) triples that changed since the last call in one pinned,
// device-mapped area; one launch (`ingest_kernel`) reads that area over PCIe, applies
// the triples and, for the host-buffer step, brings q/k/v over in the same launch.
// Attention then runs on the resident table through the kernels' row indirection.
#include <cmath>
#include <cstring>
#include <new>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/paged_attn_b200_host.h"
#include "host_logic.hpp"
#include "pa_common.cuh"

namespace pa {
int32_t set_error(int32_t code, const std::string &msg);
}
using namespace pa_host;

namespace {

pa_status err(const std::string &msg, pa_status code = PA_ERR_INVALID_ARG) { return pa::set_error(code, msg); }
pa_status cuda_err(cudaError_t e, const char *what) {
  return pa::set_error(e == cudaErrorMemoryAllocation ? PA_ERR_OOM : PA_ERR_CUDA,
                       std::string(what) + ": " + cudaGetErrorString(e));
}
#define KV_CUDA(call)                                   \
  do {                                                  \
    cudaError_t e_ = (call);                            \
    if (e_ != cudaSuccess) return cuda_err(e_, #call);  \
  } while (0)
#define KV_TRY(call)                 \
  do {                               \
    pa_status s_ = (call);           \
    if (s_ != PA_OK) return s_;      \
  } while (0)

struct DeviceScope {
  int prev = -1;
  explicit DeviceScope(int dev) {
    if (cudaGetDevice(&prev) != cudaSuccess || prev == dev) prev = -1;
    else cudaSetDevice(dev);
  }
  ~DeviceScope() {
    if (prev >= 0) cudaSetDevice(prev);
  }
};

// One staged call, as the ingest kernel reads it (host-mapped memory).
struct StageHeader {
  uint32_t n;          // sequences of the batch
  uint32_t n_updates;  // (row, col, id) triples
  uint32_t has_slots;  // slots[] valid
  uint32_t pad;
  // bulk copies (host-buffer step): q, k, v; 16-byte units
  const uint4 *src[3];
  uint4 *dst[3];
  uint64_t units[3];
};
struct TableUpdate {
  int32_t row, col, id;
};

// grid: any; CTA 0 applies the metadata, all CTAs share the bulk copies.
__global__ void __launch_bounds__(256)
ingest_kernel(const StageHeader *__restrict__ hdr, const int32_t *__restrict__ rows_in,
              const int32_t *__restrict__ lens_in, const int64_t *__restrict__ slots_in,
              const TableUpdate *__restrict__ upd, int32_t *rows_out, int32_t *lens_out,
              int64_t *slots_out, int32_t *tables, int MB) {
  const StageHeader h = *hdr;
  if (blockIdx.x == 0) {
    for (uint32_t i = threadIdx.x; i < h.n; i += blockDim.x) {
      rows_out[i] = rows_in[i];
      lens_out[i] = lens_in[i];
      if (h.has_slots) slots_out[i] = slots_in[i];
    }
    for (uint32_t i = threadIdx.x; i < h.n_updates; i += blockDim.x) {
      const TableUpdate u = upd[i];
      tables[(size_t)u.row * MB + u.col] = u.id;
    }
  }
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (int c = 0; c < 3; c++)
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < h.units[c]; i += stride)
      h.dst[c][i] = h.src[c][i];
}

// max |x| over 16-bit floats: order-preserving on the magnitude bits once widened to f32
__global__ void __launch_bounds__(256)
max_abs_kernel(const uint16_t *__restrict__ x, size_t n, int is_f16, unsigned *out) {
  float m = 0.f;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    float v;
    if (is_f16) asm("cvt.f32.f16 %0, %1;" : "=f"(v) : "h"(x[i]));
    else v = __uint_as_float((uint32_t)x[i] << 16);
    v = fabsf(v);
    m = v > m ? v : m;  // NaN compares false and is skipped
  }
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0) atomicMax(out, __float_as_uint(m));
}

}  // namespace

struct PaKvBinding {
  PaKvHost *kv = nullptr;
  PagedAttnCache *cache = nullptr;
  PagedAttnConfig cfg{};
  int device = 0;
  bool fp8 = false;
  uint32_t MB = 0;
  // resident tables
  struct Row {
    int32_t row;
    uint64_t version;
    std::vector<int32_t> sent;
  };
  std::unordered_map<uint32_t, Row> rows;
  std::vector<int32_t> free_rows;
  int32_t rows_cap = 0, next_row = 0;
  int32_t *tables_dev = nullptr;
  // per-call device arrays
  int32_t *rows_dev = nullptr, *lens_dev = nullptr;
  int64_t *slots_dev = nullptr;
  size_t batch_cap = 0;
  // pinned staging ring
  static constexpr int kRing = 4;
  char *stage[kRing] = {};
  size_t stage_cap[kRing] = {};
  cudaEvent_t stage_done[kRing] = {};
  int stage_next = 0;
  // workspace, host-step staging, own stream
  void *ws = nullptr;
  size_t ws_bytes = 0;
  char *io = nullptr;
  size_t io_cap = 0;
  cudaStream_t stream = nullptr;
  unsigned *scalar_dev = nullptr;  // two words for the calibration reductions
  PaKvScaleManager *scales = nullptr;
  int num_sms = 0;
  uint64_t entries_sent = 0, calls = 0;
};

namespace {

pa_status grow_dev(void **p, size_t *have, size_t need) {
  if (*have >= need) return PA_OK;
  if (*p) KV_CUDA(cudaFree(*p));
  *p = nullptr;
  *have = 0;
  const size_t sz = (need + 65535) & ~(size_t)65535;
  KV_CUDA(cudaMalloc(p, sz));
  *have = sz;
  return PA_OK;
}

pa_status ensure_batch(PaKvBinding *b, size_t n) {
  if (n <= b->batch_cap) return PA_OK;
  const size_t cap = (n + 255) & ~(size_t)255;
  if (b->rows_dev) cudaFree(b->rows_dev);
  if (b->lens_dev) cudaFree(b->lens_dev);
  if (b->slots_dev) cudaFree(b->slots_dev);
  b->rows_dev = b->lens_dev = nullptr;
  b->slots_dev = nullptr;
  b->batch_cap = 0;
  KV_CUDA(cudaMalloc(&b->rows_dev, cap * 4));
  KV_CUDA(cudaMalloc(&b->lens_dev, cap * 4));
  KV_CUDA(cudaMalloc(&b->slots_dev, cap * 8));
  b->batch_cap = cap;
  return PA_OK;
}

// A table row for `seq_id`: a free one, a fresh one, one reclaimed from a sequence the
// host cache no longer has, or (the table grown) a fresh one.
pa_status row_for(PaKvBinding *b, uint32_t seq_id, PaKvBinding::Row **out, cudaStream_t st) {
  auto it = b->rows.find(seq_id);
  if (it != b->rows.end()) {
    *out = &it->second;
    return PA_OK;
  }
  if (b->free_rows.empty() && b->next_row == b->rows_cap) {
    for (auto r = b->rows.begin(); r != b->rows.end();) {
      if (!b->kv->kv->sequence(r->first)) {
        b->free_rows.push_back(r->second.row);
        r = b->rows.erase(r);
      } else {
        ++r;
      }
    }
  }
  if (b->free_rows.empty() && b->next_row == b->rows_cap) {
    const int32_t cap = b->rows_cap ? b->rows_cap * 2 : 256;
    int32_t *t = nullptr;
    KV_CUDA(cudaMalloc(&t, (size_t)cap * b->MB * 4));
    if (b->tables_dev) {
      KV_CUDA(cudaMemcpyAsync(t, b->tables_dev, (size_t)b->rows_cap * b->MB * 4, cudaMemcpyDeviceToDevice, st));
      KV_CUDA(cudaStreamSynchronize(st));
      KV_CUDA(cudaFree(b->tables_dev));
    }
    b->tables_dev = t;
    b->rows_cap = cap;
  }
  int32_t row;
  if (!b->free_rows.empty()) {
    row = b->free_rows.back();
    b->free_rows.pop_back();
  } else {
    row = b->next_row++;
  }
  PaKvBinding::Row &r = b->rows[seq_id];
  r.row = row;
  r.version = 0;
  r.sent.clear();
  *out = &r;
  return PA_OK;
}

struct Staged {
  StageHeader *hdr;
  int32_t *rows, *lens;
  int64_t *slots;
  TableUpdate *upd;
  size_t upd_cap;
};

// The next staging area of the ring, large enough for n sequences and `max_upd` triples.
pa_status stage_area(PaKvBinding *b, size_t n, size_t max_upd, Staged *s) {
  const int k = b->stage_next;
  b->stage_next = (k + 1) % PaKvBinding::kRing;
  if (b->stage_done[k]) KV_CUDA(cudaEventSynchronize(b->stage_done[k]));
  const size_t need = 256 + ((n * 16 + 255) & ~(size_t)255) + max_upd * sizeof(TableUpdate);
  if (need > b->stage_cap[k]) {
    if (b->stage[k]) cudaFreeHost(b->stage[k]);
    b->stage[k] = nullptr;
    b->stage_cap[k] = 0;
    const size_t sz = (2 * need + 4095) & ~(size_t)4095;
    KV_CUDA(cudaHostAlloc(reinterpret_cast<void **>(&b->stage[k]), sz, cudaHostAllocMapped | cudaHostAllocPortable));
    b->stage_cap[k] = sz;
  }
  if (!b->stage_done[k]) KV_CUDA(cudaEventCreateWithFlags(&b->stage_done[k], cudaEventDisableTiming));
  char *p = b->stage[k];
  s->hdr = reinterpret_cast<StageHeader *>(p);
  s->slots = reinterpret_cast<int64_t *>(p + 256);
  s->rows = reinterpret_cast<int32_t *>(p + 256 + n * 8);
  s->lens = s->rows + n;
  s->upd = reinterpret_cast<TableUpdate *>(p + 256 + ((n * 16 + 255) & ~(size_t)255));
  s->upd_cap = max_upd;
  memset(s->hdr, 0, sizeof(StageHeader));
  return PA_OK;
}

// Stages the batch: rows, lengths (the tables' own, or `ctx_override`), optionally the
// decode slots, and the table entries that changed.  Launches the ingest kernel.
pa_status sync_batch(PaKvBinding *b, const uint32_t *seq_ids, size_t n, const uint32_t *ctx_override,
                     bool want_slots, const void *const bulk_src[3], void *const bulk_dst[3],
                     const size_t bulk_bytes[3], cudaStream_t st) {
  KV_TRY(ensure_batch(b, n));
  const PagedKVCache &kv = *b->kv->kv;
  // upper bound of the triples: every block of every sequence whose table changed
  size_t max_upd = 0;
  std::vector<const SequenceBlockTable *> tabs(n);
  std::vector<PaKvBinding::Row *> rws(n);
  for (size_t i = 0; i < n; i++) {
    const SequenceBlockTable *t = kv.sequence(seq_ids[i]);
    if (!t) return err("Sequence " + std::to_string(seq_ids[i]) + " not found");
    if (t->num_blocks() > b->MB)
      return err("Sequence " + std::to_string(seq_ids[i]) + " has more blocks than max_seq_len allows");
    tabs[i] = t;
  }
  for (size_t i = 0; i < n; i++) {  // rows first: growing the table synchronises
    KV_TRY(row_for(b, seq_ids[i], &rws[i], st));
    if (rws[i]->version != tabs[i]->version()) max_upd += tabs[i]->num_blocks();
  }
  // row_for may have rehashed the map: take the pointers again
  for (size_t i = 0; i < n; i++) rws[i] = &b->rows.find(seq_ids[i])->second;
  Staged s;
  KV_TRY(stage_area(b, n, max_upd, &s));
  const uint32_t bs = kv.block_size();
  size_t n_upd = 0;
  for (size_t i = 0; i < n; i++) {
    const SequenceBlockTable *t = tabs[i];
    PaKvBinding::Row *r = rws[i];
    if (r->version != t->version()) {
      const auto &blocks = t->blocks();
      if (r->sent.size() > blocks.size()) r->sent.resize(blocks.size());
      for (size_t j = 0; j < blocks.size(); j++) {
        const int32_t id = (int32_t)blocks[j]->block_id;
        if (j < r->sent.size() && r->sent[j] == id) continue;
        if (j < r->sent.size()) r->sent[j] = id;
        else r->sent.push_back(id);
        s.upd[n_upd++] = TableUpdate{r->row, (int32_t)j, id};
      }
      r->version = t->version();
    }
    const uint32_t ctx = ctx_override ? ctx_override[i] : t->num_tokens();
    s.rows[i] = r->row;
    s.lens[i] = (int32_t)ctx;
    if (want_slots) {
      // get_slot_mapping_decode (paged_kv_cache.rs:539-552): position context_len - 1
      if (ctx == 0) return err("Sequence " + std::to_string(seq_ids[i]) + " has context_len 0");
      int64_t slot = -1;
      if (!t->absolute_slot_index(ctx - 1, &slot))
        return err("Position " + std::to_string(ctx - 1) + " is beyond the blocks of sequence " +
                   std::to_string(seq_ids[i]));
      s.slots[i] = slot;
    }
  }
  (void)bs;
  s.hdr->n = (uint32_t)n;
  s.hdr->n_updates = (uint32_t)n_upd;
  s.hdr->has_slots = want_slots ? 1u : 0u;
  size_t bulk_units = 0;
  for (int c = 0; c < 3; c++) {
    s.hdr->src[c] = bulk_src ? static_cast<const uint4 *>(bulk_src[c]) : nullptr;
    s.hdr->dst[c] = bulk_src ? static_cast<uint4 *>(bulk_dst[c]) : nullptr;
    s.hdr->units[c] = bulk_src ? bulk_bytes[c] / 16 : 0;
    bulk_units += s.hdr->units[c];
  }
  b->entries_sent += n_upd;
  b->calls++;
  // device views of the staged arrays
  char *dbase = nullptr;
  KV_CUDA(cudaHostGetDevicePointer(reinterpret_cast<void **>(&dbase), reinterpret_cast<char *>(s.hdr), 0));
  auto dv = [&](const void *host_ptr) {
    return dbase + (reinterpret_cast<const char *>(host_ptr) - reinterpret_cast<const char *>(s.hdr));
  };
  int grid = 1;
  if (bulk_units) grid = (int)std::min<size_t>((bulk_units + 1023) / 1024 + 1, (size_t)2 * b->num_sms);
  ingest_kernel<<<grid, 256, 0, st>>>(
      reinterpret_cast<const StageHeader *>(dv(s.hdr)), reinterpret_cast<const int32_t *>(dv(s.rows)),
      reinterpret_cast<const int32_t *>(dv(s.lens)), reinterpret_cast<const int64_t *>(dv(s.slots)),
      reinterpret_cast<const TableUpdate *>(dv(s.upd)), b->rows_dev, b->lens_dev, b->slots_dev, b->tables_dev,
      (int)b->MB);
  KV_CUDA(cudaGetLastError());
  __atomic_fetch_add(&pa::g_launch_count, 1ull, __ATOMIC_RELAXED);
  const int k = (b->stage_next + PaKvBinding::kRing - 1) % PaKvBinding::kRing;
  KV_CUDA(cudaEventRecord(b->stage_done[k], st));
  return PA_OK;
}

// FP8: the scales the reference would hand its kernels for this layer (paged_kv_cache.rs:826-834)
pa_status apply_scales(PaKvBinding *b, uint32_t layer) {
  if (!b->fp8 || !b->scales) return PA_OK;
  return pa_cache_set_kv_scales(b->cache, layer, b->scales->m.k_scale(layer), b->scales->m.v_scale(layer));
}

pa_status check_binding(const PaKvBinding *b, uint32_t layer) {
  if (!b) return err("binding is null");
  if (layer >= b->cfg.num_layers) return err("Layer " + std::to_string(layer) + " not found");
  return PA_OK;
}

}  // namespace

extern "C" {

pa_status pa_kv_bind(PaKvHost *kv, PagedAttnCache *cache, PaKvBinding **out) {
  if (!out) return err("out is null");
  *out = nullptr;
  if (!kv || !cache) return err("null argument");
  PagedAttnConfig cfg{};
  KV_TRY(pa_cache_get_config(cache, &cfg));
  const PagedAttentionConfig &hc = kv->kv->config();
  if (cfg.block_size != hc.block_size || cfg.num_kv_heads != hc.num_kv_heads || cfg.head_size != hc.head_size ||
      cfg.num_layers != hc.num_layers)
    return err("host cache and device cache disagree on block_size / num_kv_heads / head_size / num_layers");
  if (cfg.num_blocks < kv->kv->total_blocks())
    return err("device cache has fewer blocks than the host allocator hands out");
  PaKvBinding *b = new (std::nothrow) PaKvBinding();
  if (!b) return err("host allocation failed", PA_ERR_OOM);
  b->kv = kv;
  b->cache = cache;
  b->cfg = cfg;
  b->fp8 = pa_cache_is_fp8(cache) != 0;
  b->MB = kv->kv->max_blocks_per_seq();
  // the device the pools live on
  cudaPointerAttributes attr{};
  if (cudaPointerGetAttributes(&attr, pa_cache_key_ptr(cache, 0)) == cudaSuccess) b->device = attr.device;
  DeviceScope g(b->device);
  pa_status st = PA_OK;
  do {
    cudaError_t e = cudaDeviceGetAttribute(&b->num_sms, cudaDevAttrMultiProcessorCount, b->device);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&b->stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaMalloc(&b->scalar_dev, 64);
    b->ws_bytes = pa_attention_workspace_bytes(cache);
    if (e == cudaSuccess) e = cudaMalloc(&b->ws, b->ws_bytes);
    if (e != cudaSuccess) {
      st = cuda_err(e, "pa_kv_bind");
      break;
    }
    if (b->fp8) {  // PagedKVCache::new, paged_kv_cache.rs:75-83: a manager with default scales
      b->scales = new (std::nothrow) PaKvScaleManager(cfg.num_layers, 0.1f);
      if (b->scales) b->scales->m.init_default_scales();
    }
  } while (false);
  if (st != PA_OK) {
    const std::string keep = pa_last_error_string();
    pa_kv_unbind(b);
    return pa::set_error(st, keep);
  }
  *out = b;
  return PA_OK;
}

void pa_kv_unbind(PaKvBinding *b) {
  if (!b) return;
  DeviceScope g(b->device);
  if (b->stream) cudaStreamSynchronize(b->stream);
  for (int k = 0; k < PaKvBinding::kRing; k++) {
    if (b->stage_done[k]) {
      cudaEventSynchronize(b->stage_done[k]);
      cudaEventDestroy(b->stage_done[k]);
    }
    if (b->stage[k]) cudaFreeHost(b->stage[k]);
  }
  if (b->tables_dev) cudaFree(b->tables_dev);
  if (b->rows_dev) cudaFree(b->rows_dev);
  if (b->lens_dev) cudaFree(b->lens_dev);
  if (b->slots_dev) cudaFree(b->slots_dev);
  if (b->ws) cudaFree(b->ws);
  if (b->io) cudaFree(b->io);
  if (b->scalar_dev) cudaFree(b->scalar_dev);
  if (b->stream) cudaStreamDestroy(b->stream);
  delete b->scales;
  delete b;
}

pa_status pa_kv_update(PaKvBinding *b, uint32_t layer, const void *keys, const void *values,
                       const int64_t *slots_dev, int64_t num_tokens, void *stream) {
  KV_TRY(check_binding(b, layer));
  DeviceScope g(b->device);
  KV_TRY(apply_scales(b, layer));
  const int64_t row = (int64_t)b->cfg.num_kv_heads * b->cfg.head_size;
  return pa_reshape_and_cache(b->cache, layer, keys, values, slots_dev, num_tokens, row, row, stream);
}

pa_status pa_kv_update_with_slots(PaKvBinding *b, uint32_t layer, const void *keys, const void *values,
                                  const int64_t *slots_host, int64_t num_tokens, void *stream) {
  KV_TRY(check_binding(b, layer));
  if (num_tokens < 0) return err("num_tokens < 0");
  if (num_tokens == 0) return PA_OK;
  if (!slots_host) return err("slot_mapping is null");
  DeviceScope g(b->device);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // the slots travel through a staging area of the ring (reused only after its copy ran)
  Staged s;
  KV_TRY(stage_area(b, (size_t)num_tokens, 0, &s));
  memcpy(s.slots, slots_host, (size_t)num_tokens * 8);
  KV_TRY(grow_dev(reinterpret_cast<void **>(&b->io), &b->io_cap, (size_t)num_tokens * 8));
  KV_CUDA(cudaMemcpyAsync(b->io, s.slots, (size_t)num_tokens * 8, cudaMemcpyHostToDevice, st));
  const int k = (b->stage_next + PaKvBinding::kRing - 1) % PaKvBinding::kRing;
  KV_CUDA(cudaEventRecord(b->stage_done[k], st));
  KV_TRY(apply_scales(b, layer));
  const int64_t row = (int64_t)b->cfg.num_kv_heads * b->cfg.head_size;
  return pa_reshape_and_cache(b->cache, layer, keys, values, reinterpret_cast<const int64_t *>(b->io),
                              num_tokens, row, row, stream);
}

static pa_status attention_common(PaKvBinding *b, uint32_t layer, void *out, const void *q,
                                  const uint32_t *seq_ids, const uint32_t *ctx, size_t n, uint32_t Hq,
                                  float scale, void *stream) {
  KV_TRY(check_binding(b, layer));
  if (n == 0) return PA_OK;
  if (!seq_ids || !out || !q) return err("null argument");
  DeviceScope g(b->device);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  KV_TRY(sync_batch(b, seq_ids, n, ctx, false, nullptr, nullptr, nullptr, st));
  KV_TRY(apply_scales(b, layer));
  const int64_t row = (int64_t)Hq * b->cfg.head_size;
  return pa_paged_attention_decode_rows(b->cache, layer, out, q, b->tables_dev, b->rows_dev, b->lens_dev,
                                        (int32_t)n, (int32_t)Hq, (int32_t)b->MB, row, row, scale, 1.0f, b->ws,
                                        b->ws_bytes, stream);
}

pa_status pa_kv_attention(PaKvBinding *b, uint32_t layer, void *out, const void *q, const uint32_t *seq_ids,
                          size_t n, uint32_t Hq, float scale, void *stream) {
  return attention_common(b, layer, out, q, seq_ids, nullptr, n, Hq, scale, stream);
}

pa_status pa_kv_attention_with_context(PaKvBinding *b, uint32_t layer, void *out, const void *q,
                                       const uint32_t *seq_ids, const uint32_t *context_lens, size_t n,
                                       uint32_t Hq, float scale, void *stream) {
  if (n && !context_lens) return err("context_lens is null");
  return attention_common(b, layer, out, q, seq_ids, context_lens, n, Hq, scale, stream);
}

pa_status pa_kv_decode_step(PaKvBinding *b, uint32_t layer, void *out, const void *q, const void *keys,
                            const void *values, const uint32_t *seq_ids, size_t n, uint32_t Hq, float scale,
                            void *stream) {
  KV_TRY(check_binding(b, layer));
  if (n == 0) return PA_OK;
  if (!seq_ids || !out || !q || !keys || !values) return err("null argument");
  DeviceScope g(b->device);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  KV_TRY(sync_batch(b, seq_ids, n, nullptr, true, nullptr, nullptr, nullptr, st));
  KV_TRY(apply_scales(b, layer));
  const int64_t row = (int64_t)Hq * b->cfg.head_size, kv_row = (int64_t)b->cfg.num_kv_heads * b->cfg.head_size;
  return pa_decode_step_rows(b->cache, layer, out, q, keys, values, b->slots_dev, b->tables_dev, b->rows_dev,
                             b->lens_dev, (int32_t)n, (int32_t)Hq, (int32_t)b->MB, row, row, kv_row, kv_row,
                             scale, 1.0f, b->ws, b->ws_bytes, stream);
}

pa_status pa_kv_decode_step_host(PaKvBinding *b, uint32_t layer, void *out_host, const void *q_host,
                                 const void *k_host, const void *v_host, const uint32_t *seq_ids, size_t n,
                                 uint32_t Hq, float scale) {
  KV_TRY(check_binding(b, layer));
  if (n == 0) return PA_OK;
  if (!seq_ids || !out_host || !q_host || !k_host || !v_host) return err("null host pointer");
  DeviceScope g(b->device);
  cudaStream_t st = b->stream;
  const size_t D = b->cfg.head_size, Hkv = b->cfg.num_kv_heads;
  auto up = [](size_t x) { return (x + 255) & ~(size_t)255; };
  const size_t q_b = n * Hq * D * 2, kv_b = n * Hkv * D * 2;
  const size_t o_q = 0, o_k = up(q_b), o_v = o_k + up(kv_b), o_out = o_v + up(kv_b), total = o_out + up(q_b);
  KV_TRY(grow_dev(reinterpret_cast<void **>(&b->io), &b->io_cap, total));
  char *io = b->io;
  // Pinned (device-mapped) buffers are read in place by the ingest launch, next to the
  // batch's metadata; pageable ones go through the copy engine first.
  auto mapped = [](const void *h) -> const void * {
    cudaPointerAttributes a{};
    if (cudaPointerGetAttributes(&a, h) != cudaSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    return a.type == cudaMemoryTypeHost && !((uintptr_t)a.devicePointer & 15u) ? a.devicePointer : nullptr;
  };
  const void *src[3] = {mapped(q_host), mapped(k_host), mapped(v_host)};
  void *dst[3] = {io + o_q, io + o_k, io + o_v};
  const size_t bytes[3] = {q_b, kv_b, kv_b};
  // Small batches: the ingest launch reads the three arrays itself (one launch instead of
  // three copies, about 10 us for 0.3 MB).  Large ones go through the copy engine, which
  // moves a few megabytes at the full PCIe rate where SM loads from host memory reach about
  // two thirds of it (measured: 2.6 MB in 72 us against 47 us).
  const bool zero_copy = src[0] && src[1] && src[2] && q_b + 2 * kv_b <= ((size_t)512 << 10);
  if (!zero_copy) {
    KV_CUDA(cudaMemcpyAsync(io + o_q, q_host, q_b, cudaMemcpyHostToDevice, st));
    KV_CUDA(cudaMemcpyAsync(io + o_k, k_host, kv_b, cudaMemcpyHostToDevice, st));
    KV_CUDA(cudaMemcpyAsync(io + o_v, v_host, kv_b, cudaMemcpyHostToDevice, st));
  }
  KV_TRY(sync_batch(b, seq_ids, n, nullptr, true, zero_copy ? src : nullptr, dst, bytes, st));
  KV_TRY(apply_scales(b, layer));
  const int64_t row = (int64_t)Hq * D, kv_row = (int64_t)Hkv * D;
  KV_TRY(pa_decode_step_rows(b->cache, layer, io + o_out, io + o_q, io + o_k, io + o_v, b->slots_dev,
                             b->tables_dev, b->rows_dev, b->lens_dev, (int32_t)n, (int32_t)Hq, (int32_t)b->MB,
                             row, row, kv_row, kv_row, scale, 1.0f, b->ws, b->ws_bytes, st));
  KV_CUDA(cudaMemcpyAsync(out_host, io + o_out, q_b, cudaMemcpyDeviceToHost, st));
  KV_CUDA(cudaStreamSynchronize(st));
  return pa_cache_check_errors_fast(b->cache, st);
}

void pa_kv_binding_stats(const PaKvBinding *b, uint64_t *entries, uint64_t *calls, uint32_t *rows) {
  if (!b) return;
  if (entries) *entries = b->entries_sent;
  if (calls) *calls = b->calls;
  if (rows) *rows = (uint32_t)b->rows.size();
}

PaKvScaleManager *pa_kv_scale_manager(PaKvBinding *b) { return b ? b->scales : nullptr; }

/* ---- scale manager ---------------------------------------------------------------- */
PaKvScaleManager *pa_scale_create(uint32_t num_layers, float alpha) {
  return new (std::nothrow) PaKvScaleManager(num_layers, alpha);
}
void pa_scale_destroy(PaKvScaleManager *m) { delete m; }
uint32_t pa_scale_num_layers(const PaKvScaleManager *m) { return m ? m->m.num_layers() : 0; }
float pa_scale_alpha(const PaKvScaleManager *m) { return m ? m->m.alpha() : 0.f; }
void pa_scale_init_default_scales(PaKvScaleManager *m) { if (m) m->m.init_default_scales(); }
float pa_scale_k(const PaKvScaleManager *m, uint32_t layer) { return m ? m->m.k_scale(layer) : 1.f; }
float pa_scale_v(const PaKvScaleManager *m, uint32_t layer) { return m ? m->m.v_scale(layer) : 1.f; }
int32_t pa_scale_is_calibrated(const PaKvScaleManager *m) { return m && m->m.is_calibrated(); }
void pa_scale_calibrate_layer_max(PaKvScaleManager *m, uint32_t layer, float k_max, float v_max, float *k,
                                  float *v) {
  if (!m) return;
  const auto r = m->m.calibrate_layer(layer, k_max, v_max);
  if (k) *k = r.first;
  if (v) *v = r.second;
}
void pa_scale_update_layer_ema_max(PaKvScaleManager *m, uint32_t layer, float k_max, float v_max, float *k,
                                   float *v) {
  if (!m) return;
  const auto r = m->m.update_layer_ema(layer, k_max, v_max);
  if (k) *k = r.first;
  if (v) *v = r.second;
}
pa_status pa_scale_calibrate_layer(PaKvScaleManager *m, uint32_t layer, const void *keys, const void *values,
                                   size_t count, int32_t dtype, int32_t ema, float *k_scale, float *v_scale,
                                   void *stream) {
  if (!m) return err("scale manager is null");
  if (!keys || !values) return err("Null tensor pointer");
  if (dtype != 0 && dtype != 1) return err("dtype must be 0 (f16) or 1 (bf16)", PA_ERR_UNSUPPORTED);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  unsigned *words = nullptr;
  KV_CUDA(cudaMalloc(&words, 8));
  unsigned host[2] = {0u, 0u};
  cudaError_t e = cudaMemsetAsync(words, 0, 8, st);
  if (e == cudaSuccess && count) {
    const int grid = (int)std::min<size_t>((count + 4095) / 4096, 1184);
    max_abs_kernel<<<grid, 256, 0, st>>>(static_cast<const uint16_t *>(keys), count, dtype == 0, words);
    max_abs_kernel<<<grid, 256, 0, st>>>(static_cast<const uint16_t *>(values), count, dtype == 0, words + 1);
    __atomic_fetch_add(&pa::g_launch_count, 2ull, __ATOMIC_RELAXED);
    e = cudaGetLastError();
  }
  if (e == cudaSuccess) e = cudaMemcpyAsync(host, words, 8, cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  cudaFree(words);
  if (e != cudaSuccess) return cuda_err(e, "pa_scale_calibrate_layer");
  float km, vm;
  memcpy(&km, &host[0], 4);
  memcpy(&vm, &host[1], 4);
  if (ema) pa_scale_update_layer_ema_max(m, layer, km, vm, k_scale, v_scale);
  else pa_scale_calibrate_layer_max(m, layer, km, vm, k_scale, v_scale);
  return PA_OK;
}
void pa_scale_set_scales(PaKvScaleManager *m, uint32_t layer, float k, float v) { if (m) m->m.set_scales(layer, k, v); }
void pa_scale_get_all_scales(const PaKvScaleManager *m, float *k_out, float *v_out) {
  if (!m) return;
  std::vector<float> k, v;
  m->m.get_all_scales(&k, &v);
  if (k_out) memcpy(k_out, k.data(), k.size() * 4);
  if (v_out) memcpy(v_out, v.data(), v.size() * 4);
}
void pa_scale_load_scales(PaKvScaleManager *m, const float *k, size_t nk, const float *v, size_t nv) {
  if (m) m->m.load_scales(k, k ? nk : 0, v, v ? nv : 0);
}
void pa_scale_reset(PaKvScaleManager *m) { if (m) m->m.reset(); }
void pa_scale_stats(const PaKvScaleManager *m, PaKvScaleStats *out) {
  if (!m || !out) return;
  const KvScaleStats s = m->m.stats();
  *out = PaKvScaleStats{s.num_layers_calibrated, s.k_scale_min, s.k_scale_max, s.k_scale_mean,
                        s.v_scale_min, s.v_scale_max, s.v_scale_mean};
}

}  // extern "C"

/* ---- input metadata ----------------------------------------------------------------- */
struct PaInputMetadata {
  InputMetadata m;
  int device = -1;
  int32_t *tables_dev = nullptr, *lens_dev = nullptr;
  int64_t *slots_dev = nullptr;
};

extern "C" {

PaInputMetadata *pa_metadata_create(const int32_t *tables, size_t nt, const int32_t *lens, size_t ns,
                                    const int64_t *slots, size_t nk, uint32_t max_ctx, int32_t is_prefill,
                                    uint32_t MB) {
  PaInputMetadata *m = new (std::nothrow) PaInputMetadata();
  if (!m) return nullptr;
  if (tables) m->m.block_tables.assign(tables, tables + nt);
  if (lens) m->m.context_lens.assign(lens, lens + ns);
  if (slots) m->m.slot_mappings.assign(slots, slots + nk);
  m->m.max_context_len = max_ctx;
  m->m.is_prefill = is_prefill != 0;
  m->m.num_seqs = (uint32_t)m->m.context_lens.size();
  m->m.max_blocks_per_seq = MB;
  return m;
}
PaInputMetadata *pa_metadata_dummy(void) {
  const int32_t t = 0, l = 1;
  const int64_t s = 0;
  return pa_metadata_create(&t, 1, &l, 1, &s, 1, 1, 1, 1);
}
void pa_metadata_invalidate_buffers(PaInputMetadata *m) {
  if (!m || m->device < 0) return;
  DeviceScope g(m->device);
  cudaFree(m->tables_dev);
  cudaFree(m->lens_dev);
  cudaFree(m->slots_dev);
  m->tables_dev = m->lens_dev = nullptr;
  m->slots_dev = nullptr;
  m->device = -1;
}
void pa_metadata_destroy(PaInputMetadata *m) {
  pa_metadata_invalidate_buffers(m);
  delete m;
}
uint32_t pa_metadata_num_seqs(const PaInputMetadata *m) { return m ? m->m.num_seqs : 0; }
size_t pa_metadata_num_tokens(const PaInputMetadata *m) { return m ? m->m.slot_mappings.size() : 0; }
int32_t pa_metadata_is_prefill(const PaInputMetadata *m) { return m && m->m.is_prefill; }
uint32_t pa_metadata_max_context_len(const PaInputMetadata *m) { return m ? m->m.max_context_len : 0; }
uint32_t pa_metadata_max_blocks_per_seq(const PaInputMetadata *m) { return m ? m->m.max_blocks_per_seq : 0; }

pa_status pa_metadata_device_buffers(PaInputMetadata *m, int32_t device, const int32_t **tables,
                                     const int32_t **lens, const int64_t **slots) {
  if (!m) return err("metadata is null");
  if (m->device >= 0 && m->device != device) pa_metadata_invalidate_buffers(m);
  if (m->device < 0) {
    DeviceScope g(device);
    auto upload = [&](void **dst, const void *src, size_t bytes) -> cudaError_t {
      cudaError_t e = cudaMalloc(dst, bytes ? bytes : 16);
      if (e == cudaSuccess && bytes) e = cudaMemcpy(*dst, src, bytes, cudaMemcpyHostToDevice);
      return e;
    };
    cudaError_t e = upload(reinterpret_cast<void **>(&m->tables_dev), m->m.block_tables.data(),
                           m->m.block_tables.size() * 4);
    if (e == cudaSuccess)
      e = upload(reinterpret_cast<void **>(&m->lens_dev), m->m.context_lens.data(), m->m.context_lens.size() * 4);
    if (e == cudaSuccess)
      e = upload(reinterpret_cast<void **>(&m->slots_dev), m->m.slot_mappings.data(),
                 m->m.slot_mappings.size() * 8);
    m->device = device;
    if (e != cudaSuccess) {
      pa_metadata_invalidate_buffers(m);
      return cuda_err(e, "pa_metadata_device_buffers");
    }
  }
  if (tables) *tables = m->tables_dev;
  if (lens) *lens = m->lens_dev;
  if (slots) *slots = m->slots_dev;
  return PA_OK;
}

/* ---- attention layer ------------------------------------------------------------------ */
PaAttentionLayer *pa_layer_create(const PaLayerParams *p) {
  if (!p) return nullptr;
  AttentionLayerParams a;
  a.layer_idx = p->layer_idx;
  a.num_heads = p->num_heads;
  a.num_kv_heads = p->num_kv_heads;
  a.head_size = p->head_size;
  a.scale = p->scale;
  a.block_size = p->block_size;
  a.softcap = p->softcap;
  a.use_fp8 = p->use_fp8 != 0;
  a.k_scale = p->k_scale;
  a.v_scale = p->v_scale;
  return new (std::nothrow) PaAttentionLayer(AttentionLayer(a));
}
PaAttentionLayer *pa_layer_from_cache_config(uint32_t layer_idx, uint32_t num_heads, const PaHostConfig *c) {
  if (!c) return nullptr;
  PagedAttentionConfig cfg;
  cfg.block_size = c->block_size;
  cfg.head_size = c->head_size;
  cfg.num_kv_heads = c->num_kv_heads;
  cfg.num_layers = c->num_layers;
  cfg.use_fp8_cache = c->use_fp8_cache != 0;
  return new (std::nothrow) PaAttentionLayer(AttentionLayer::from_cache_config(layer_idx, num_heads, cfg));
}
void pa_layer_destroy(PaAttentionLayer *l) { delete l; }
void pa_layer_get(const PaAttentionLayer *l, PaLayerParams *out) {
  if (!l || !out) return;
  const AttentionLayer &a = l->l;
  *out = PaLayerParams{a.layer_idx, a.num_heads, a.num_kv_heads, a.head_size, a.scale, a.block_size,
                       a.softcap, a.use_fp8 ? 1u : 0u, a.k_scale, a.v_scale};
}
void pa_layer_set_kv_scales(PaAttentionLayer *l, float k, float v) {
  if (!l) return;
  l->l.k_scale = k;
  l->l.v_scale = v;
}

pa_status pa_layer_forward(const PaAttentionLayer *l, PaKvBinding *b, void *out, const void *q, const void *k,
                           const void *v, PaInputMetadata *meta, int32_t *has_output, void *stream) {
  if (!l || !meta || !has_output) return err("null argument");
  *has_output = 0;
  const AttentionLayer &a = l->l;
  KV_TRY(check_binding(b, a.layer_idx));
  if (a.num_kv_heads != b->cfg.num_kv_heads || a.head_size != b->cfg.head_size || a.block_size != b->cfg.block_size)
    return err("layer geometry differs from the cache's");
  if (a.use_fp8 != b->fp8) return err("layer and cache disagree on the FP8 cache");
  DeviceScope g(b->device);
  const int32_t *tables = nullptr, *lens = nullptr;
  const int64_t *slots = nullptr;
  KV_TRY(pa_metadata_device_buffers(meta, b->device, &tables, &lens, &slots));
  // the layer's own scales (attention_layer.rs:273-285), not the cache manager's
  if (b->fp8) KV_TRY(pa_cache_set_kv_scales(b->cache, a.layer_idx, a.k_scale, a.v_scale));
  const int64_t kv_row = (int64_t)a.num_kv_heads * a.head_size;
  // step 1: K/V of every token of the batch (attention_layer.rs:268-313)
  KV_TRY(pa_reshape_and_cache(b->cache, a.layer_idx, k, v, slots, (int64_t)meta->m.slot_mappings.size(), kv_row,
                              kv_row, stream));
  // step 2: prefill -> the caller attends densely (:316-318)
  if (meta->m.is_prefill) return PA_OK;
  // step 3: decode
  const int64_t row = (int64_t)a.num_heads * a.head_size;
  KV_TRY(pa_paged_attention_decode(b->cache, a.layer_idx, out, q, tables, lens, (int32_t)meta->m.num_seqs,
                                   (int32_t)a.num_heads, (int32_t)meta->m.max_blocks_per_seq, row, row, a.scale,
                                   a.softcap, b->ws, b->ws_bytes, stream));
  *has_output = 1;
  return PA_OK;
}

pa_status pa_layer_forward_decode(const PaAttentionLayer *l, PaKvBinding *b, void *out, const void *q,
                                  const void *k, const void *v, PaInputMetadata *meta, void *stream) {
  if (!meta) return err("null argument");
  if (meta->m.is_prefill) return err("forward_decode called during prefill phase. Use forward() instead.");
  int32_t has = 0;
  KV_TRY(pa_layer_forward(l, b, out, q, k, v, meta, &has, stream));
  return has ? PA_OK : err("Expected output for decode phase");
}

}  // extern "C"

struct PaAttentionLayers {
  std::vector<PaAttentionLayer> layers;
};

extern "C" {

PaAttentionLayers *pa_layers_create(uint32_t num_layers, uint32_t num_heads, uint32_t num_kv_heads,
                                    uint32_t head_size, uint32_t block_size, int32_t use_fp8) {
  PaAttentionLayers *ls = new (std::nothrow) PaAttentionLayers();
  if (!ls) return nullptr;
  for (uint32_t i = 0; i < num_layers; i++) {
    AttentionLayerParams a;
    a.layer_idx = i;
    a.num_heads = num_heads;
    a.num_kv_heads = num_kv_heads;
    a.head_size = head_size;
    a.block_size = block_size;
    a.use_fp8 = use_fp8 != 0;
    ls->layers.emplace_back(AttentionLayer(a));
  }
  return ls;
}
PaAttentionLayers *pa_layers_from_cache_config(uint32_t num_heads, const PaHostConfig *c) {
  if (!c) return nullptr;
  return pa_layers_create(c->num_layers, num_heads, c->num_kv_heads, c->head_size, c->block_size,
                          (int32_t)c->use_fp8_cache);
}
void pa_layers_destroy(PaAttentionLayers *ls) { delete ls; }
const PaAttentionLayer *pa_layers_get(const PaAttentionLayers *ls, uint32_t i) {
  return ls && i < ls->layers.size() ? &ls->layers[i] : nullptr;
}
uint32_t pa_layers_num_layers(const PaAttentionLayers *ls) { return ls ? (uint32_t)ls->layers.size() : 0; }

pa_status pa_kv_create_bound(const PaHostConfig *cfg, int32_t device, uint32_t dtype, PaKvHost **kv_out,
                             PagedAttnCache **cache_out, PaKvBinding **binding_out) {
  if (!cfg || !kv_out || !cache_out || !binding_out) return err("null argument");
  *kv_out = nullptr;
  *cache_out = nullptr;
  *binding_out = nullptr;
  KV_TRY(pa_host_config_validate(cfg));
  PaKvHost *kv = nullptr;
  KV_TRY(pa_kv_create(cfg, &kv));
  PagedAttnConfig dc{cfg->block_size, kv->kv->total_blocks(), cfg->head_size, cfg->num_kv_heads, cfg->num_layers,
                     dtype};
  PagedAttnCache *cache = nullptr;
  pa_status st = cfg->use_fp8_cache ? pa_cache_create_fp8(&dc, device, &cache) : pa_cache_create(&dc, device, &cache);
  PaKvBinding *b = nullptr;
  if (st == PA_OK) st = pa_kv_bind(kv, cache, &b);
  if (st != PA_OK) {
    const std::string keep = pa_last_error_string();
    pa_cache_free(cache);
    pa_kv_destroy(kv);
    return pa::set_error(st, keep);
  }
  *kv_out = kv;
  *cache_out = cache;
  *binding_out = b;
  return PA_OK;
}

}  // extern "C"
