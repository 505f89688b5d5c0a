// C ABI of the library (declared in include/paged_attn_b200.h): cache handle,
// argument validation, launch orchestration, the reference-named tier-1 entry
// points and the host-buffer decode step.  No tensor-library types cross this
// boundary and there is no CPU fallback: without a CUDA device every compute
// entry fails with PA_ERR_CUDA.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <cmath>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/paged_attn_b200.h"
#include "pa_common.cuh"

namespace {

thread_local std::string t_err;
thread_local int t_device = 0;
thread_local cudaStream_t t_stream = nullptr;

pa_status fail(pa_status code, const std::string &msg) {
  t_err = msg;
  return code;
}
pa_status cuda_fail(cudaError_t e, const char *what) {
  return fail(e == cudaErrorMemoryAllocation ? PA_ERR_OOM : PA_ERR_CUDA,
              std::string(what) + ": " + cudaGetErrorString(e));
}
#define PA_CUDA(call)                                        \
  do {                                                       \
    cudaError_t e_ = (call);                                 \
    if (e_ != cudaSuccess) return cuda_fail(e_, #call);      \
  } while (0)

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

struct DeviceGuard {
  int prev = -1;
  bool ok = false;
  explicit DeviceGuard(int dev) {
    if (cudaGetDevice(&prev) != cudaSuccess) return;
    ok = prev == dev || cudaSetDevice(dev) == cudaSuccess;
    if (prev == dev) prev = -1;
  }
  ~DeviceGuard() {
    if (prev >= 0) cudaSetDevice(prev);
  }
};

}  // namespace

namespace pa {
// shared with the host-logic ABI (host_api.cpp): same per-thread error string
int32_t set_error(int32_t code, const std::string &msg) { return fail(code, msg); }
}  // namespace pa

struct PagedAttnCache {
  PagedAttnConfig cfg{};
  int device = 0;
  bool owns = false;
  int num_sms = 0;
  std::vector<void *> k, v;
  // FP8 (E4M3) pools: one byte per element; cfg.dtype is then the type of q, out and of
  // the keys and values handed to the write.  Per-layer dequantisation factors.
  bool fp8 = false;
  std::vector<float> k_scale, v_scale;
  std::vector<pa::TensorMapBlob> v_maps;  // per layer: tensor map of the V pool (16-bit pools)
  std::vector<pa::TensorMapBlob> k_maps;  // per layer: row view of the K pool (16-bit pools, 16-token blocks)
  // the tile kernel that fetches K by TMA gather serves 16-bit pools of 16-token blocks
  bool has_tile64() const { return !fp8 && bs_shift == 0 && cfg.head_size == (uint32_t)pa::kHeadSize; }
  // log2(block_size / 16): -1, 0 or 1.  32-token blocks: per layer, the maps that fetch
  // one 16-token unit of a chunk for the split-KV kernel
  int bs_shift = 0;
  std::vector<pa::UnitMaps> unit_maps;
  const pa::UnitMaps *unit_map(uint32_t layer) const {
    return bs_shift > 0 && !unit_maps.empty() ? &unit_maps[layer] : nullptr;
  }
  // the tcgen05 tile kernel reads pools of 16- or 32-token blocks (16-bit or FP8)
  bool has_tile_kernel() const { return bs_shift >= 0 && cfg.head_size == (uint32_t)pa::kHeadSize; }
  unsigned *err_dev = nullptr;
  // pinned, device-mapped copy of the error word, written by the last kernel of an
  // attention call, so that the host-buffer step reads it without a copy of its own
  unsigned *err_host = nullptr, *err_host_dev = nullptr;
  // FP8: device word next to the error word, non-zero once a pool may hold a byte with
  // exponent field 15 (infinity / NaN in the cache format)
  unsigned *fp8_special() const { return err_dev + 16; }
  // arrival counters of the split-KV kernel (pa::AttnParams::sync): zero between launches
  unsigned *sync_dev = nullptr;
  // scratch owned by the handle: attention workspace for tier 1 / the host step,
  // per-call metadata (cu_q_lens copy, tile work list), host-step staging
  void *ws = nullptr;
  size_t ws_bytes = 0;
  void *meta = nullptr;
  size_t meta_bytes = 0;
  void *stage = nullptr;
  size_t stage_bytes = 0;
  cudaStream_t step_stream = nullptr;
  // second stream and fork/join events for calls that run two kernels side by side
  cudaStream_t aux_stream = nullptr;
  cudaStream_t lane_stream[2] = {nullptr, nullptr};
  cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
  cudaEvent_t ev_lane[2] = {nullptr, nullptr};
};

struct mlx_array {
  void *data = nullptr;
  int32_t dtype = 1;
  int32_t device = 0;
  size_t ndim = 0;
  int64_t shape[8] = {0};
  bool owns = false;
  // set on the views mlx_paged_attn_get_key_cache / get_value_cache return, so that
  // forward can run on the cache's own handle (error word, scratch) without setting one up
  PagedAttnCache *owner = nullptr;
  uint32_t layer = 0;
};

namespace {

size_t dtype_size(int32_t d) {
  switch (d) {
    case 0: case 1: return 2;
    case 2: case 3: case 5: return 4;
    case 4: return 8;
    default: return 0;
  }
}

pa_status validate_config(const PagedAttnConfig *c) {
  if (!c) return fail(PA_ERR_INVALID_ARG, "config is null");
  // Same acceptance rules as PagedAttentionConfig::validate
  // (crates/mlx-paged-attn/src/config.rs:36-75) before the narrower "built" test.
  static const uint32_t heads[] = {32, 64, 80, 96, 112, 120, 128, 192, 256};
  bool head_ok = false;
  for (uint32_t hs : heads) head_ok |= hs == c->head_size;
  if (c->block_size != 8 && c->block_size != 16 && c->block_size != 32)
    return fail(PA_ERR_INVALID_ARG, "block_size must be 8, 16, or 32");
  if (!head_ok) return fail(PA_ERR_INVALID_ARG, "unsupported head_size");
  if (c->num_blocks == 0 || c->num_kv_heads == 0 || c->num_layers == 0)
    return fail(PA_ERR_INVALID_ARG, "num_blocks, num_kv_heads and num_layers must be > 0");
  if (c->dtype > 2) return fail(PA_ERR_INVALID_ARG, "dtype must be 0 (f16), 1 (bf16) or 2 (f32)");
  if (c->dtype == 2) return fail(PA_ERR_UNSUPPORTED, "dtype 2 (f32) is not built; use 0 (f16) or 1 (bf16)");
  if (c->head_size != pa::kHeadSize && (c->block_size == 8 || (c->block_size == 32 && c->head_size > pa::kHeadSize)))
    return fail(PA_ERR_UNSUPPORTED, "head sizes other than 128 are built for 16-token blocks and, up to 128, "
                                    "for 32-token blocks");
  // with 32-token blocks a unit is addressed as 2 * (block * heads + head) + half in 32 bits
  if (c->block_size == 32 && (uint64_t)c->num_blocks * c->num_kv_heads >= (1ull << 31))
    return fail(PA_ERR_INVALID_ARG, "num_blocks * num_kv_heads must be below 2^31 with block_size 32");
  return PA_OK;
}

size_t layer_bytes(const PagedAttnConfig &c, bool fp8) {
  return (size_t)c.num_blocks * c.num_kv_heads * c.head_size * c.block_size * (fp8 ? 1 : 2);
}
int64_t block_bytes_of(const PagedAttnCache *c) {  // K (or V) bytes of one block, all heads
  return (int64_t)c->cfg.num_kv_heads * c->cfg.head_size * c->cfg.block_size * (c->fp8 ? 1 : 2);
}

pa_status finish_create(PagedAttnCache *c) {
  int sms = 0;
  PA_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, c->device));
  int major = 0;
  PA_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, c->device));
  if (major != 10) return fail(PA_ERR_UNSUPPORTED, "this library is built for sm_100a only");
  c->num_sms = sms;
  c->bs_shift = c->cfg.block_size == 32 ? 1 : (c->cfg.block_size == 8 ? -1 : 0);
  PA_CUDA(cudaMalloc(&c->err_dev, 256));
  PA_CUDA(cudaMemset(c->err_dev, 0, 256));
  PA_CUDA(cudaMalloc(&c->sync_dev, pa::kSyncWords * sizeof(unsigned)));
  PA_CUDA(cudaMemset(c->sync_dev, 0, pa::kSyncWords * sizeof(unsigned)));
  PA_CUDA(cudaHostAlloc(reinterpret_cast<void **>(&c->err_host), 64,
                        cudaHostAllocMapped | cudaHostAllocPortable));
  *c->err_host = 0;
  PA_CUDA(cudaHostGetDevicePointer(reinterpret_cast<void **>(&c->err_host_dev), c->err_host, 0));
  PA_CUDA(pa::splitkv_configure());
  PA_CUDA(pa::tile_configure());
  PA_CUDA(pa::tile64_configure());
  // the tile kernel fetches V of 16-bit pools through a tensor map (FP8 pools are read with
  // plain loads: their entries stay zero and unused)
  c->v_maps.assign(c->cfg.num_layers, pa::TensorMapBlob{});
  if (!c->fp8 && c->has_tile_kernel()) {
    for (uint32_t i = 0; i < c->cfg.num_layers; i++)
      PA_CUDA(pa::tile_encode_v_map(&c->v_maps[i], c->v[i],
                                    (uint64_t)c->cfg.num_blocks * c->cfg.num_kv_heads,
                                    (int)c->cfg.block_size));
  }
  if (c->has_tile64()) {
    c->k_maps.assign(c->cfg.num_layers, pa::TensorMapBlob{});
    for (uint32_t i = 0; i < c->cfg.num_layers; i++)
      PA_CUDA(pa::tile64_encode_k_map(&c->k_maps[i], c->k[i], (uint64_t)c->cfg.num_blocks * c->cfg.num_kv_heads));
  }
  if (c->bs_shift > 0 && c->cfg.head_size == (uint32_t)pa::kHeadSize) {
    c->unit_maps.resize(c->cfg.num_layers);
    for (uint32_t i = 0; i < c->cfg.num_layers; i++)
      PA_CUDA(pa::encode_unit_maps(&c->unit_maps[i], c->k[i], c->v[i],
                                   (uint64_t)c->cfg.num_blocks * c->cfg.num_kv_heads,
                                   (int)c->cfg.block_size, c->fp8));
  }
  PA_CUDA(cudaStreamCreateWithFlags(&c->step_stream, cudaStreamNonBlocking));
  PA_CUDA(cudaStreamCreateWithFlags(&c->aux_stream, cudaStreamNonBlocking));
  PA_CUDA(cudaEventCreateWithFlags(&c->ev_fork, cudaEventDisableTiming));
  PA_CUDA(cudaEventCreateWithFlags(&c->ev_join, cudaEventDisableTiming));
  for (int i = 0; i < 2; i++) {
    PA_CUDA(cudaStreamCreateWithFlags(&c->lane_stream[i], cudaStreamNonBlocking));
    PA_CUDA(cudaEventCreateWithFlags(&c->ev_lane[i], cudaEventDisableTiming));
  }
  return PA_OK;
}

pa_status grow(void **buf, size_t *have, size_t need) {
  if (*have >= need) return PA_OK;
  if (*buf) PA_CUDA(cudaFree(*buf));
  *buf = nullptr;
  *have = 0;
  const size_t sz = (need + (1u << 20) - 1) & ~((size_t)(1u << 20) - 1);
  PA_CUDA(cudaMalloc(buf, sz));
  *have = sz;
  return PA_OK;
}

pa_status check_layer(const PagedAttnCache *c, uint32_t layer) {
  if (!c) return fail(PA_ERR_INVALID_ARG, "cache is null");
  if (layer >= c->cfg.num_layers) return fail(PA_ERR_INVALID_ARG, "layer_idx out of range");
  return PA_OK;
}

}  // namespace

extern "C" {

const char *pa_last_error_string(void) { return t_err.c_str(); }
int32_t pa_version(void) { return 100; }
uint64_t pa_kernel_launch_count(void) {
  return __atomic_load_n(&pa::g_launch_count, __ATOMIC_RELAXED);
}

pa_status pa_set_device(int32_t device) {
  int n = 0;
  PA_CUDA(cudaGetDeviceCount(&n));
  if (device < 0 || device >= n) return fail(PA_ERR_INVALID_ARG, "no such device");
  t_device = device;
  return PA_OK;
}
pa_status pa_set_stream(void *cuda_stream) {
  t_stream = static_cast<cudaStream_t>(cuda_stream);
  return PA_OK;
}

static pa_status cache_create_impl(const PagedAttnConfig *config, int32_t device, bool fp8,
                                   PagedAttnCache **out);
static pa_status cache_wrap_impl(const PagedAttnConfig *config, int32_t device, bool fp8,
                                 void *const *key_ptrs, void *const *value_ptrs,
                                 PagedAttnCache **out);

pa_status pa_cache_create(const PagedAttnConfig *config, int32_t device, PagedAttnCache **out) {
  return cache_create_impl(config, device, false, out);
}
pa_status pa_cache_create_fp8(const PagedAttnConfig *config, int32_t device, PagedAttnCache **out) {
  return cache_create_impl(config, device, true, out);
}
pa_status pa_cache_wrap(const PagedAttnConfig *config, int32_t device, void *const *key_ptrs,
                        void *const *value_ptrs, PagedAttnCache **out) {
  return cache_wrap_impl(config, device, false, key_ptrs, value_ptrs, out);
}
pa_status pa_cache_wrap_fp8(const PagedAttnConfig *config, int32_t device, void *const *key_ptrs,
                            void *const *value_ptrs, PagedAttnCache **out) {
  return cache_wrap_impl(config, device, true, key_ptrs, value_ptrs, out);
}
int32_t pa_cache_is_fp8(const PagedAttnCache *c) { return c && c->fp8 ? 1 : 0; }
pa_status pa_cache_set_kv_scales(PagedAttnCache *c, uint32_t layer, float k_scale, float v_scale) {
  pa_status st = check_layer(c, layer);
  if (st != PA_OK) return st;
  if (!c->fp8) return fail(PA_ERR_INVALID_ARG, "scales apply to an FP8 cache only");
  if (!(k_scale > 0.f) || !(v_scale > 0.f) || std::isinf(k_scale) || std::isinf(v_scale))
    return fail(PA_ERR_INVALID_ARG, "scales must be finite and > 0");
  c->k_scale[layer] = k_scale;
  c->v_scale[layer] = v_scale;
  return PA_OK;
}
pa_status pa_cache_fp8_set_exact_decode(PagedAttnCache *c, int32_t on) {
  if (!c) return fail(PA_ERR_INVALID_ARG, "cache is null");
  if (!c->fp8) return fail(PA_ERR_INVALID_ARG, "not an FP8 cache");
  DeviceGuard g(c->device);
  const unsigned word = on ? 1u : 0u;
  PA_CUDA(cudaMemcpy(c->fp8_special(), &word, sizeof(word), cudaMemcpyHostToDevice));
  return PA_OK;
}
pa_status pa_cache_get_kv_scales(const PagedAttnCache *c, uint32_t layer, float *k_scale,
                                 float *v_scale) {
  pa_status st = check_layer(c, layer);
  if (st != PA_OK) return st;
  if (!k_scale || !v_scale) return fail(PA_ERR_INVALID_ARG, "null argument");
  *k_scale = c->fp8 ? c->k_scale[layer] : 1.f;
  *v_scale = c->fp8 ? c->v_scale[layer] : 1.f;
  return PA_OK;
}

static pa_status cache_create_impl(const PagedAttnConfig *config, int32_t device, bool fp8,
                                   PagedAttnCache **out) {
  if (!out) return fail(PA_ERR_INVALID_ARG, "out_cache is null");
  *out = nullptr;
  pa_status st = validate_config(config);
  if (st != PA_OK) return st;
  if (fp8 && config->block_size == 8)  // crates/mlx-paged-attn/src/config.rs:71-76
    return fail(PA_ERR_INVALID_ARG, "FP8 cache requires block_size 16 or 32 for optimal alignment.");
  if (fp8 && config->head_size != (uint32_t)pa::kHeadSize)
    return fail(PA_ERR_UNSUPPORTED, "the FP8 cache is built for head size 128");
  DeviceGuard g(device);
  if (!g.ok) return fail(PA_ERR_CUDA, "cannot select device");
  PagedAttnCache *c = new (std::nothrow) PagedAttnCache();
  if (!c) return fail(PA_ERR_OOM, "host allocation failed");
  c->cfg = *config;
  c->device = device;
  c->owns = true;
  c->fp8 = fp8;
  c->k_scale.assign(config->num_layers, 1.f);
  c->v_scale.assign(config->num_layers, 1.f);
  const size_t bytes = layer_bytes(*config, fp8);
  for (uint32_t i = 0; i < config->num_layers; i++) {
    void *kp = nullptr, *vp = nullptr;
    cudaError_t e = cudaMalloc(&kp, bytes);
    if (e == cudaSuccess) e = cudaMalloc(&vp, bytes);
    // zero-filled, as the reference's create_cache (crates/mlx-sys/src/mlx.cpp:3847-3863)
    if (e == cudaSuccess) e = cudaMemset(kp, 0, bytes);
    if (e == cudaSuccess) e = cudaMemset(vp, 0, bytes);
    if (kp) c->k.push_back(kp);
    if (vp) c->v.push_back(vp);
    if (e != cudaSuccess) {
      cuda_fail(e, "pool allocation");
      cudaGetLastError();
      std::string keep = t_err;
      pa_cache_free(c);
      return fail(e == cudaErrorMemoryAllocation ? PA_ERR_OOM : PA_ERR_CUDA, keep);
    }
  }
  st = finish_create(c);
  if (st != PA_OK) {
    std::string keep = t_err;
    pa_cache_free(c);
    return fail(st, keep);
  }
  *out = c;
  return PA_OK;
}

static pa_status cache_wrap_impl(const PagedAttnConfig *config, int32_t device, bool fp8,
                                 void *const *key_ptrs, void *const *value_ptrs,
                                 PagedAttnCache **out) {
  if (!out) return fail(PA_ERR_INVALID_ARG, "out_cache is null");
  *out = nullptr;
  pa_status st = validate_config(config);
  if (st != PA_OK) return st;
  if (fp8 && config->block_size == 8)  // crates/mlx-paged-attn/src/config.rs:71-76
    return fail(PA_ERR_INVALID_ARG, "FP8 cache requires block_size 16 or 32 for optimal alignment.");
  if (fp8 && config->head_size != (uint32_t)pa::kHeadSize)
    return fail(PA_ERR_UNSUPPORTED, "the FP8 cache is built for head size 128");
  if (!key_ptrs || !value_ptrs) return fail(PA_ERR_INVALID_ARG, "pool pointer arrays are null");
  for (uint32_t i = 0; i < config->num_layers; i++) {
    if (!key_ptrs[i] || !value_ptrs[i]) return fail(PA_ERR_INVALID_ARG, "a pool pointer is null");
    if ((reinterpret_cast<uintptr_t>(key_ptrs[i]) | reinterpret_cast<uintptr_t>(value_ptrs[i])) & 127u)
      return fail(PA_ERR_INVALID_ARG, "pool pointers must be 128-byte aligned");
  }
  DeviceGuard g(device);
  if (!g.ok) return fail(PA_ERR_CUDA, "cannot select device");
  PagedAttnCache *c = new (std::nothrow) PagedAttnCache();
  if (!c) return fail(PA_ERR_OOM, "host allocation failed");
  c->cfg = *config;
  c->device = device;
  c->owns = false;
  c->fp8 = fp8;
  c->k_scale.assign(config->num_layers, 1.f);
  c->v_scale.assign(config->num_layers, 1.f);
  c->k.assign(key_ptrs, key_ptrs + config->num_layers);
  c->v.assign(value_ptrs, value_ptrs + config->num_layers);
  st = finish_create(c);
  if (st == PA_OK && fp8) st = pa_cache_fp8_set_exact_decode(c, 1);  // contents unknown
  if (st != PA_OK) {
    std::string keep = t_err;
    pa_cache_free(c);
    return fail(st, keep);
  }
  *out = c;
  return PA_OK;
}

pa_status pa_cache_free(PagedAttnCache *c) {
  if (!c) return PA_OK;
  DeviceGuard g(c->device);
  if (c->owns) {
    for (void *p : c->k) cudaFree(p);
    for (void *p : c->v) cudaFree(p);
  }
  if (c->err_dev) cudaFree(c->err_dev);
  if (c->sync_dev) cudaFree(c->sync_dev);
  if (c->err_host) cudaFreeHost(c->err_host);
  if (c->ws) cudaFree(c->ws);
  if (c->meta) cudaFree(c->meta);
  if (c->stage) cudaFree(c->stage);
  if (c->step_stream) cudaStreamDestroy(c->step_stream);
  if (c->aux_stream) cudaStreamDestroy(c->aux_stream);
  if (c->ev_fork) cudaEventDestroy(c->ev_fork);
  if (c->ev_join) cudaEventDestroy(c->ev_join);
  for (int i = 0; i < 2; i++) {
    if (c->lane_stream[i]) cudaStreamDestroy(c->lane_stream[i]);
    if (c->ev_lane[i]) cudaEventDestroy(c->ev_lane[i]);
  }
  delete c;
  return PA_OK;
}

void *pa_cache_key_ptr(PagedAttnCache *c, uint32_t layer) {
  return check_layer(c, layer) == PA_OK ? c->k[layer] : nullptr;
}
void *pa_cache_value_ptr(PagedAttnCache *c, uint32_t layer) {
  return check_layer(c, layer) == PA_OK ? c->v[layer] : nullptr;
}
pa_status pa_cache_get_config(const PagedAttnCache *c, PagedAttnConfig *out) {
  if (!c || !out) return fail(PA_ERR_INVALID_ARG, "null argument");
  *out = c->cfg;
  return PA_OK;
}

pa_status pa_cache_check_errors(PagedAttnCache *c, void *cuda_stream) {
  if (!c) return fail(PA_ERR_INVALID_ARG, "cache is null");
  DeviceGuard g(c->device);
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  unsigned word = 0;
  PA_CUDA(cudaMemcpyAsync(&word, c->err_dev, sizeof(word), cudaMemcpyDeviceToHost, st));
  PA_CUDA(cudaStreamSynchronize(st));
  if (word == 0) return PA_OK;
  PA_CUDA(cudaMemsetAsync(c->err_dev, 0, sizeof(word), st));
  // a kernel that gave up may have left arrival counters behind
  if (word & pa::kErrTimeout)
    PA_CUDA(cudaMemsetAsync(c->sync_dev, 0, pa::kSyncWords * sizeof(unsigned), st));
  PA_CUDA(cudaStreamSynchronize(st));
  *c->err_host = 0;
  if (word & pa::kErrTimeout) return fail(PA_ERR_TIMEOUT, "a bounded device-side wait ran out");
  if (word & pa::kErrStepSlot)
    return fail(PA_ERR_INVALID_ARG,
                "decode step: a slot_mapping entry is not position context_len - 1 of its sequence "
                "(that token was not written)");
  if (word & pa::kErrSlotRange)
    return fail(PA_ERR_OUT_OF_RANGE, "slot_mapping entry beyond num_blocks*block_size (skipped)");
  return fail(PA_ERR_OUT_OF_RANGE, "block id beyond num_blocks (read as block 0)");
}

pa_status pa_reshape_and_cache(PagedAttnCache *c, uint32_t layer, const void *key,
                               const void *value, const int64_t *slot_mapping, int64_t num_tokens,
                               int64_t key_stride, int64_t value_stride, void *cuda_stream) {
  pa_status st = check_layer(c, layer);
  if (st != PA_OK) return st;
  if (num_tokens < 0) return fail(PA_ERR_INVALID_ARG, "num_tokens < 0");
  if (num_tokens == 0) return PA_OK;
  if (!key || !value || !slot_mapping) return fail(PA_ERR_INVALID_ARG, "null tensor pointer");
  const int64_t row = (int64_t)c->cfg.num_kv_heads * c->cfg.head_size;
  if (key_stride < row || value_stride < row || (key_stride & 7) || (value_stride & 7))
    return fail(PA_ERR_INVALID_ARG, "key/value stride must be >= num_kv_heads*head_size and a multiple of 8");
  if (!aligned16(key) || !aligned16(value))
    return fail(PA_ERR_INVALID_ARG, "key/value must be 16-byte aligned");
  if (num_tokens > ((int64_t)1 << 34)) return fail(PA_ERR_INVALID_ARG, "num_tokens too large");
  DeviceGuard g(c->device);
  if (c->fp8) {
    PA_CUDA(pa::launch_reshape_and_cache_fp8(
        static_cast<const pa::elem16 *>(key), static_cast<const pa::elem16 *>(value),
        static_cast<uint8_t *>(c->k[layer]), static_cast<uint8_t *>(c->v[layer]), slot_mapping,
        num_tokens, key_stride, value_stride, (int)c->cfg.num_kv_heads, c->cfg.num_blocks,
        c->bs_shift, c->k_scale[layer], c->v_scale[layer], c->cfg.dtype == 0, c->err_dev, c->fp8_special(),
        static_cast<cudaStream_t>(cuda_stream)));
    return PA_OK;
  }
  PA_CUDA(pa::launch_reshape_and_cache(
      static_cast<const pa::elem16 *>(key), static_cast<const pa::elem16 *>(value),
      static_cast<pa::elem16 *>(c->k[layer]), static_cast<pa::elem16 *>(c->v[layer]),
      slot_mapping, num_tokens, key_stride, value_stride, (int)c->cfg.num_kv_heads,
      c->cfg.num_blocks, c->bs_shift, c->err_dev, static_cast<cudaStream_t>(cuda_stream),
      (int)c->cfg.head_size));
  return PA_OK;
}

pa_status pa_qk_norm_rope_and_cache(PagedAttnCache *c, uint32_t layer, void *q_out, const void *q,
                                    const void *k, const void *v, const void *q_norm_weight,
                                    const void *k_norm_weight, float eps,
                                    const int32_t *positions, float rope_base,
                                    uint32_t rope_dims, const int64_t *slot_mapping,
                                    int64_t num_tokens, int32_t num_q_heads, int64_t q_stride,
                                    int64_t q_out_stride, int64_t k_stride, int64_t v_stride,
                                    void *cuda_stream) {
  pa_status st = check_layer(c, layer);
  if (st != PA_OK) return st;
  if (num_tokens < 0) return fail(PA_ERR_INVALID_ARG, "num_tokens < 0");
  if (num_tokens == 0) return PA_OK;
  if (!q_out || !q || !k || !v || !positions || !slot_mapping)
    return fail(PA_ERR_INVALID_ARG, "null tensor pointer");
  const int Hkv = (int)c->cfg.num_kv_heads, D = (int)c->cfg.head_size;
  if (D != pa::kHeadSize)
    return fail(PA_ERR_UNSUPPORTED, "the fused norm + rotary + write launch is built for head size 128");
  if (num_q_heads <= 0 || num_q_heads % Hkv)
    return fail(PA_ERR_INVALID_ARG, "num_q_heads must be a positive multiple of num_kv_heads");
  if (rope_dims > (uint32_t)D || (rope_dims & 1))
    return fail(PA_ERR_INVALID_ARG, "rope_dims must be even and <= head_size");
  if (!(rope_base > 0.f) || !(eps >= 0.f)) return fail(PA_ERR_INVALID_ARG, "bad rope_base or eps");
  const int64_t q_row = (int64_t)num_q_heads * D, kv_row = (int64_t)Hkv * D;
  if (q_stride < q_row || q_out_stride < q_row || k_stride < kv_row || v_stride < kv_row ||
      ((q_stride | q_out_stride | k_stride | v_stride) & 7))
    return fail(PA_ERR_INVALID_ARG, "row strides must cover a row and be multiples of 8");
  if (!aligned16(q) || !aligned16(q_out) || !aligned16(k) || !aligned16(v) ||
      (q_norm_weight && !aligned16(q_norm_weight)) || (k_norm_weight && !aligned16(k_norm_weight)))
    return fail(PA_ERR_INVALID_ARG, "tensors must be 16-byte aligned");
  if (num_tokens > ((int64_t)1 << 34)) return fail(PA_ERR_INVALID_ARG, "num_tokens too large");
  if (c->fp8)
    return fail(PA_ERR_UNSUPPORTED, "the fused producer writes 16-bit pools; with an FP8 cache "
                                    "rotate into a buffer and call pa_reshape_and_cache");
  pa::ProducerParams p{};
  p.q_in = static_cast<const pa::elem16 *>(q);
  p.q_out = static_cast<pa::elem16 *>(q_out);
  p.k = static_cast<const pa::elem16 *>(k);
  p.v = static_cast<const pa::elem16 *>(v);
  p.q_norm_w = static_cast<const pa::elem16 *>(q_norm_weight);
  p.k_norm_w = static_cast<const pa::elem16 *>(k_norm_weight);
  p.positions = positions;
  p.slot_mapping = slot_mapping;
  p.k_pool = static_cast<pa::elem16 *>(c->k[layer]);
  p.v_pool = static_cast<pa::elem16 *>(c->v[layer]);
  p.num_tokens = num_tokens;
  p.q_stride = q_stride;
  p.q_out_stride = q_out_stride;
  p.k_stride = k_stride;
  p.v_stride = v_stride;
  p.Hq = num_q_heads;
  p.Hkv = Hkv;
  p.rope_dims = (int)rope_dims;
  p.num_blocks = c->cfg.num_blocks;
  p.bs_shift = c->bs_shift;
  p.eps = eps;
  p.err = c->err_dev;
  const int half = (int)rope_dims / 2;
  for (int i = 0; i < half; i++)
    p.inv_freq[i] = (float)std::pow((double)rope_base, -(double)i / (double)half);
  DeviceGuard g(c->device);
  PA_CUDA(pa::launch_qk_norm_rope_cache(p, c->cfg.dtype == 0, c->num_sms,
                                        static_cast<cudaStream_t>(cuda_stream)));
  return PA_OK;
}

pa_status pa_copy_blocks(PagedAttnCache *c, uint32_t layer, const int64_t *mapping,
                         int64_t num_pairs, void *cuda_stream) {
  pa_status st = check_layer(c, layer);
  if (st != PA_OK) return st;
  if (num_pairs < 0) return fail(PA_ERR_INVALID_ARG, "num_pairs < 0");
  if (num_pairs == 0) return PA_OK;
  if (!mapping) return fail(PA_ERR_INVALID_ARG, "block_mapping is null");
  DeviceGuard g(c->device);
  const int64_t bpb = block_bytes_of(c);
  PA_CUDA(pa::launch_copy_blocks(static_cast<pa::elem16 *>(c->k[layer]),
                                 static_cast<pa::elem16 *>(c->v[layer]), mapping, num_pairs, bpb,
                                 c->cfg.num_blocks, c->err_dev,
                                 static_cast<cudaStream_t>(cuda_stream)));
  return PA_OK;
}

pa_status pa_gather_heads_peer_store(PagedAttnCache *c, const void *local_out, int64_t num_tokens,
                                     int32_t heads_local, int32_t world, int32_t rank,
                                     void *const *peer_out, uint32_t *const *peer_flags,
                                     uint32_t epoch, int32_t wait, void *cuda_stream) {
  if (!c) return fail(PA_ERR_INVALID_ARG, "cache is null");
  if (world < 1 || world > pa::kMaxPeers || rank < 0 || rank >= world)
    return fail(PA_ERR_INVALID_ARG, "world must be 1..8 and 0 <= rank < world");
  if (num_tokens < 0 || heads_local <= 0) return fail(PA_ERR_INVALID_ARG, "bad sizes");
  // an empty step moves no rows, so its data pointers may be null; the flags are still published
  const bool empty = num_tokens == 0;
  if ((!local_out && !empty) || !peer_out || !peer_flags) return fail(PA_ERR_INVALID_ARG, "null pointer");
  pa::PeerGather a{};
  a.local_out = local_out;
  for (int w = 0; w < world; w++) {
    if ((!peer_out[w] && !empty) || !peer_flags[w] || !aligned16(peer_out[w]))
      return fail(PA_ERR_INVALID_ARG, "peer buffers must be non-null and 16-byte aligned");
    a.peer_out[w] = peer_out[w];
    a.peer_flags[w] = peer_flags[w];
  }
  if (!aligned16(local_out)) return fail(PA_ERR_INVALID_ARG, "local_out must be 16-byte aligned");
  a.counter = c->err_dev + 32;  // a zeroed word of the handle, next to the error word
  a.num_tokens = num_tokens;
  a.row_bytes_local = heads_local * (int32_t)c->cfg.head_size * 2;
  a.world = world;
  a.rank = rank;
  a.epoch = epoch;
  DeviceGuard g(c->device);
  PA_CUDA(pa::launch_peer_gather(a, static_cast<cudaStream_t>(cuda_stream)));
  if (wait)
    PA_CUDA(pa::launch_peer_wait(peer_flags[rank], world, epoch, c->err_dev,
                                 static_cast<cudaStream_t>(cuda_stream)));
  return PA_OK;
}

pa_status pa_gather_heads_wait(PagedAttnCache *c, const uint32_t *my_flags, int32_t world,
                               uint32_t epoch, void *cuda_stream) {
  if (!c) return fail(PA_ERR_INVALID_ARG, "cache is null");
  if (!my_flags || world < 1 || world > pa::kMaxPeers)
    return fail(PA_ERR_INVALID_ARG, "flags null or world not in 1..8");
  DeviceGuard g(c->device);
  PA_CUDA(pa::launch_peer_wait(my_flags, world, epoch, c->err_dev,
                               static_cast<cudaStream_t>(cuda_stream)));
  return PA_OK;
}

/* ---- swap ------------------------------------------------------------------------ */
}  // extern "C"

// Host copies of swapped blocks: slabs of pinned, device-mapped memory cut into
// (K, V) slots; a free list; and a pinned argument area the swap kernel reads.
struct PaCpuBlockCache {
  int device = 0;
  size_t block_bytes = 0;  // bytes of one block's K (== V) for one layer
  static constexpr int kSlotsPerSlab = 64;
  static constexpr int kMaxPerLaunch = 4096;
  std::vector<char *> slabs;
  std::vector<char *> free_slots;                    // each slot = K bytes then V bytes
  // (layer, block id) -> slot: one host cache serves every layer of a model, a block id
  // being the same block in each layer's pool
  std::unordered_map<uint64_t, char *> swapped;
  std::unordered_map<uint32_t, uint32_t> layers_of;  // block id -> layers that hold a host copy
  static uint64_t key(uint32_t layer, uint32_t id) { return ((uint64_t)layer << 32) | id; }
  char *args = nullptr;                              // pinned: ids | host_k ptrs | host_v ptrs
};

namespace {
pa_status cpu_slot(PaCpuBlockCache *cpu, char **slot) {
  if (cpu->free_slots.empty()) {
    char *slab = nullptr;
    PA_CUDA(cudaHostAlloc(reinterpret_cast<void **>(&slab),
                          2 * cpu->block_bytes * PaCpuBlockCache::kSlotsPerSlab,
                          cudaHostAllocMapped | cudaHostAllocPortable));
    cpu->slabs.push_back(slab);
    for (int i = PaCpuBlockCache::kSlotsPerSlab - 1; i >= 0; i--)
      cpu->free_slots.push_back(slab + (size_t)i * 2 * cpu->block_bytes);
  }
  *slot = cpu->free_slots.back();
  cpu->free_slots.pop_back();
  return PA_OK;
}
}  // namespace

extern "C" {

PaCpuBlockCache *pa_cpu_cache_create(const PagedAttnCache *c) {
  if (!c) {
    fail(PA_ERR_INVALID_ARG, "cache is null");
    return nullptr;
  }
  PaCpuBlockCache *cpu = new (std::nothrow) PaCpuBlockCache();
  if (!cpu) return nullptr;
  cpu->device = c->device;
  cpu->block_bytes = (size_t)block_bytes_of(c);
  return cpu;
}
void pa_cpu_cache_free(PaCpuBlockCache *cpu) {
  if (!cpu) return;
  DeviceGuard g(cpu->device);
  for (char *s : cpu->slabs) cudaFreeHost(s);
  if (cpu->args) cudaFreeHost(cpu->args);
  delete cpu;
}
int32_t pa_cpu_cache_is_swapped(const PaCpuBlockCache *cpu, uint32_t id) {
  return cpu && cpu->layers_of.count(id) != 0;
}
int32_t pa_cpu_cache_is_swapped_layer(const PaCpuBlockCache *cpu, uint32_t layer, uint32_t id) {
  return cpu && cpu->swapped.count(PaCpuBlockCache::key(layer, id)) != 0;
}
size_t pa_cpu_cache_num_swapped(const PaCpuBlockCache *cpu) { return cpu ? cpu->layers_of.size() : 0; }
pa_status pa_cpu_cache_block_ptrs(const PaCpuBlockCache *cpu, uint32_t layer, uint32_t id, void **key,
                                  void **value) {
  if (!cpu || !key || !value) return fail(PA_ERR_INVALID_ARG, "null argument");
  auto it = cpu->swapped.find(PaCpuBlockCache::key(layer, id));
  if (it == cpu->swapped.end())
    return fail(PA_ERR_INVALID_ARG, "Block " + std::to_string(id) + " not found in CPU cache");
  *key = it->second;
  *value = it->second + cpu->block_bytes;
  return PA_OK;
}
void pa_swap_block_bytes(uint32_t num_kv_heads, uint32_t head_size, uint32_t block_size, int32_t use_fp8,
                         uint64_t *key_bytes, uint64_t *value_bytes) {
  const uint64_t n = (uint64_t)num_kv_heads * head_size * block_size * (use_fp8 ? 1 : 2);
  if (key_bytes) *key_bytes = n;
  if (value_bytes) *value_bytes = n;
}

static pa_status swap_impl(PagedAttnCache *c, uint32_t layer, const uint32_t *ids, size_t n,
                           PaCpuBlockCache *cpu, void *cuda_stream, bool to_host) {
  pa_status st = check_layer(c, layer);
  if (st != PA_OK) return st;
  if (!cpu) return fail(PA_ERR_INVALID_ARG, "cpu cache is null");
  if (n == 0) return PA_OK;
  if (!ids) return fail(PA_ERR_INVALID_ARG, "block_ids is null");
  if (cpu->device != c->device ||
      cpu->block_bytes != (size_t)block_bytes_of(c))
    return fail(PA_ERR_INVALID_ARG, "cpu cache was created for a different cache geometry");
  DeviceGuard g(c->device);
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  constexpr int kMax = PaCpuBlockCache::kMaxPerLaunch;
  if (!cpu->args)
    PA_CUDA(cudaHostAlloc(reinterpret_cast<void **>(&cpu->args), (size_t)kMax * (4 + 8 + 8),
                          cudaHostAllocMapped | cudaHostAllocPortable));
  uint32_t *a_ids = reinterpret_cast<uint32_t *>(cpu->args);
  char **a_k = reinterpret_cast<char **>(cpu->args + (size_t)kMax * 4);
  char **a_v = a_k + kMax;
  if (!to_host)  // every block must have a host copy before anything moves
    for (size_t i = 0; i < n; i++)
      if (!cpu->swapped.count(PaCpuBlockCache::key(layer, ids[i])))
        return fail(PA_ERR_INVALID_ARG, "Block " + std::to_string(ids[i]) + " not found in CPU cache");
  for (size_t base = 0; base < n; base += kMax) {
    int m = 0;
    for (size_t i = base; i < n && i < base + kMax; i++) {
      const uint32_t id = ids[i];
      if (id >= c->cfg.num_blocks) return fail(PA_ERR_OUT_OF_RANGE, "block id beyond num_blocks");
      char *slot = nullptr;
      if (to_host) {
        if (cpu->swapped.count(PaCpuBlockCache::key(layer, id))) continue;  // already swapped out
        st = cpu_slot(cpu, &slot);
        if (st != PA_OK) return st;
        cpu->swapped[PaCpuBlockCache::key(layer, id)] = slot;
        cpu->layers_of[id]++;
      } else {
        slot = cpu->swapped[PaCpuBlockCache::key(layer, id)];
      }
      a_ids[m] = id;
      a_k[m] = slot;
      a_v[m] = slot + cpu->block_bytes;
      m++;
    }
    PA_CUDA(pa::launch_swap_blocks(static_cast<pa::elem16 *>(c->k[layer]),
                                   static_cast<pa::elem16 *>(c->v[layer]), a_ids, a_k, a_v, m,
                                   (int64_t)cpu->block_bytes, to_host ? 1 : 0, c->cfg.num_blocks,
                                   c->err_dev, stream));
    PA_CUDA(cudaStreamSynchronize(stream));  // the argument area is reused; the reference blocks too
  }
  if (!to_host)
    for (size_t i = 0; i < n; i++) {
      auto it = cpu->swapped.find(PaCpuBlockCache::key(layer, ids[i]));
      if (it != cpu->swapped.end()) {
        cpu->free_slots.push_back(it->second);
        cpu->swapped.erase(it);
        auto l = cpu->layers_of.find(ids[i]);
        if (l != cpu->layers_of.end() && --l->second == 0) cpu->layers_of.erase(l);
      }
    }
  return PA_OK;
}
pa_status pa_swap_out(PagedAttnCache *c, uint32_t layer, const uint32_t *ids, size_t n,
                      PaCpuBlockCache *cpu, void *stream) {
  return swap_impl(c, layer, ids, n, cpu, stream, true);
}
pa_status pa_swap_in(PagedAttnCache *c, uint32_t layer, const uint32_t *ids, size_t n,
                     PaCpuBlockCache *cpu, void *stream) {
  return swap_impl(c, layer, ids, n, cpu, stream, false);
}

size_t pa_attention_workspace_bytes(const PagedAttnCache *c) {
  if (!c) return 0;
  // an FP8 cache and one with small heads may run the narrow kernel with two CTAs per SM
  return pa::splitkv_workspace_bytes(c->num_sms * pa::splitkv_narrow_ctas_per_sm((int)c->cfg.head_size, c->fp8));
}

}  // extern "C"

namespace {
// The step's new tokens for a decode call that also writes them (see AttnParams::k_new).
struct StepWrite {
  const void *k, *v;
  const int64_t *slots;
  int64_t k_stride, v_stride;
};
// Whether the split-KV kernel can write the step's tokens itself: 16-bit pools of
// 16-token blocks and a GQA group that fits the narrow kernel.
// The fused write sits on the critical path of the CTA that ends a (sequence, kv head) item:
// measured on B200 about 3 us per item and CTA, against about 4 us for a write launch of
// its own.  It pays while a CTA ends at most a couple of items (few kv heads per GPU, as
// under kv-head sharding); beyond that the step runs the write kernel first.
bool can_fuse_write(const PagedAttnCache *c, int num_q_heads, int num_seqs) {
  return !c->fp8 && c->bs_shift == 0 && c->cfg.head_size == (uint32_t)pa::kHeadSize && num_q_heads > 0 &&
         num_q_heads % (int)c->cfg.num_kv_heads == 0 && num_q_heads / (int)c->cfg.num_kv_heads <= 8 &&
         (int64_t)num_seqs * c->cfg.num_kv_heads <= 2 * (int64_t)c->num_sms;
}

cudaError_t launch_tiles(PagedAttnCache *c, uint32_t layer, const pa::AttnParams &p,
                         const pa::TileWork *work_dev, int n, cudaStream_t st) {
  if (c->has_tile64())
    return pa::launch_tile64_attention(p, work_dev, n, &c->k_maps[layer], &c->v_maps[layer], st);
  return pa::launch_tile_attention(p, work_dev, n, &c->v_maps[layer], st);
}

pa_status attention_impl(PagedAttnCache *c, uint32_t layer, void *out, const void *q,
                         const int32_t *block_tables, const int32_t *context_lens,
                         const int32_t *cu_q_lens_host, const int32_t *context_lens_host,
                         int32_t num_seqs, int32_t num_q_heads, int32_t max_blocks_per_seq,
                         int64_t q_stride, int64_t out_stride, float scale, float softcap,
                         void *workspace, size_t workspace_bytes, void *cuda_stream,
                         const StepWrite *write, const int32_t *seq_rows = nullptr) {
  pa_status st = check_layer(c, layer);
  if (st != PA_OK) return st;
  if (num_seqs < 0) return fail(PA_ERR_INVALID_ARG, "num_seqs < 0");
  if (num_seqs == 0) return PA_OK;
  if (!out || !q || !block_tables || !context_lens)
    return fail(PA_ERR_INVALID_ARG, "null tensor pointer");
  const int Hkv = (int)c->cfg.num_kv_heads;
  if (num_q_heads <= 0 || num_q_heads % Hkv != 0)
    return fail(PA_ERR_INVALID_ARG, "num_q_heads must be a positive multiple of num_kv_heads");
  const int G = num_q_heads / Hkv;
  // any group size whose columns fit the widest split-KV kernel: 24 (16 with head size 192, 8
  // with 256); rows and columns are (query token, head of the group) pairs by plain division
  if (G > pa::splitkv_max_cols_for((int)c->cfg.head_size))
    return fail(PA_ERR_UNSUPPORTED, "more query heads per kv head than the kernels take: 24 (16 with head size "
                                    "192, 8 with head size 256)");
  if (max_blocks_per_seq <= 0) return fail(PA_ERR_INVALID_ARG, "max_blocks_per_seq must be > 0");
  const int64_t row = (int64_t)num_q_heads * c->cfg.head_size;
  if (q_stride < row || out_stride < row || (q_stride & 7) || (out_stride & 7))
    return fail(PA_ERR_INVALID_ARG, "q/out stride must be >= num_q_heads*head_size and a multiple of 8");
  if (!aligned16(q) || !aligned16(out)) return fail(PA_ERR_INVALID_ARG, "q/out must be 16-byte aligned");
  if (!workspace || workspace_bytes < pa::splitkv_workspace_bytes(c->num_sms) ||
      (reinterpret_cast<uintptr_t>(workspace) & 255u))
    return fail(PA_ERR_INVALID_ARG, "workspace missing, too small or not 256-byte aligned");
  if (!(scale > 0.f) || !(softcap > 0.f)) return fail(PA_ERR_INVALID_ARG, "scale and softcap must be > 0");

  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  DeviceGuard g(c->device);
  pa::AttnParams p{};
  p.q = static_cast<const pa::elem16 *>(q);
  p.out = static_cast<pa::elem16 *>(out);
  p.k_pool = static_cast<const pa::elem16 *>(c->k[layer]);
  p.v_pool = static_cast<const pa::elem16 *>(c->v[layer]);
  p.block_tables = block_tables;
  p.context_lens = context_lens;
  p.cu_q_lens = nullptr;
  p.S = num_seqs;
  p.Hq = num_q_heads;
  p.Hkv = Hkv;
  p.G = G;
  p.MB = max_blocks_per_seq;
  p.head_size = (int)c->cfg.head_size;
  p.bs_shift = c->bs_shift;
  p.num_blocks = c->cfg.num_blocks;
  p.q_stride = q_stride;
  p.out_stride = out_stride;
  p.scale = scale;
  p.softcap = softcap;
  p.ws = static_cast<float *>(workspace);
  p.ws_ctas = (int)std::min<size_t>(workspace_bytes / pa::splitkv_workspace_bytes(1), 1u << 20);
  p.err = c->err_dev;
  p.err_mirror = c->err_host_dev;
  p.sync = c->sync_dev;
  p.seq_base = 0;
  p.is_f16 = c->cfg.dtype == 0 ? 1 : 0;
  p.is_fp8 = c->fp8 ? 1 : 0;
  p.k_scale = c->fp8 ? c->k_scale[layer] : 1.f;
  p.v_scale = c->fp8 ? c->v_scale[layer] : 1.f;
  p.fp8_special = c->fp8_special();
  p.early_trigger = 1;

  if (!cu_q_lens_host) {  // decode: one query per sequence
    p.min_cols = 1;
    p.max_cols = G;
    p.seq_row = seq_rows;
    if (write) {
      p.k_new = static_cast<const pa::elem16 *>(write->k);
      p.v_new = static_cast<const pa::elem16 *>(write->v);
      p.slot_mapping = write->slots;
      p.k_new_stride = write->k_stride;
      p.v_new_stride = write->v_stride;
    }
    PA_CUDA(pa::launch_splitkv_attention(p, c->num_sms, stream, c->unit_map(layer)));
    return PA_OK;
  }

  // Classify sequences by their number of columns (queries x heads of a group):
  // up to 24 columns -> split-KV kernel, one launch per 8-column width class so that
  // plain decode sequences run in the narrow, deepest-pipelined variant even when the
  // batch also holds multi-token (verify) sequences; more -> tile kernel.
  const int split_cols = pa::splitkv_max_cols_for((int)c->cfg.head_size);
  const int tile_q = pa::tile_queries_per_cta(G);
  bool have_class[3] = {false, false, false};
  std::vector<pa::TileWork> tiles;
  double tile_flops = 0.0, split_bytes = 0.0;  // work estimates, only with host context lengths
  double class_bytes[3] = {0.0, 0.0, 0.0};
  // a chunk too long for the split-KV kernel on a cache the tile kernel does not read
  // (8-token blocks)
  bool in_pieces = false;
  for (int s = 0; s < num_seqs; s++) {
    const int ql = cu_q_lens_host[s + 1] - cu_q_lens_host[s];
    if (ql < 0) return fail(PA_ERR_INVALID_ARG, "cu_q_lens must be non-decreasing");
    if (ql == 0) continue;
    const double kv = context_lens_host ? (double)context_lens_host[s] : 0.0;
    if (ql * G <= split_cols) {
      have_class[(ql * G - 1) / 8] = true;
      split_bytes += kv * 2.0 * Hkv * c->cfg.head_size * (c->fp8 ? 1.0 : 2.0);
      class_bytes[(ql * G - 1) / 8] += kv * 2.0 * Hkv * c->cfg.head_size * (c->fp8 ? 1.0 : 2.0);
    } else {
      if (!c->has_tile_kernel()) {  // served below as several shorter sequences
        in_pieces = true;
        continue;
      }
      // Tiles of one (sequence, kv head) are neighbours in launch order so that they
      // share the head's KV blocks in L2; later tiles see more keys and go first.
      for (int h = 0; h < Hkv; h++)
        for (int qb = ((ql - 1) / tile_q) * tile_q; qb >= 0; qb -= tile_q)
          tiles.push_back(pa::TileWork{s, h, qb, ql - qb < tile_q ? ql - qb : tile_q});
      tile_flops += 4.0 * c->cfg.head_size * num_q_heads * ql * (kv - 0.5 * ql);
    }
  }
  // The tile kernel reads 16- or 32-token blocks only.  With 8-token blocks a longer chunk
  // is handed to the split-KV kernel as consecutive pieces of at most 24/G query tokens, each a
  // sequence of its own with the same block-table row and the context length that ends
  // at its last query: the same results (the KV of the chunk's sequence is read once per
  // piece, from L2 mostly), at the price of that re-reading.
  std::vector<int32_t> v_cu, v_ctx, v_row;
  if (in_pieces) {
    if (!context_lens_host)
      return fail(PA_ERR_INVALID_ARG,
                  "with 8-token blocks or a head size other than 128, chunks of more than " +
                      std::to_string(split_cols / G) + " query tokens need context_lens_host");
    const int piece = split_cols / G;
    v_cu.push_back(0);
    have_class[0] = have_class[1] = have_class[2] = false;
    split_bytes = 0.0;
    class_bytes[0] = class_bytes[1] = class_bytes[2] = 0.0;
    for (int s = 0; s < num_seqs; s++) {
      const int ql = cu_q_lens_host[s + 1] - cu_q_lens_host[s];
      const int kv_len = context_lens_host[s];
      for (int qa = 0; qa < ql || qa == 0; qa += piece) {
        const int qb = std::min(ql, qa + piece);
        v_cu.push_back(v_cu.back() + (qb - qa));
        v_ctx.push_back(ql ? kv_len - ql + qb : kv_len);
        v_row.push_back(s);
        if (qb > qa) {
          have_class[((qb - qa) * G - 1) / 8] = true;
          split_bytes += (double)v_ctx.back() * 2.0 * Hkv * c->cfg.head_size * (c->fp8 ? 1.0 : 2.0);
          class_bytes[((qb - qa) * G - 1) / 8] += (double)v_ctx.back() * 2.0 * Hkv * c->cfg.head_size * (c->fp8 ? 1.0 : 2.0);
        }
        if (ql == 0) break;
      }
    }
  }
  const int num_items = in_pieces ? (int)v_row.size() : num_seqs;
  const bool any_split = have_class[0] || have_class[1] || have_class[2];
  const size_t cu_bytes = ((size_t)(num_items + 1) * 4 + 255) & ~(size_t)255;
  const size_t vx_bytes = in_pieces ? (((size_t)num_items * 4 + 255) & ~(size_t)255) : 0;
  const size_t need = cu_bytes + 2 * vx_bytes + tiles.size() * sizeof(pa::TileWork);
  st = grow(&c->meta, &c->meta_bytes, need);
  if (st != PA_OK) return st;
  char *meta = static_cast<char *>(c->meta);
  PA_CUDA(cudaMemcpyAsync(meta, in_pieces ? v_cu.data() : cu_q_lens_host, (size_t)(num_items + 1) * 4,
                          cudaMemcpyHostToDevice, stream));
  p.cu_q_lens = reinterpret_cast<const int32_t *>(meta);
  if (in_pieces) {
    PA_CUDA(cudaMemcpyAsync(meta + cu_bytes, v_ctx.data(), (size_t)num_items * 4,
                            cudaMemcpyHostToDevice, stream));
    PA_CUDA(cudaMemcpyAsync(meta + cu_bytes + vx_bytes, v_row.data(), (size_t)num_items * 4,
                            cudaMemcpyHostToDevice, stream));
    p.context_lens = reinterpret_cast<const int32_t *>(meta + cu_bytes);
    p.seq_row = reinterpret_cast<const int32_t *>(meta + cu_bytes + vx_bytes);
    p.S = num_items;
  }
  pa::TileWork *work_dev = reinterpret_cast<pa::TileWork *>(meta + cu_bytes + 2 * vx_bytes);
  if (!tiles.empty())
    PA_CUDA(cudaMemcpyAsync(work_dev, tiles.data(), tiles.size() * sizeof(pa::TileWork),
                            cudaMemcpyHostToDevice, stream));

  // A batch that holds several kinds of work runs them side by side, each kernel on a
  // share of the SMs and on a stream of its own: the tensor-bound tile kernel and one
  // memory-bound split-KV launch per width class present (each launch "lane" keeps its
  // partial slots and counters apart from the others').  Run one after the other, every
  // kernel would pay its start-up and tail on the whole GPU and a few verify sequences
  // would hold 148 SMs for tens of microseconds.  The shares come from a small model
  // measured on B200: the narrow split-KV kernel streams about 70 GB/s per SM up to about
  // 6 TB/s in total (100 SMs already saturate HBM); the wider ones (two and three column
  // tiles: more tensor work per unit, a two-stage ring) a half and two fifths of that per
  // SM; a tile CTA sustains about 1.1 PFLOP/s / 148 (0.9 with 32-token blocks) and tile
  // CTAs run in waves over the SMs they get.  Without host context lengths there is no
  // estimate and the kernels run back to back.
  int n_classes = 0;
  for (int k = 0; k < 3; k++) n_classes += have_class[k] ? 1 : 0;
  const double class_weight[3] = {1.0, 2.0, 2.5};
  double eff_bytes = 0.0;  // bytes in units of the narrow kernel's per-SM rate
  for (int k = 0; k < 3; k++) eff_bytes += class_bytes[k] * class_weight[k];
  // (FP8 cache: the tile kernel converts bytes as it goes and sustains about 0.6 PFLOP/s;
  // the split-KV kernel streams about 30 GB/s per SM, 4.4 TB/s on the whole GPU)
  const double tile_rate = c->fp8 ? 0.6e15 : (c->has_tile64() ? 1.1e15 : 0.9e15);
  const double sm_bw = c->fp8 ? 30e9 : 70e9, bw_cap = c->fp8 ? 4.4e12 : 6.0e12;
  int tile_sms = 0;
  bool concurrent = false;
  if (context_lens_host && any_split && eff_bytes / bw_cap > 20e-6) {
    if (!tiles.empty()) {
      const double t_cta = tile_flops / (double)tiles.size() / (tile_rate / c->num_sms);
      const double t_tile_alone = t_cta * (double)((tiles.size() + c->num_sms - 1) / c->num_sms);
      if (t_tile_alone > 20e-6) {
        double best = 1e30;
        for (int n2 = 8; n2 <= c->num_sms - 32; n2++) {
          const double bw = std::min(bw_cap, (c->num_sms - n2) * sm_bw);
          const double waves = (double)((tiles.size() + n2 - 1) / n2);
          const double cost = std::max(eff_bytes / bw, waves * t_cta);
          if (cost < best - 1e-9) {
            best = cost;
            tile_sms = n2;
          }
        }
        if (best >= t_tile_alone + eff_bytes / bw_cap) tile_sms = 0;
      }
    }
    // (width classes side by side without tiles: measured a gain on 16-bit pools only; the
    // FP8 kernels are latency-bound per SM and lose on a share of the SMs)
    concurrent = tile_sms > 0 || (n_classes > 1 && !c->fp8);
  }
  if (!concurrent) {
    if (!tiles.empty()) PA_CUDA(launch_tiles(c, layer, p, work_dev, (int)tiles.size(), stream));
    for (int k = 0; k < 3; k++) {
      if (!have_class[k]) continue;
      p.min_cols = 8 * k + 1;
      p.max_cols = 8 * k + 8;
      PA_CUDA(pa::launch_splitkv_attention(p, c->num_sms, stream, c->unit_map(layer)));
    }
    return PA_OK;
  }
  // SMs of the split-KV classes, in proportion to their weighted bytes, four at least
  const int split_sms = c->num_sms - tile_sms;
  int share[3] = {0, 0, 0};
  {
    int given = 0, largest = 0;
    for (int k = 0; k < 3; k++) {
      if (!have_class[k]) continue;
      share[k] = std::max(4, (int)(split_sms * class_bytes[k] * class_weight[k] / eff_bytes));
      given += share[k];
      if (class_bytes[k] * class_weight[k] > class_bytes[largest] * class_weight[largest] || !have_class[largest])
        largest = k;
    }
    share[largest] += split_sms - given;  // rounding, and what the minimum shares took
    if (share[largest] < 4) {             // cannot happen with 148 SMs and three classes; stay safe
      share[largest] = 4;
    }
  }
  // No early trigger: dependents parked on the SMs would hold registers and shared memory
  // the other kernels' CTAs need.
  p.early_trigger = 0;
  PA_CUDA(cudaEventRecord(c->ev_fork, stream));
  // the largest class on the caller's stream, first, so that it gets its SMs; then the
  // other classes; the tile CTAs fill the rest and, as split-KV CTAs finish, theirs too
  int order[3] = {0, 1, 2};
  std::sort(order, order + 3, [&](int x, int y) { return share[x] > share[y]; });
  int lane = 0, cta_base = 0;
  for (int i = 0; i < 3; i++) {
    const int k = order[i];
    if (!have_class[k]) continue;
    cudaStream_t ls = lane == 0 ? stream : c->lane_stream[lane - 1];
    if (lane > 0) PA_CUDA(cudaStreamWaitEvent(ls, c->ev_fork, 0));
    p.min_cols = 8 * k + 1;
    p.max_cols = 8 * k + 8;
    p.lane = lane;
    p.cta_base = cta_base;
    PA_CUDA(pa::launch_splitkv_attention(p, share[k], ls, c->unit_map(layer)));
    if (lane > 0) {
      PA_CUDA(cudaEventRecord(c->ev_lane[lane - 1], ls));
      PA_CUDA(cudaStreamWaitEvent(stream, c->ev_lane[lane - 1], 0));
    }
    // (the narrow kernel may run two CTAs per SM)
    cta_base += (k == 0 ? pa::splitkv_narrow_ctas_per_sm((int)c->cfg.head_size, c->fp8) : 1) * share[k];
    lane++;
  }
  if (tile_sms > 0) {
    PA_CUDA(cudaStreamWaitEvent(c->aux_stream, c->ev_fork, 0));
    PA_CUDA(launch_tiles(c, layer, p, work_dev, (int)tiles.size(), c->aux_stream));
    PA_CUDA(cudaEventRecord(c->ev_join, c->aux_stream));
    PA_CUDA(cudaStreamWaitEvent(stream, c->ev_join, 0));
  } else if (!tiles.empty()) {
    PA_CUDA(launch_tiles(c, layer, p, work_dev, (int)tiles.size(), stream));
  }
  return PA_OK;
}

}  // namespace

extern "C" {

pa_status pa_paged_attention_varlen(PagedAttnCache *c, uint32_t layer, void *out, const void *q,
                                    const int32_t *block_tables, const int32_t *context_lens,
                                    const int32_t *cu_q_lens_host,
                                    const int32_t *context_lens_host, int32_t num_seqs,
                                    int32_t num_q_heads, int32_t max_blocks_per_seq,
                                    int64_t q_stride, int64_t out_stride, float scale,
                                    float softcap, int32_t max_context_len, void *workspace,
                                    size_t workspace_bytes, void *cuda_stream) {
  (void)max_context_len;
  return attention_impl(c, layer, out, q, block_tables, context_lens, cu_q_lens_host,
                        context_lens_host, num_seqs, num_q_heads, max_blocks_per_seq, q_stride,
                        out_stride, scale, softcap, workspace, workspace_bytes, cuda_stream, nullptr);
}

static pa_status decode_step_impl(PagedAttnCache *c, uint32_t layer, void *out, const void *q,
                                  const void *key, const void *value, const int64_t *slot_mapping,
                                  const int32_t *block_tables, const int32_t *seq_rows,
                                  const int32_t *context_lens, int32_t num_seqs, int32_t num_q_heads,
                                  int32_t max_blocks_per_seq, int64_t q_stride, int64_t out_stride,
                                  int64_t key_stride, int64_t value_stride, float scale, float softcap,
                                  void *workspace, size_t workspace_bytes, void *cuda_stream) {
  pa_status st = check_layer(c, layer);
  if (st != PA_OK) return st;
  if (num_seqs < 0) return fail(PA_ERR_INVALID_ARG, "num_seqs < 0");
  if (num_seqs == 0) return PA_OK;
  if (!key || !value || !slot_mapping) return fail(PA_ERR_INVALID_ARG, "null tensor pointer");
  const int64_t row = (int64_t)c->cfg.num_kv_heads * c->cfg.head_size;
  if (key_stride < row || value_stride < row || (key_stride & 7) || (value_stride & 7))
    return fail(PA_ERR_INVALID_ARG, "key/value stride must be >= num_kv_heads*head_size and a multiple of 8");
  if (!aligned16(key) || !aligned16(value))
    return fail(PA_ERR_INVALID_ARG, "key/value must be 16-byte aligned");
  if (!can_fuse_write(c, num_q_heads, num_seqs)) {
    // FP8 pools (the write quantises), 8- or 32-token blocks, wide GQA groups, many items
    // per CTA: two launches
    st = pa_reshape_and_cache(c, layer, key, value, slot_mapping, num_seqs, key_stride,
                              value_stride, cuda_stream);
    if (st != PA_OK) return st;
    return attention_impl(c, layer, out, q, block_tables, context_lens, nullptr, nullptr, num_seqs,
                          num_q_heads, max_blocks_per_seq, q_stride, out_stride, scale, softcap,
                          workspace, workspace_bytes, cuda_stream, nullptr, seq_rows);
  }
  const StepWrite w{key, value, slot_mapping, key_stride, value_stride};
  return attention_impl(c, layer, out, q, block_tables, context_lens, nullptr, nullptr, num_seqs,
                        num_q_heads, max_blocks_per_seq, q_stride, out_stride, scale, softcap,
                        workspace, workspace_bytes, cuda_stream, &w, seq_rows);
}

pa_status pa_decode_step(PagedAttnCache *c, uint32_t layer, void *out, const void *q,
                         const void *key, const void *value, const int64_t *slot_mapping,
                         const int32_t *block_tables, const int32_t *context_lens,
                         int32_t num_seqs, int32_t num_q_heads, int32_t max_blocks_per_seq,
                         int64_t q_stride, int64_t out_stride, int64_t key_stride,
                         int64_t value_stride, float scale, float softcap, void *workspace,
                         size_t workspace_bytes, void *cuda_stream) {
  return decode_step_impl(c, layer, out, q, key, value, slot_mapping, block_tables, nullptr, context_lens,
                          num_seqs, num_q_heads, max_blocks_per_seq, q_stride, out_stride, key_stride,
                          value_stride, scale, softcap, workspace, workspace_bytes, cuda_stream);
}

pa_status pa_paged_attention_decode_rows(PagedAttnCache *c, uint32_t layer, void *out, const void *q,
                                         const int32_t *block_tables, const int32_t *seq_rows,
                                         const int32_t *context_lens, int32_t num_seqs,
                                         int32_t num_q_heads, int32_t max_blocks_per_seq,
                                         int64_t q_stride, int64_t out_stride, float scale,
                                         float softcap, void *workspace, size_t workspace_bytes,
                                         void *cuda_stream) {
  if (num_seqs > 0 && !seq_rows) return fail(PA_ERR_INVALID_ARG, "seq_rows is null");
  return attention_impl(c, layer, out, q, block_tables, context_lens, nullptr, nullptr, num_seqs,
                        num_q_heads, max_blocks_per_seq, q_stride, out_stride, scale, softcap, workspace,
                        workspace_bytes, cuda_stream, nullptr, seq_rows);
}

pa_status pa_decode_step_rows(PagedAttnCache *c, uint32_t layer, void *out, const void *q,
                              const void *key, const void *value, const int64_t *slot_mapping,
                              const int32_t *block_tables, const int32_t *seq_rows,
                              const int32_t *context_lens, int32_t num_seqs, int32_t num_q_heads,
                              int32_t max_blocks_per_seq, int64_t q_stride, int64_t out_stride,
                              int64_t key_stride, int64_t value_stride, float scale, float softcap,
                              void *workspace, size_t workspace_bytes, void *cuda_stream) {
  return decode_step_impl(c, layer, out, q, key, value, slot_mapping, block_tables, seq_rows, context_lens,
                          num_seqs, num_q_heads, max_blocks_per_seq, q_stride, out_stride, key_stride,
                          value_stride, scale, softcap, workspace, workspace_bytes, cuda_stream);
}

pa_status pa_cache_check_errors_fast(PagedAttnCache *c, void *cuda_stream) {
  if (!c) return fail(PA_ERR_INVALID_ARG, "cache is null");
  if (*reinterpret_cast<volatile unsigned *>(c->err_host) == 0) return PA_OK;
  return pa_cache_check_errors(c, cuda_stream);
}

pa_status pa_paged_attention_decode(PagedAttnCache *c, uint32_t layer, void *out, const void *q,
                                    const int32_t *block_tables, const int32_t *context_lens,
                                    int32_t num_seqs, int32_t num_q_heads,
                                    int32_t max_blocks_per_seq, int64_t q_stride,
                                    int64_t out_stride, float scale, float softcap,
                                    void *workspace, size_t workspace_bytes, void *cuda_stream) {
  return pa_paged_attention_varlen(c, layer, out, q, block_tables, context_lens, nullptr, nullptr,
                                   num_seqs, num_q_heads, max_blocks_per_seq, q_stride, out_stride,
                                   scale, softcap, 0, workspace, workspace_bytes, cuda_stream);
}

pa_status pa_paged_attention_decode_static(PagedAttnCache *c, uint32_t layer, void *out,
                                           const void *q, const int32_t *block_tables,
                                           const int32_t *context_lens, int32_t num_seqs,
                                           int32_t num_q_heads, int32_t max_blocks_per_seq,
                                           int64_t q_stride, int64_t out_stride, float scale,
                                           float softcap, void *cuda_stream) {
  pa_status st = check_layer(c, layer);
  if (st != PA_OK) return st;
  if (c->num_sms > pa::splitkv_static_max_ctas())
    return fail(PA_ERR_UNSUPPORTED,
                "this GPU has " + std::to_string(c->num_sms) + " SMs; the library-resident scratch "
                "holds partial results for at most " + std::to_string(pa::splitkv_static_max_ctas()) +
                " CTAs - use pa_paged_attention_decode with a caller workspace");
  DeviceGuard g(c->device);
  if (!g.ok) return fail(PA_ERR_CUDA, "cannot select device");
  float *scratch = nullptr;
  PA_CUDA(pa::splitkv_static_scratch(c->device, &scratch));
  return pa_paged_attention_decode(c, layer, out, q, block_tables, context_lens, num_seqs,
                                   num_q_heads, max_blocks_per_seq, q_stride, out_stride, scale,
                                   softcap, scratch, pa::splitkv_workspace_bytes(c->num_sms),
                                   cuda_stream);
}

pa_status pa_decode_step_host(PagedAttnCache *c, uint32_t layer, void *out_host,
                              const void *q_host, const void *k_host, const void *v_host,
                              const int64_t *slots_host, const int32_t *tables_host,
                              const int32_t *lens_host, int32_t num_seqs, int32_t num_q_heads,
                              int32_t max_blocks_per_seq, float scale, float softcap) {
  pa_status st = check_layer(c, layer);
  if (st != PA_OK) return st;
  if (num_seqs <= 0) return num_seqs == 0 ? PA_OK : fail(PA_ERR_INVALID_ARG, "num_seqs < 0");
  if (!out_host || !q_host || !k_host || !v_host || !slots_host || !tables_host || !lens_host)
    return fail(PA_ERR_INVALID_ARG, "null host pointer");
  if (num_q_heads <= 0 || max_blocks_per_seq <= 0) return fail(PA_ERR_INVALID_ARG, "bad sizes");
  DeviceGuard g(c->device);
  const size_t D = c->cfg.head_size, Hkv = c->cfg.num_kv_heads, S = (size_t)num_seqs;
  auto up = [](size_t x) { return (x + 255) & ~(size_t)255; };
  const size_t q_b = S * num_q_heads * D * 2, kv_b = S * Hkv * D * 2, sl_b = S * 8,
               tb_b = S * (size_t)max_blocks_per_seq * 4, ln_b = S * 4;
  const size_t o_q = 0, o_k = o_q + up(q_b), o_v = o_k + up(kv_b), o_sl = o_v + up(kv_b),
               o_tb = o_sl + up(sl_b), o_ln = o_tb + up(tb_b), o_out = o_ln + up(ln_b),
               total = o_out + up(q_b);
  st = grow(&c->stage, &c->stage_bytes, total);
  if (st != PA_OK) return st;
  st = grow(&c->ws, &c->ws_bytes, pa_attention_workspace_bytes(c));
  if (st != PA_OK) return st;
  char *base = static_cast<char *>(c->stage);
  cudaStream_t s = c->step_stream;
  // Pinned, device-mapped host buffers (cudaHostAlloc / cudaHostRegister, which is what
  // frameworks' pinned tensors are) are read by the kernels themselves: the KV write takes
  // k, v and the slots straight from host memory and one ingest launch brings q, the
  // tables and the lengths over, instead of six DMA operations in a row.  Anything else
  // (pageable memory) goes through cudaMemcpyAsync.
  auto mapped = [](const void *h) -> const void * {
    cudaPointerAttributes a{};
    if (cudaPointerGetAttributes(&a, h) != cudaSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    return a.type == cudaMemoryTypeHost ? a.devicePointer : nullptr;
  };
  const void *q_m = mapped(q_host), *k_m = mapped(k_host), *v_m = mapped(v_host),
             *sl_m = mapped(slots_host), *tb_m = mapped(tables_host), *ln_m = mapped(lens_host);
  const bool zero_copy = q_m && k_m && v_m && sl_m && tb_m && ln_m && aligned16(q_m) &&
                         aligned16(k_m) && aligned16(v_m) && aligned16(tb_m) && aligned16(ln_m);
  const void *k_src = base + o_k, *v_src = base + o_v, *sl_src = base + o_sl;
  if (zero_copy) {
    pa::StageCopy sc{{q_m, tb_m, ln_m}, {base + o_q, base + o_tb, base + o_ln}, {q_b, tb_b, ln_b}};
    PA_CUDA(pa::launch_stage_copy(sc, s));
    k_src = k_m;
    v_src = v_m;
    sl_src = sl_m;
  } else {
    PA_CUDA(cudaMemcpyAsync(base + o_q, q_host, q_b, cudaMemcpyHostToDevice, s));
    PA_CUDA(cudaMemcpyAsync(base + o_k, k_host, kv_b, cudaMemcpyHostToDevice, s));
    PA_CUDA(cudaMemcpyAsync(base + o_v, v_host, kv_b, cudaMemcpyHostToDevice, s));
    PA_CUDA(cudaMemcpyAsync(base + o_sl, slots_host, sl_b, cudaMemcpyHostToDevice, s));
    PA_CUDA(cudaMemcpyAsync(base + o_tb, tables_host, tb_b, cudaMemcpyHostToDevice, s));
    PA_CUDA(cudaMemcpyAsync(base + o_ln, lens_host, ln_b, cudaMemcpyHostToDevice, s));
  }
  st = pa_decode_step(c, layer, base + o_out, base + o_q, k_src, v_src,
                      static_cast<const int64_t *>(sl_src),
                      reinterpret_cast<const int32_t *>(base + o_tb),
                      reinterpret_cast<const int32_t *>(base + o_ln), num_seqs, num_q_heads,
                      max_blocks_per_seq, (int64_t)(num_q_heads * D), (int64_t)(num_q_heads * D),
                      (int64_t)(Hkv * D), (int64_t)(Hkv * D), scale, softcap, c->ws, c->ws_bytes, s);
  if (st != PA_OK) return st;
  PA_CUDA(cudaMemcpyAsync(out_host, base + o_out, q_b, cudaMemcpyDeviceToHost, s));
  PA_CUDA(cudaStreamSynchronize(s));
  // the attention kernel left a copy of the error word in host-visible memory
  if (*reinterpret_cast<volatile unsigned *>(c->err_host) != 0) return pa_cache_check_errors(c, s);
  return PA_OK;
}

pa_status pa_varlen_step_host(PagedAttnCache *c, uint32_t layer, void *out_host, const void *q_host,
                              const void *k_host, const void *v_host, const int64_t *slots_host,
                              const int32_t *tables_host, const int32_t *lens_host,
                              const int32_t *cu_q_lens_host, int32_t num_seqs, int32_t num_q_heads,
                              int32_t max_blocks_per_seq, float scale, float softcap) {
  pa_status st = check_layer(c, layer);
  if (st != PA_OK) return st;
  if (num_seqs <= 0) return num_seqs == 0 ? PA_OK : fail(PA_ERR_INVALID_ARG, "num_seqs < 0");
  if (!out_host || !q_host || !k_host || !v_host || !slots_host || !tables_host || !lens_host ||
      !cu_q_lens_host)
    return fail(PA_ERR_INVALID_ARG, "null host pointer");
  if (num_q_heads <= 0 || max_blocks_per_seq <= 0) return fail(PA_ERR_INVALID_ARG, "bad sizes");
  const int64_t T = cu_q_lens_host[num_seqs];
  if (T < 0) return fail(PA_ERR_INVALID_ARG, "cu_q_lens must be non-decreasing from 0");
  if (T == 0) return PA_OK;
  DeviceGuard g(c->device);
  const size_t D = c->cfg.head_size, Hkv = c->cfg.num_kv_heads, S = (size_t)num_seqs;
  auto up = [](size_t x) { return (x + 255) & ~(size_t)255; };
  const size_t q_b = (size_t)T * num_q_heads * D * 2, kv_b = (size_t)T * Hkv * D * 2, sl_b = (size_t)T * 8,
               tb_b = S * (size_t)max_blocks_per_seq * 4, ln_b = S * 4;
  const size_t o_q = 0, o_k = o_q + up(q_b), o_v = o_k + up(kv_b), o_sl = o_v + up(kv_b),
               o_tb = o_sl + up(sl_b), o_ln = o_tb + up(tb_b), o_out = o_ln + up(ln_b),
               total = o_out + up(q_b);
  st = grow(&c->stage, &c->stage_bytes, total);
  if (st != PA_OK) return st;
  st = grow(&c->ws, &c->ws_bytes, pa_attention_workspace_bytes(c));
  if (st != PA_OK) return st;
  char *base = static_cast<char *>(c->stage);
  cudaStream_t s = c->step_stream;
  // A chunk's inputs are megabytes: the copy engine moves them (a kernel reading pinned
  // host memory in place is the better route only for the few hundred kilobytes of a
  // decode step).
  PA_CUDA(cudaMemcpyAsync(base + o_q, q_host, q_b, cudaMemcpyHostToDevice, s));
  PA_CUDA(cudaMemcpyAsync(base + o_k, k_host, kv_b, cudaMemcpyHostToDevice, s));
  PA_CUDA(cudaMemcpyAsync(base + o_v, v_host, kv_b, cudaMemcpyHostToDevice, s));
  PA_CUDA(cudaMemcpyAsync(base + o_sl, slots_host, sl_b, cudaMemcpyHostToDevice, s));
  PA_CUDA(cudaMemcpyAsync(base + o_tb, tables_host, tb_b, cudaMemcpyHostToDevice, s));
  PA_CUDA(cudaMemcpyAsync(base + o_ln, lens_host, ln_b, cudaMemcpyHostToDevice, s));
  st = pa_reshape_and_cache(c, layer, base + o_k, base + o_v,
                            reinterpret_cast<const int64_t *>(base + o_sl), T, (int64_t)(Hkv * D),
                            (int64_t)(Hkv * D), s);
  if (st != PA_OK) return st;
  st = pa_paged_attention_varlen(c, layer, base + o_out, base + o_q,
                                 reinterpret_cast<const int32_t *>(base + o_tb),
                                 reinterpret_cast<const int32_t *>(base + o_ln), cu_q_lens_host,
                                 lens_host, num_seqs, num_q_heads, max_blocks_per_seq,
                                 (int64_t)(num_q_heads * D), (int64_t)(num_q_heads * D), scale,
                                 softcap, 0, c->ws, c->ws_bytes, s);
  if (st != PA_OK) return st;
  PA_CUDA(cudaMemcpyAsync(out_host, base + o_out, q_b, cudaMemcpyDeviceToHost, s));
  // every kernel of the call has finished when this copy runs, the tile kernel included
  PA_CUDA(cudaMemcpyAsync(c->err_host, c->err_dev, sizeof(unsigned), cudaMemcpyDeviceToHost, s));
  PA_CUDA(cudaStreamSynchronize(s));
  if (*reinterpret_cast<volatile unsigned *>(c->err_host) != 0) return pa_cache_check_errors(c, s);
  return PA_OK;
}

/* ---- tier 1 ------------------------------------------------------------------ */

mlx_array *pa_array_from_device(void *device_ptr, int32_t dtype, const int64_t *shape, size_t ndim) {
  if (!device_ptr || !shape || ndim > 8 || dtype_size(dtype) == 0) {
    fail(PA_ERR_INVALID_ARG, "pa_array_from_device: bad argument");
    return nullptr;
  }
  mlx_array *a = new (std::nothrow) mlx_array();
  if (!a) return nullptr;
  a->data = device_ptr;
  a->dtype = dtype;
  a->device = t_device;
  a->ndim = ndim;
  for (size_t i = 0; i < ndim; i++) a->shape[i] = shape[i];
  return a;
}

mlx_array *pa_array_from_host(const void *host_ptr, int32_t dtype, const int64_t *shape, size_t ndim) {
  if (!host_ptr || !shape || ndim > 8 || dtype_size(dtype) == 0) {
    fail(PA_ERR_INVALID_ARG, "pa_array_from_host: bad argument");
    return nullptr;
  }
  size_t n = dtype_size(dtype);
  for (size_t i = 0; i < ndim; i++) n *= (size_t)shape[i];
  DeviceGuard g(t_device);
  void *d = nullptr;
  cudaError_t e = cudaMalloc(&d, n ? n : 16);
  if (e == cudaSuccess && n) e = cudaMemcpyAsync(d, host_ptr, n, cudaMemcpyHostToDevice, t_stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(t_stream);
  if (e != cudaSuccess) {
    cuda_fail(e, "pa_array_from_host");
    if (d) cudaFree(d);
    return nullptr;
  }
  mlx_array *a = pa_array_from_device(d, dtype, shape, ndim);
  if (!a) {
    cudaFree(d);
    return nullptr;
  }
  a->owns = true;
  return a;
}

void *pa_array_data(mlx_array *a) { return a ? a->data : nullptr; }
size_t mlx_array_ndim(mlx_array *a) { return a ? a->ndim : 0; }
void mlx_array_shape(mlx_array *a, int64_t *out) {
  if (!a || !out) return;
  for (size_t i = 0; i < a->ndim; i++) out[i] = a->shape[i];
}
int32_t mlx_array_dtype(mlx_array *a) { return a ? a->dtype : -1; }
void mlx_array_delete(mlx_array *a) {
  if (!a) return;
  if (a->owns && a->data) {
    DeviceGuard g(a->device);
    cudaFree(a->data);
  }
  delete a;
}

PagedAttnCache *mlx_paged_attn_create_cache(const PagedAttnConfig *config) {
  PagedAttnCache *c = nullptr;
  if (pa_cache_create(config, t_device, &c) != PA_OK) return nullptr;
  return c;
}
void mlx_paged_attn_free_cache(PagedAttnCache *cache) { pa_cache_free(cache); }

static mlx_array *pool_view(PagedAttnCache *c, uint32_t layer, bool key) {
  if (check_layer(c, layer) != PA_OK) return nullptr;
  const PagedAttnConfig &f = c->cfg;
  mlx_array *a = new (std::nothrow) mlx_array();
  if (!a) return nullptr;
  a->data = key ? c->k[layer] : c->v[layer];
  a->dtype = (int32_t)f.dtype;
  a->device = c->device;
  a->owner = c;
  a->layer = layer;
  if (key) {
    a->ndim = 5;
    const int64_t sh[5] = {f.num_blocks, f.num_kv_heads, f.head_size / 8, f.block_size, 8};
    memcpy(a->shape, sh, sizeof(sh));
  } else {
    a->ndim = 4;
    const int64_t sh[4] = {f.num_blocks, f.num_kv_heads, f.head_size, f.block_size};
    memcpy(a->shape, sh, sizeof(sh));
  }
  return a;
}
mlx_array *mlx_paged_attn_get_key_cache(PagedAttnCache *c, uint32_t layer) { return pool_view(c, layer, true); }
mlx_array *mlx_paged_attn_get_value_cache(PagedAttnCache *c, uint32_t layer) { return pool_view(c, layer, false); }

void mlx_paged_attn_reshape_and_cache(PagedAttnCache *c, uint32_t layer, mlx_array *keys,
                                      mlx_array *values, mlx_array *slot_mapping) {
  if (!c || !keys || !values || !slot_mapping) {
    fail(PA_ERR_INVALID_ARG, "reshape_and_cache: null argument");
    return;
  }
  if (keys->ndim != 3 || values->ndim != 3 || slot_mapping->dtype != 4 ||
      keys->dtype != (int32_t)c->cfg.dtype || values->dtype != (int32_t)c->cfg.dtype ||
      keys->shape[1] != c->cfg.num_kv_heads ||
      keys->shape[2] != c->cfg.head_size || slot_mapping->shape[0] != keys->shape[0]) {
    fail(PA_ERR_INVALID_ARG, "reshape_and_cache: keys/values must be [T,Hkv,D] in the cache dtype, slots int64 [T]");
    return;
  }
  const int64_t row = keys->shape[1] * keys->shape[2];
  pa_reshape_and_cache(c, layer, keys->data, values->data,
                       static_cast<const int64_t *>(slot_mapping->data), keys->shape[0], row, row,
                       t_stream);
}

mlx_array *mlx_paged_attn_forward(mlx_array *q, mlx_array *kc, mlx_array *vc, mlx_array *bt,
                                  mlx_array *cl, float scale, uint32_t block_size,
                                  uint32_t max_context_len) {
  if (!q || !kc || !vc || !bt || !cl) {
    fail(PA_ERR_INVALID_ARG, "forward: null argument");
    return nullptr;
  }
  if (q->ndim != 3 || kc->ndim != 5 || vc->ndim != 4 || bt->ndim != 2 || q->dtype > 1 ||
      kc->dtype != q->dtype || vc->dtype != q->dtype || bt->dtype != 3 || cl->dtype != 3 ||
      (int64_t)block_size != vc->shape[3] || bt->shape[0] != q->shape[0]) {
    fail(PA_ERR_INVALID_ARG, "forward: expected f16/bf16 q [S,Hq,D], pools of the same dtype, int32 tables [S,MB] and lens [S]");
    return nullptr;
  }
  PagedAttnConfig cfg{(uint32_t)vc->shape[3], (uint32_t)vc->shape[0], (uint32_t)vc->shape[2],
                      (uint32_t)vc->shape[1], 1, (uint32_t)q->dtype};
  void *kp = kc->data, *vp = vc->data;
  // This entry takes the pools as arrays, not the cache handle
  // (crates/mlx-sys/src/lib.rs:782-791).  Views handed out by get_key_cache /
  // get_value_cache remember their cache; for any other pair of arrays a transient
  // handle is wrapped around the pools for the duration of the call.
  const bool owned = kc->owner && kc->owner == vc->owner && kc->layer == vc->layer;
  PagedAttnCache *c = owned ? kc->owner : nullptr;
  const uint32_t layer = owned ? kc->layer : 0;
  if (!owned && pa_cache_wrap(&cfg, kc->device, &kp, &vp, &c) != PA_OK) return nullptr;
  const int64_t S = q->shape[0], Hq = q->shape[1], D = q->shape[2];
  DeviceGuard g(c->device);
  void *out = nullptr;
  mlx_array *res = nullptr;
  cudaError_t e = cudaMalloc(&out, (size_t)(S * Hq * D * 2 > 0 ? S * Hq * D * 2 : 16));
  if (e != cudaSuccess) {
    cuda_fail(e, "forward: allocation");
  } else if (grow(&c->ws, &c->ws_bytes, pa_attention_workspace_bytes(c)) == PA_OK &&
             pa_paged_attention_varlen(c, layer, out, q->data, static_cast<const int32_t *>(bt->data),
                                       static_cast<const int32_t *>(cl->data), nullptr, nullptr,
                                       (int32_t)S, (int32_t)Hq, (int32_t)bt->shape[1], Hq * D, Hq * D, scale,
                                       1.0f, (int32_t)max_context_len, c->ws, c->ws_bytes,
                                       t_stream) == PA_OK &&
             cudaStreamSynchronize(t_stream) == cudaSuccess) {
    const int64_t sh[3] = {S, Hq, D};
    res = pa_array_from_device(out, q->dtype, sh, 3);
    if (res) {
      res->owns = true;
      res->device = c->device;
      out = nullptr;
    }
  }
  if (out) cudaFree(out);
  if (!owned) pa_cache_free(c);
  return res;
}

void mlx_paged_attn_copy_blocks(PagedAttnCache *c, uint32_t layer, mlx_array *mapping) {
  if (!c || !mapping) {
    fail(PA_ERR_INVALID_ARG, "copy_blocks: null argument");
    return;
  }
  if (mapping->dtype != 4) {
    fail(PA_ERR_INVALID_ARG, "copy_blocks: block_mapping must be int64");
    return;
  }
  // [num_pairs, 2] or flat [2*num_pairs] (crates/mlx-sys/src/mlx.cpp:4185-4192)
  const bool is_2d = mapping->ndim == 2 && mapping->shape[1] == 2;
  const int64_t pairs = is_2d ? mapping->shape[0] : mapping->shape[0] / 2;
  pa_copy_blocks(c, layer, static_cast<const int64_t *>(mapping->data), pairs, t_stream);
}

}  // extern "C"
