"""ctypes binding of the host-side pool management ABI
(include/paged_attn_b200_host.h): block allocator, token tracker, paged KV cache
bookkeeping and the continuous-batching scheduler, with the method names of the
reference crate (crates/mlx-paged-attn/src/lib.rs:21-51)."""
from __future__ import annotations

import ctypes as C
import re
import os

from . import PagedAttnError, _check, last_error, load_library

u8, u32, i32, i64, u64, sz, vp, f32 = (C.c_uint8, C.c_uint32, C.c_int32, C.c_int64, C.c_uint64,
                                       C.c_size_t, C.c_void_p, C.c_float)
P = C.POINTER


class PaHostConfig(C.Structure):
    _fields_ = [(n, u32) for n in ("block_size", "gpu_memory_mb", "head_size", "num_kv_heads",
                                   "num_layers", "use_fp8_cache", "max_seq_len", "max_batch_size")]


class PaTrackerStats(C.Structure):
    _fields_ = [("num_tracked_blocks", u32), ("total_tracked_tokens", u32),
                ("avg_tokens_per_block", f32), ("prefix_index_size", u32)]


class PaMemoryStats(C.Structure):
    _fields_ = [(n, u32) for n in ("total_blocks", "free_blocks", "allocated_blocks",
                                   "total_memory_mb", "used_memory_mb")] + \
               [("utilization_percent", C.c_double)]


class PaSchedulerConfig(C.Structure):
    _fields_ = [(n, u32) for n in ("max_batch_size", "max_tokens_per_step", "max_prefill_per_step",
                                   "prioritize_decode", "eos_token_id")]


class PaBatchTotals(C.Structure):
    _fields_ = [(n, u32) for n in ("total_tokens", "num_prefill", "num_decode")]


class PaHybridConfig(C.Structure):
    _fields_ = [(n, u32) for n in ("max_batch_size", "max_tokens_per_step", "prefill_chunk_size",
                                   "max_prefill_per_step", "prioritize_decode", "eos_token_id")]


class PaHybridTotals(C.Structure):
    _fields_ = [(n, u32) for n in ("total_tokens", "num_prefill", "num_decode", "num_verify")]


class PaKvScaleStats(C.Structure):
    _fields_ = [("num_layers_calibrated", u32)] + \
               [(n, f32) for n in ("k_scale_min", "k_scale_max", "k_scale_mean", "v_scale_min",
                                   "v_scale_max", "v_scale_mean")]


class PaLayerParams(C.Structure):
    _fields_ = [("layer_idx", u32), ("num_heads", u32), ("num_kv_heads", u32), ("head_size", u32),
                ("scale", f32), ("block_size", u32), ("softcap", f32), ("use_fp8", u32),
                ("k_scale", f32), ("v_scale", f32)]


class PaSchedulerStats(C.Structure):
    _fields_ = [(n, u32) for n in ("num_waiting", "num_running", "num_completed", "num_prefill",
                                   "num_decode", "total_running_tokens")]


_SIGS = {
    "pa_host_config_default": (None, [P(PaHostConfig)]),
    "pa_host_config_validate": (i32, [P(PaHostConfig)]),
    "pa_host_config_num_blocks": (u32, [P(PaHostConfig)]),
    "pa_hash_tokens": (u64, [P(u32), sz, u64]),
    "pa_compute_token_hash": (u64, [P(u32), sz]),
    "pa_kv_compute_scale": (f32, [f32]),
    "pa_shard_head_ranges": (i32, [i32, i32, i32, i32, C.POINTER(i32), C.POINTER(i32), C.POINTER(i32),
                                   C.POINTER(i32)]),
    "pa_alloc_create": (vp, [u32, u32]), "pa_alloc_destroy": (None, [vp]),
    "pa_alloc_allocate": (i64, [vp]), "pa_alloc_release": (i32, [vp, u32]),
    "pa_alloc_incref": (i32, [vp, u32]), "pa_alloc_ref_count": (i64, [vp, u32]),
    "pa_alloc_copy_on_write": (i64, [vp, u32]), "pa_alloc_register_prefix": (i32, [vp, u32, u64]),
    "pa_alloc_lookup_prefix": (i64, [vp, u64]), "pa_alloc_num_free": (u32, [vp]),
    "pa_alloc_num_allocated": (u32, [vp]), "pa_alloc_total": (u32, [vp]),
    "pa_alloc_can_allocate": (i32, [vp, u32]), "pa_alloc_set_max_prefix_entries": (None, [vp, u32]),
    "pa_alloc_prefix_cache_len": (u32, [vp]), "pa_alloc_has_block_hash": (i32, [vp, u32]),
    "pa_alloc_clear_lru_order": (None, [vp]),
    "pa_tracker_create": (vp, [u32, i32]), "pa_tracker_destroy": (None, [vp]),
    "pa_tracker_is_enabled": (i32, [vp]),
    "pa_tracker_track_tokens": (u64, [vp, u32, P(u32), sz, u32]),
    "pa_tracker_get_block_tokens": (u32, [vp, u32, P(u32), sz]),
    "pa_tracker_remove_block": (None, [vp, u32]), "pa_tracker_copy_block": (None, [vp, u32, u32]),
    "pa_tracker_find_prefix_matches": (sz, [vp, P(u32), sz, P(u32), sz]),
    "pa_tracker_find_longest_prefix": (sz, [vp, P(u32), sz, P(u32), sz, P(u32)]),
    "pa_tracker_stats": (None, [vp, P(PaTrackerStats)]), "pa_tracker_clear": (None, [vp]),
    "pa_tracker_memory_usage": (sz, [vp]),
    "pa_table_free_slots_in_last_block": (u32, [u32, u32, u32]),
    "pa_table_blocks_needed": (u32, [u32, u32, u32, u32]),
    "pa_table_is_last_block_full": (i32, [u32, u32]),
    "pa_table_slot_index": (None, [u32, u32, P(u32), P(u32)]),
    "pa_kv_create": (i32, [P(PaHostConfig), P(vp)]), "pa_kv_destroy": (None, [vp]),
    "pa_kv_add_sequence": (i32, [vp, u32, P(u32)]), "pa_kv_remove_sequence": (i32, [vp, u32]),
    "pa_kv_extend_sequence": (i32, [vp, u32, u32]), "pa_kv_fork_sequence": (i32, [vp, u32, P(u32)]),
    "pa_kv_handle_cow": (i32, [vp, u32, u32, P(i32), P(u32), P(u32)]),
    "pa_kv_can_allocate": (i32, [vp, u32]), "pa_kv_num_sequences": (u32, [vp]),
    "pa_kv_num_free_blocks": (u32, [vp]), "pa_kv_total_blocks": (u32, [vp]),
    "pa_kv_block_size": (u32, [vp]), "pa_kv_max_blocks_per_seq": (u32, [vp]),
    "pa_kv_get_context_lens": (sz, [vp, P(u32), sz]), "pa_kv_get_seq_ids": (sz, [vp, P(u32), sz]),
    "pa_kv_build_block_tables": (sz, [vp, P(u32), sz]),
    "pa_kv_sequence_blocks": (i32, [vp, u32, P(u32), sz, P(sz)]),
    "pa_kv_get_slot_mapping": (i32, [vp, u32, u32, u32, P(i64)]),
    "pa_kv_get_slot_mapping_batch": (i32, [vp, P(u32), P(u32), P(u8), P(u32), sz, P(i64), sz, P(sz)]),
    "pa_kv_build_input_metadata": (i32, [vp, P(u32), P(u32), P(u8), sz, P(i32), sz, P(i32), sz, P(i64), sz,
                                         P(sz), P(u32), P(i32)]),
    "pa_kv_memory_stats": (None, [vp, P(PaMemoryStats)]),
    "pa_kv_track_sequence_tokens": (i32, [vp, u32, P(u32), sz, u32]),
    "pa_kv_get_sequence_tokens": (i32, [vp, u32, P(u32), sz, P(sz)]),
    "pa_kv_find_prefix_matches": (sz, [vp, P(u32), sz, P(u32), sz]),
    "pa_kv_find_longest_prefix": (sz, [vp, P(u32), sz, P(u32), sz, P(u32)]),
    "pa_kv_get_block_tokens": (u32, [vp, u32, P(u32), sz]),
    "pa_kv_tracker_stats": (None, [vp, P(PaTrackerStats)]), "pa_kv_tracker_memory": (sz, [vp]),
    "pa_sched_config_default": (None, [P(PaSchedulerConfig)]),
    "pa_sched_create": (vp, [u32, P(PaSchedulerConfig)]), "pa_sched_destroy": (None, [vp]),
    "pa_sched_add_request": (None, [vp, C.c_char_p, P(u32), sz, u32, i32]),
    "pa_sched_schedule_step": (u32, [vp, vp]),
    "pa_sched_batch_totals": (None, [vp, P(PaBatchTotals)]),
    "pa_sched_batch_entry": (i32, [vp, u32, P(u32), P(i32), P(u32), P(u32)]),
    "pa_sched_batch_tokens": (u32, [vp, u32, P(u32), sz]),
    "pa_sched_batch_request_id": (C.c_char_p, [vp, u32]),
    "pa_sched_process_outputs": (i32, [vp, vp, P(u32), P(u32), P(u8), sz]),
    "pa_sched_take_completed": (u32, [vp]),
    "pa_sched_completed_request_id": (C.c_char_p, [vp, u32]),
    "pa_sched_completed_finish_reason": (C.c_char_p, [vp, u32]),
    "pa_sched_completed_tokens": (u32, [vp, u32, P(u32), sz, P(u32)]),
    "pa_sched_abort_request": (i32, [vp, vp, C.c_char_p, P(i32)]),
    "pa_sched_is_empty": (i32, [vp]), "pa_sched_stats": (None, [vp, P(PaSchedulerStats)]),
    "pa_sched_running_is_prefill": (i32, [vp, u32]),
    "pa_hybrid_config_default": (None, [P(PaHybridConfig)]),
    "pa_hybrid_create": (vp, [u32, P(PaHybridConfig)]), "pa_hybrid_destroy": (None, [vp]),
    "pa_hybrid_add_request": (None, [vp, C.c_char_p, P(u32), sz, u32, i32]),
    "pa_hybrid_set_draft_tokens": (i32, [vp, u32, P(u32), sz]),
    "pa_hybrid_schedule_step": (u32, [vp, vp]),
    "pa_hybrid_batch_totals": (None, [vp, P(PaHybridTotals)]),
    "pa_hybrid_batch_entry": (i32, [vp, u32, P(u32), P(i32), P(u32), P(u32), P(i32)]),
    "pa_hybrid_batch_tokens": (u32, [vp, u32, P(u32), sz]),
    "pa_hybrid_batch_request_id": (C.c_char_p, [vp, u32]),
    "pa_hybrid_batch_metadata": (i32, [vp, vp, P(i32), sz, P(i32), P(i32), sz, P(i64), sz, P(u32)]),
    "pa_hybrid_process_outputs": (i32, [vp, vp, P(u32), P(u32), P(u32), P(u8), sz]),
    "pa_hybrid_take_completed": (u32, [vp]),
    "pa_hybrid_completed_request_id": (C.c_char_p, [vp, u32]),
    "pa_hybrid_completed_finish_reason": (C.c_char_p, [vp, u32]),
    "pa_hybrid_completed_tokens": (u32, [vp, u32, P(u32), sz, P(u32)]),
    "pa_hybrid_is_empty": (i32, [vp]), "pa_hybrid_num_waiting": (u32, [vp]),
    "pa_hybrid_num_running": (u32, [vp]),
    "pa_kv_truncate_sequence": (i32, [vp, u32, u32]),
    "pa_kv_extend_sequences": (i32, [vp, P(u32), sz, u32]),
    # the host cache bound to a device cache
    "pa_kv_bind": (i32, [vp, vp, P(vp)]), "pa_kv_unbind": (None, [vp]),
    "pa_kv_update": (i32, [vp, u32, vp, vp, vp, i64, vp]),
    "pa_kv_update_with_slots": (i32, [vp, u32, vp, vp, P(i64), i64, vp]),
    "pa_kv_attention": (i32, [vp, u32, vp, vp, P(u32), sz, u32, f32, vp]),
    "pa_kv_attention_with_context": (i32, [vp, u32, vp, vp, P(u32), P(u32), sz, u32, f32, vp]),
    "pa_kv_decode_step": (i32, [vp, u32, vp, vp, vp, vp, P(u32), sz, u32, f32, vp]),
    "pa_kv_decode_step_host": (i32, [vp, u32, vp, vp, vp, vp, P(u32), sz, u32, f32]),
    "pa_kv_binding_stats": (None, [vp, P(u64), P(u64), P(u32)]),
    "pa_kv_scale_manager": (vp, [vp]),
    "pa_kv_create_bound": (i32, [P(PaHostConfig), i32, u32, P(vp), P(vp), P(vp)]),
    "pa_scale_create": (vp, [u32, f32]), "pa_scale_destroy": (None, [vp]),
    "pa_scale_num_layers": (u32, [vp]), "pa_scale_alpha": (f32, [vp]),
    "pa_scale_init_default_scales": (None, [vp]), "pa_scale_k": (f32, [vp, u32]),
    "pa_scale_v": (f32, [vp, u32]), "pa_scale_is_calibrated": (i32, [vp]),
    "pa_scale_calibrate_layer_max": (None, [vp, u32, f32, f32, P(f32), P(f32)]),
    "pa_scale_update_layer_ema_max": (None, [vp, u32, f32, f32, P(f32), P(f32)]),
    "pa_scale_calibrate_layer": (i32, [vp, u32, vp, vp, sz, i32, i32, P(f32), P(f32), vp]),
    "pa_scale_set_scales": (None, [vp, u32, f32, f32]),
    "pa_scale_get_all_scales": (None, [vp, P(f32), P(f32)]),
    "pa_scale_load_scales": (None, [vp, P(f32), sz, P(f32), sz]),
    "pa_scale_reset": (None, [vp]), "pa_scale_stats": (None, [vp, P(PaKvScaleStats)]),
    "pa_metadata_create": (vp, [P(i32), sz, P(i32), sz, P(i64), sz, u32, i32, u32]),
    "pa_metadata_dummy": (vp, []), "pa_metadata_destroy": (None, [vp]),
    "pa_metadata_num_seqs": (u32, [vp]), "pa_metadata_num_tokens": (sz, [vp]),
    "pa_metadata_is_prefill": (i32, [vp]), "pa_metadata_max_context_len": (u32, [vp]),
    "pa_metadata_max_blocks_per_seq": (u32, [vp]),
    "pa_metadata_device_buffers": (i32, [vp, i32, P(vp), P(vp), P(vp)]),
    "pa_metadata_invalidate_buffers": (None, [vp]),
    "pa_layer_create": (vp, [P(PaLayerParams)]),
    "pa_layer_from_cache_config": (vp, [u32, u32, P(PaHostConfig)]),
    "pa_layer_destroy": (None, [vp]), "pa_layer_get": (None, [vp, P(PaLayerParams)]),
    "pa_layer_set_kv_scales": (None, [vp, f32, f32]),
    "pa_layer_forward": (i32, [vp, vp, vp, vp, vp, vp, vp, P(i32), vp]),
    "pa_layer_forward_decode": (i32, [vp, vp, vp, vp, vp, vp, vp, vp]),
    "pa_layers_create": (vp, [u32, u32, u32, u32, u32, i32]),
    "pa_layers_from_cache_config": (vp, [u32, P(PaHostConfig)]),
    "pa_layers_destroy": (None, [vp]), "pa_layers_get": (vp, [vp, u32]),
    "pa_layers_num_layers": (u32, [vp]),
}
HOST_SYMBOLS = sorted(_SIGS)

_bound = None


def lib():
    global _bound
    if _bound is None:
        l = load_library()
        for name, (res, args) in _SIGS.items():
            fn = getattr(l, name)
            fn.restype, fn.argtypes = res, args
        _bound = l
    return _bound


def _arr(values, ctype=u32):
    values = list(values)
    return (ctype * max(len(values), 1))(*values), len(values)


def hash_tokens(tokens, parent_hash=0) -> int:
    a, n = _arr(tokens)
    return int(lib().pa_hash_tokens(a, n, parent_hash))


def compute_token_hash(tokens) -> int:
    a, n = _arr(tokens)
    return int(lib().pa_compute_token_hash(a, n))


def host_config(**kw) -> PaHostConfig:
    """PagedAttentionConfig { ..Default::default() } with overrides."""
    cfg = PaHostConfig()
    lib().pa_host_config_default(C.byref(cfg))
    for k, v in kw.items():
        setattr(cfg, k, int(v))
    return cfg


class BlockAllocator:
    def __init__(self, num_blocks, block_size):
        self.h = lib().pa_alloc_create(num_blocks, block_size)

    def __del__(self):
        try:  # at interpreter shutdown the module's globals may already be gone
            lib().pa_alloc_destroy(self.h)
        except Exception:
            pass

    def allocate(self):
        r = lib().pa_alloc_allocate(self.h)
        return None if r < 0 else int(r)

    def free(self, block_id): _check(lib().pa_alloc_release(self.h, block_id))
    def incref(self, block_id): _check(lib().pa_alloc_incref(self.h, block_id))
    def ref_count(self, block_id): return int(lib().pa_alloc_ref_count(self.h, block_id))

    def copy_on_write(self, block_id):
        r = lib().pa_alloc_copy_on_write(self.h, block_id)
        return None if r < 0 else int(r)

    def register_prefix(self, block_id, h): _check(lib().pa_alloc_register_prefix(self.h, block_id, h))

    def lookup_prefix(self, h):
        r = lib().pa_alloc_lookup_prefix(self.h, h)
        return None if r < 0 else int(r)

    def num_free_blocks(self): return int(lib().pa_alloc_num_free(self.h))
    def num_allocated_blocks(self): return int(lib().pa_alloc_num_allocated(self.h))
    def total_blocks(self): return int(lib().pa_alloc_total(self.h))
    def can_allocate(self, n): return bool(lib().pa_alloc_can_allocate(self.h, n))
    def set_max_prefix_cache_entries(self, n): lib().pa_alloc_set_max_prefix_entries(self.h, n)
    def prefix_cache_len(self): return int(lib().pa_alloc_prefix_cache_len(self.h))
    def has_block_hash(self, block_id): return bool(lib().pa_alloc_has_block_hash(self.h, block_id))
    def clear_lru_order(self): lib().pa_alloc_clear_lru_order(self.h)


class _TrackerOps:
    """Shared by the standalone tracker and the one inside PagedKVCacheHost."""
    _prefix = "pa_tracker_"

    def _f(self, name): return getattr(lib(), self._prefix + name)

    def get_block_tokens(self, block_id):
        buf = (u32 * 4096)()
        n = self._f("get_block_tokens")(self.h, block_id, buf, 4096)
        return list(buf[:n])

    def find_prefix_matches(self, tokens):
        a, n = _arr(tokens)
        out = (u32 * 8192)()
        m = self._f("find_prefix_matches")(self.h, a, n, out, 4096)
        return [(out[2 * i], out[2 * i + 1]) for i in range(m)]

    def find_longest_prefix(self, tokens):
        a, n = _arr(tokens)
        out, matched = (u32 * 4096)(), u32()
        m = self._f("find_longest_prefix")(self.h, a, n, out, 4096, C.byref(matched))
        return list(out[:m]), int(matched.value)


class TokenTracker(_TrackerOps):
    def __init__(self, block_size, enabled=True):
        self.h = lib().pa_tracker_create(block_size, int(enabled))

    def __del__(self):
        try:  # at interpreter shutdown the module's globals may already be gone
            lib().pa_tracker_destroy(self.h)
        except Exception:
            pass

    def is_enabled(self): return bool(lib().pa_tracker_is_enabled(self.h))

    def track_tokens(self, block_id, tokens, start_offset):
        a, n = _arr(tokens)
        return int(lib().pa_tracker_track_tokens(self.h, block_id, a, n, start_offset))

    def get_block_token_count(self, block_id): return len(self.get_block_tokens(block_id))
    def remove_block(self, block_id): lib().pa_tracker_remove_block(self.h, block_id)
    def copy_block(self, src, dst): lib().pa_tracker_copy_block(self.h, src, dst)

    def stats(self):
        s = PaTrackerStats()
        lib().pa_tracker_stats(self.h, C.byref(s))
        return s

    def clear(self): lib().pa_tracker_clear(self.h)
    def memory_usage(self): return int(lib().pa_tracker_memory_usage(self.h))


class PagedKVCacheHost(_TrackerOps):
    """Host bookkeeping of PagedKVCache (crates/mlx-paged-attn/src/paged_kv_cache.rs)."""
    _prefix = "pa_kv_"

    def __init__(self, cfg: PaHostConfig):
        self.h = vp()
        _check(lib().pa_kv_create(C.byref(cfg), C.byref(self.h)))

    def __del__(self):
        try:  # at interpreter shutdown the module's globals may already be gone
            if getattr(self, "h", None):
                lib().pa_kv_destroy(self.h)
        except Exception:
            pass

    def add_sequence(self, prompt_len):
        sid = u32()
        _check(lib().pa_kv_add_sequence(self.h, prompt_len, C.byref(sid)))
        return int(sid.value)

    def remove_sequence(self, seq_id): _check(lib().pa_kv_remove_sequence(self.h, seq_id))
    def extend_sequence(self, seq_id, n): _check(lib().pa_kv_extend_sequence(self.h, seq_id, n))

    def extend_sequences(self, seq_ids, n):
        """extend_sequence for a whole batch; seq_ids a list or a seq_id_array()."""
        s, count = seq_ids if isinstance(seq_ids, tuple) else _arr(seq_ids)
        _check(lib().pa_kv_extend_sequences(self.h, s, count, n))

    def fork_sequence(self, parent):
        c = u32()
        _check(lib().pa_kv_fork_sequence(self.h, parent, C.byref(c)))
        return int(c.value)

    def handle_cow(self, seq_id, block_idx):
        copied, src, dst = i32(), u32(), u32()
        _check(lib().pa_kv_handle_cow(self.h, seq_id, block_idx, C.byref(copied), C.byref(src), C.byref(dst)))
        return (int(src.value), int(dst.value)) if copied.value else None

    def can_allocate(self, n): return bool(lib().pa_kv_can_allocate(self.h, n))
    def num_sequences(self): return int(lib().pa_kv_num_sequences(self.h))
    def num_free_blocks(self): return int(lib().pa_kv_num_free_blocks(self.h))
    def total_blocks(self): return int(lib().pa_kv_total_blocks(self.h))
    def get_block_size(self): return int(lib().pa_kv_block_size(self.h))
    def get_max_blocks_per_seq(self): return int(lib().pa_kv_max_blocks_per_seq(self.h))

    def _list(self, fn, cap=1 << 16):
        buf = (u32 * cap)()
        n = fn(self.h, buf, cap)
        return list(buf[:n])

    def get_context_lens(self): return self._list(lib().pa_kv_get_context_lens)
    def get_seq_ids(self): return self._list(lib().pa_kv_get_seq_ids)
    def build_block_tables(self): return self._list(lib().pa_kv_build_block_tables, 1 << 20)

    def sequence_blocks(self, seq_id):
        buf, n = (u32 * 8192)(), sz()
        _check(lib().pa_kv_sequence_blocks(self.h, seq_id, buf, 8192, C.byref(n)))
        return list(buf[:n.value])

    def get_slot_mapping(self, seq_id, start_pos, num_tokens):
        out = (i64 * max(num_tokens, 1))()
        _check(lib().pa_kv_get_slot_mapping(self.h, seq_id, start_pos, num_tokens, out))
        return list(out[:num_tokens])

    def get_slot_mapping_batch(self, seq_ids, context_lens, is_prefill, input_lens):
        s, n = _arr(seq_ids)
        c, _ = _arr(context_lens)
        p, _ = _arr([int(x) for x in is_prefill], u8)
        l, _ = _arr(input_lens)
        cap = sum(input_lens) + n + 1
        out, cnt = (i64 * cap)(), sz()
        _check(lib().pa_kv_get_slot_mapping_batch(self.h, s, c, p, l, n, out, cap, C.byref(cnt)))
        return list(out[:cnt.value])

    def get_slot_mapping_decode(self, seq_ids, context_lens):
        return self.get_slot_mapping_batch(seq_ids, context_lens, [False] * len(seq_ids), [1] * len(seq_ids))

    def build_input_metadata(self, seq_ids, input_lens, is_prefill):
        s, n = _arr(seq_ids)
        l, _ = _arr(input_lens)
        p, _ = _arr([int(x) for x in is_prefill], u8)
        mb = self.get_max_blocks_per_seq()
        tables, lens = (i32 * max(n * mb, 1))(), (i32 * max(n, 1))()
        cap = sum(input_lens) + n + 1
        slots, cnt, mx, pf = (i64 * cap)(), sz(), u32(), i32()
        _check(lib().pa_kv_build_input_metadata(self.h, s, l, p, n, tables, max(n * mb, 1), lens, max(n, 1),
                                                slots, cap, C.byref(cnt), C.byref(mx), C.byref(pf)))
        return {"block_tables": list(tables[:n * mb]), "context_lens": list(lens[:n]),
                "slot_mappings": list(slots[:cnt.value]), "max_context_len": int(mx.value),
                "is_prefill": bool(pf.value), "num_seqs": n, "max_blocks_per_seq": mb}

    def build_decode_metadata(self, seq_ids):
        return self.build_input_metadata(seq_ids, [1] * len(seq_ids), [False] * len(seq_ids))

    def build_prefill_metadata(self, seq_ids, prompt_lens):
        return self.build_input_metadata(seq_ids, prompt_lens, [True] * len(seq_ids))

    def get_memory_stats(self):
        s = PaMemoryStats()
        lib().pa_kv_memory_stats(self.h, C.byref(s))
        return s

    def track_sequence_tokens(self, seq_id, tokens, start_pos):
        a, n = _arr(tokens)
        _check(lib().pa_kv_track_sequence_tokens(self.h, seq_id, a, n, start_pos))

    def get_sequence_tokens(self, seq_id):
        buf, n = (u32 * (1 << 16))(), sz()
        _check(lib().pa_kv_get_sequence_tokens(self.h, seq_id, buf, 1 << 16, C.byref(n)))
        return list(buf[:n.value])

    def get_token_tracker_stats(self):
        s = PaTrackerStats()
        lib().pa_kv_tracker_stats(self.h, C.byref(s))
        return s

    def get_token_tracker_memory(self): return int(lib().pa_kv_tracker_memory(self.h))

    def truncate_sequence(self, seq_id, new_num_tokens):
        _check(lib().pa_kv_truncate_sequence(self.h, seq_id, new_num_tokens))


class Scheduler:
    """ContinuousBatchingScheduler (crates/mlx-paged-attn/src/scheduler.rs)."""

    def __init__(self, block_size, **cfg):
        c = None
        if cfg:
            c = PaSchedulerConfig()
            lib().pa_sched_config_default(C.byref(c))
            for k, v in cfg.items():
                setattr(c, k, int(v))
        self.h = lib().pa_sched_create(block_size, C.byref(c) if c is not None else None)

    def __del__(self):
        try:  # at interpreter shutdown the module's globals may already be gone
            lib().pa_sched_destroy(self.h)
        except Exception:
            pass

    def add_request(self, request_id, prompt_tokens, max_new_tokens, priority=0):
        a, n = _arr(prompt_tokens)
        lib().pa_sched_add_request(self.h, request_id.encode(), a, n, max_new_tokens, priority)

    def schedule_step(self, cache: PagedKVCacheHost):
        n = lib().pa_sched_schedule_step(self.h, cache.h)
        if n == 0:
            return None
        t = PaBatchTotals()
        lib().pa_sched_batch_totals(self.h, C.byref(t))
        batch = {"seq_ids": [], "request_ids": [], "input_tokens": [], "is_prefill": [],
                 "context_lens": [], "total_tokens": t.total_tokens, "num_prefill": t.num_prefill,
                 "num_decode": t.num_decode}
        for i in range(n):
            sid, pf, ctx, ni = u32(), i32(), u32(), u32()
            _check(lib().pa_sched_batch_entry(self.h, i, C.byref(sid), C.byref(pf), C.byref(ctx), C.byref(ni)))
            buf = (u32 * max(ni.value, 1))()
            lib().pa_sched_batch_tokens(self.h, i, buf, ni.value)
            batch["seq_ids"].append(int(sid.value))
            batch["is_prefill"].append(bool(pf.value))
            batch["context_lens"].append(int(ctx.value))
            batch["input_tokens"].append(list(buf[:ni.value]))
            batch["request_ids"].append(lib().pa_sched_batch_request_id(self.h, i).decode())
        return batch

    def process_outputs(self, outputs, cache: PagedKVCacheHost):
        """outputs: iterable of (seq_id, token, is_eos)."""
        outputs = list(outputs)
        s, n = _arr([o[0] for o in outputs])
        t, _ = _arr([o[1] for o in outputs])
        e, _ = _arr([int(o[2]) for o in outputs], u8)
        _check(lib().pa_sched_process_outputs(self.h, cache.h, s, t, e, n))

    def get_completed(self):
        n = lib().pa_sched_take_completed(self.h)
        out = []
        for i in range(n):
            buf, total = (u32 * (1 << 16))(), u32()
            k = lib().pa_sched_completed_tokens(self.h, i, buf, 1 << 16, C.byref(total))
            out.append({"request_id": lib().pa_sched_completed_request_id(self.h, i).decode(),
                        "finish_reason": lib().pa_sched_completed_finish_reason(self.h, i).decode(),
                        "generated_tokens": list(buf[:k]), "total_tokens": int(total.value)})
        return out

    def abort_request(self, request_id, cache: PagedKVCacheHost):
        f = i32()
        _check(lib().pa_sched_abort_request(self.h, cache.h, request_id.encode(), C.byref(f)))
        return bool(f.value)

    def is_empty(self): return bool(lib().pa_sched_is_empty(self.h))

    def get_stats(self):
        s = PaSchedulerStats()
        lib().pa_sched_stats(self.h, C.byref(s))
        return s

    def num_waiting(self): return self.get_stats().num_waiting
    def num_running(self): return self.get_stats().num_running
    def num_completed(self): return self.get_stats().num_completed
    def running_is_prefill(self, seq_id): return lib().pa_sched_running_is_prefill(self.h, seq_id)


class HybridScheduler:
    """Chunked prefill + speculative verify + decode in one batch (no reference counterpart)."""
    KINDS = {0: "prefill", 1: "decode", 2: "verify"}

    def __init__(self, block_size, **cfg):
        c = PaHybridConfig()
        lib().pa_hybrid_config_default(C.byref(c))
        for k, v in cfg.items():
            setattr(c, k, int(v))
        self.h = lib().pa_hybrid_create(block_size, C.byref(c))

    def __del__(self):
        try:  # at interpreter shutdown the module's globals may already be gone
            lib().pa_hybrid_destroy(self.h)
        except Exception:
            pass

    def add_request(self, request_id, prompt_tokens, max_new_tokens, priority=0):
        a, n = _arr(prompt_tokens)
        lib().pa_hybrid_add_request(self.h, request_id.encode(), a, n, max_new_tokens, priority)

    def set_draft_tokens(self, seq_id, tokens):
        a, n = _arr(tokens)
        _check(lib().pa_hybrid_set_draft_tokens(self.h, seq_id, a, n))

    def schedule_step(self, cache: PagedKVCacheHost):
        n = lib().pa_hybrid_schedule_step(self.h, cache.h)
        if n == 0:
            return None
        t = PaHybridTotals()
        lib().pa_hybrid_batch_totals(self.h, C.byref(t))
        entries = []
        for i in range(n):
            sid, kind, ql, kv, ns = u32(), i32(), u32(), u32(), i32()
            _check(lib().pa_hybrid_batch_entry(self.h, i, C.byref(sid), C.byref(kind), C.byref(ql),
                                               C.byref(kv), C.byref(ns)))
            buf = (u32 * max(ql.value, 1))()
            lib().pa_hybrid_batch_tokens(self.h, i, buf, ql.value)
            entries.append({"seq_id": int(sid.value), "kind": self.KINDS[kind.value], "q_len": int(ql.value),
                            "kv_len": int(kv.value), "needs_sample": bool(ns.value),
                            "tokens": list(buf[:ql.value]),
                            "request_id": lib().pa_hybrid_batch_request_id(self.h, i).decode()})
        mb = cache.get_max_blocks_per_seq()
        tables, lens, cu = (i32 * (n * mb))(), (i32 * n)(), (i32 * (n + 1))()
        slots, mx = (i64 * max(t.total_tokens, 1))(), u32()
        _check(lib().pa_hybrid_batch_metadata(self.h, cache.h, tables, n * mb, lens, cu, n, slots,
                                              max(t.total_tokens, 1), C.byref(mx)))
        return {"entries": entries, "total_tokens": t.total_tokens, "num_prefill": t.num_prefill,
                "num_decode": t.num_decode, "num_verify": t.num_verify, "block_tables": list(tables),
                "context_lens": list(lens), "cu_q_lens": list(cu), "slot_mapping": list(slots[:t.total_tokens]),
                "max_blocks_per_seq": mb, "max_context_len": int(mx.value)}

    def process_outputs(self, outputs, cache: PagedKVCacheHost):
        """outputs: iterable of (seq_id, num_accepted, next_token, is_eos)."""
        outputs = list(outputs)
        s, n = _arr([o[0] for o in outputs])
        a, _ = _arr([o[1] for o in outputs])
        t, _ = _arr([o[2] for o in outputs])
        e, _ = _arr([int(o[3]) for o in outputs], u8)
        _check(lib().pa_hybrid_process_outputs(self.h, cache.h, s, a, t, e, n))

    def get_completed(self):
        n = lib().pa_hybrid_take_completed(self.h)
        out = []
        for i in range(n):
            buf, total = (u32 * (1 << 16))(), u32()
            k = lib().pa_hybrid_completed_tokens(self.h, i, buf, 1 << 16, C.byref(total))
            out.append({"request_id": lib().pa_hybrid_completed_request_id(self.h, i).decode(),
                        "finish_reason": lib().pa_hybrid_completed_finish_reason(self.h, i).decode(),
                        "generated_tokens": list(buf[:k]), "total_tokens": int(total.value)})
        return out

    def is_empty(self): return bool(lib().pa_hybrid_is_empty(self.h))
    def num_waiting(self): return int(lib().pa_hybrid_num_waiting(self.h))
    def num_running(self): return int(lib().pa_hybrid_num_running(self.h))


def _dev(x) -> int:
    if x is None:
        return 0
    if isinstance(x, int):
        return x
    if hasattr(x, "data_ptr"):
        return x.data_ptr()
    return x.ctypes.data


class KvScaleManager:
    """KvScaleManager of crates/mlx-paged-attn/src/metal/kv_scale.rs:36-300."""

    def __init__(self, num_layers, alpha=None, handle=None):
        self._own = handle is None
        self.h = handle if handle is not None else lib().pa_scale_create(num_layers, 0.1 if alpha is None else alpha)

    @classmethod
    def with_alpha(cls, num_layers, alpha):
        return cls(num_layers, alpha)

    def __del__(self):
        try:  # at interpreter shutdown the module's globals may already be gone
            if getattr(self, "_own", False) and self.h:
                lib().pa_scale_destroy(self.h)
        except Exception:
            pass

    @property
    def num_layers(self): return int(lib().pa_scale_num_layers(self.h))
    @property
    def alpha(self): return float(lib().pa_scale_alpha(self.h))
    def init_default_scales(self): lib().pa_scale_init_default_scales(self.h)
    def k_scale(self, layer): return float(lib().pa_scale_k(self.h, layer))
    def v_scale(self, layer): return float(lib().pa_scale_v(self.h, layer))
    def is_calibrated(self): return bool(lib().pa_scale_is_calibrated(self.h))

    def calibrate_layer_max(self, layer, k_max_abs, v_max_abs):
        k, v = f32(), f32()
        lib().pa_scale_calibrate_layer_max(self.h, layer, k_max_abs, v_max_abs, C.byref(k), C.byref(v))
        return k.value, v.value

    def update_layer_ema_max(self, layer, k_max_abs, v_max_abs):
        k, v = f32(), f32()
        lib().pa_scale_update_layer_ema_max(self.h, layer, k_max_abs, v_max_abs, C.byref(k), C.byref(v))
        return k.value, v.value

    def calibrate_layer(self, layer, keys, values, count, dtype=1, ema=False, stream=0):
        """Scales from device tensors (max |x| by a reduction kernel)."""
        k, v = f32(), f32()
        _check(lib().pa_scale_calibrate_layer(self.h, layer, _dev(keys), _dev(values), count, dtype,
                                              int(ema), C.byref(k), C.byref(v), stream))
        return k.value, v.value

    def update_layer_ema(self, layer, keys, values, count, dtype=1, stream=0):
        return self.calibrate_layer(layer, keys, values, count, dtype, ema=True, stream=stream)

    def set_scales(self, layer, k, v): lib().pa_scale_set_scales(self.h, layer, k, v)

    def get_all_scales(self):
        n = self.num_layers
        k, v = (f32 * max(n, 1))(), (f32 * max(n, 1))()
        lib().pa_scale_get_all_scales(self.h, k, v)
        return list(k[:n]), list(v[:n])

    def load_scales(self, k_scales, v_scales):
        k, nk = _arr(k_scales, f32)
        v, nv = _arr(v_scales, f32)
        lib().pa_scale_load_scales(self.h, k, nk, v, nv)

    def reset(self): lib().pa_scale_reset(self.h)

    def stats(self):
        s = PaKvScaleStats()
        lib().pa_scale_stats(self.h, C.byref(s))
        return s


class InputMetadata:
    """PagedAttentionInputMetadata (+ builder) of input_metadata.rs:29-278."""

    def __init__(self, block_tables, context_lens, slot_mappings, max_context_len, is_prefill,
                 max_blocks_per_seq, handle=None):
        if handle is not None:
            self.h = handle
            return
        t, nt = _arr(block_tables, i32)
        l, nl = _arr(context_lens, i32)
        s, ns = _arr(slot_mappings, i64)
        self.h = lib().pa_metadata_create(t, nt, l, nl, s, ns, max_context_len, int(is_prefill),
                                          max_blocks_per_seq)

    @classmethod
    def dummy(cls):
        return cls(None, None, None, 0, False, 0, handle=lib().pa_metadata_dummy())

    def __del__(self):
        try:  # at interpreter shutdown the module's globals may already be gone
            if self.h:
                lib().pa_metadata_destroy(self.h)
        except Exception:
            pass

    def num_seqs(self): return int(lib().pa_metadata_num_seqs(self.h))
    def num_tokens(self): return int(lib().pa_metadata_num_tokens(self.h))
    def is_prefill(self): return bool(lib().pa_metadata_is_prefill(self.h))
    @property
    def max_context_len(self): return int(lib().pa_metadata_max_context_len(self.h))
    @property
    def max_blocks_per_seq(self): return int(lib().pa_metadata_max_blocks_per_seq(self.h))

    def device_buffers(self, device=0):
        t, l, s = vp(), vp(), vp()
        _check(lib().pa_metadata_device_buffers(self.h, device, C.byref(t), C.byref(l), C.byref(s)))
        return t.value, l.value, s.value

    def invalidate_buffers(self): lib().pa_metadata_invalidate_buffers(self.h)


class InputMetadataBuilder:
    """PagedAttentionInputMetadataBuilder, input_metadata.rs:209-278."""

    def __init__(self):
        self._v = dict(block_tables=[], context_lens=[], slot_mappings=[], max_context_len=0,
                       is_prefill=False, max_blocks_per_seq=0)

    def __getattr__(self, name):
        if name.startswith("_") or name not in self._v:
            raise AttributeError(name)

        def setter(value):
            self._v[name] = value
            return self
        return setter

    def build(self):
        return InputMetadata(**self._v)


class AttentionLayer:
    """PagedAttentionLayer of attention_layer.rs:41-416 (None = the reference's defaults)."""

    def __init__(self, layer_idx=0, num_heads=0, num_kv_heads=0, head_size=0, scale=None, block_size=16,
                 softcap=None, use_fp8=False, k_scale=None, v_scale=None, handle=None, owner=None):
        self._owner = owner  # a layer borrowed from a collection lives as long as it
        if handle is not None:
            self.h = handle
            return
        p = PaLayerParams(layer_idx, num_heads, num_kv_heads, head_size, scale or 0.0, block_size,
                          softcap or 0.0, int(use_fp8), k_scale or 0.0, v_scale or 0.0)
        self.h = lib().pa_layer_create(C.byref(p))

    @classmethod
    def from_cache_config(cls, layer_idx, num_heads, cfg: PaHostConfig):
        return cls(handle=lib().pa_layer_from_cache_config(layer_idx, num_heads, C.byref(cfg)))

    def __del__(self):
        try:  # at interpreter shutdown the module's globals may already be gone
            if self._owner is None and self.h:
                lib().pa_layer_destroy(self.h)
        except Exception:
            pass

    def params(self):
        p = PaLayerParams()
        lib().pa_layer_get(self.h, C.byref(p))
        return p

    def layer_idx(self): return int(self.params().layer_idx)
    def num_heads(self): return int(self.params().num_heads)
    def num_kv_heads(self): return int(self.params().num_kv_heads)
    def head_size(self): return int(self.params().head_size)
    def scale(self): return float(self.params().scale)
    def set_kv_scales(self, k, v): lib().pa_layer_set_kv_scales(self.h, k, v)

    def forward(self, cache: "BoundCache", out, queries, keys, values, metadata: InputMetadata, stream=0):
        """True when `out` holds the attention output (decode); False for a prefill batch."""
        has = i32()
        _check(lib().pa_layer_forward(self.h, cache.h, _dev(out), _dev(queries), _dev(keys), _dev(values),
                                      metadata.h, C.byref(has), stream))
        return bool(has.value)

    def forward_decode(self, cache: "BoundCache", out, queries, keys, values, metadata: InputMetadata, stream=0):
        _check(lib().pa_layer_forward_decode(self.h, cache.h, _dev(out), _dev(queries), _dev(keys),
                                             _dev(values), metadata.h, stream))


class AttentionLayers:
    """PagedAttentionLayers of attention_layer.rs:418-478."""

    def __init__(self, num_layers, num_heads, num_kv_heads, head_size, block_size, use_fp8, handle=None):
        self.h = handle if handle is not None else lib().pa_layers_create(
            num_layers, num_heads, num_kv_heads, head_size, block_size, int(use_fp8))

    @classmethod
    def from_cache_config(cls, num_heads, cfg: PaHostConfig):
        return cls(0, 0, 0, 0, 0, False, handle=lib().pa_layers_from_cache_config(num_heads, C.byref(cfg)))

    def __del__(self):
        try:  # at interpreter shutdown the module's globals may already be gone
            if self.h:
                lib().pa_layers_destroy(self.h)
        except Exception:
            pass

    def num_layers(self): return int(lib().pa_layers_num_layers(self.h))

    def get(self, layer_idx):
        h = lib().pa_layers_get(self.h, layer_idx)
        return AttentionLayer(handle=h, owner=self) if h else None

    def __iter__(self):
        return (self.get(i) for i in range(self.num_layers()))


class BoundCache:
    """A host cache bound to a device cache: the device-touching methods of the
    reference's PagedKVCache (paged_kv_cache.rs:753-1347) on raw device pointers."""

    def __init__(self, host: PagedKVCacheHost, device_cache):
        self.host, self.device_cache = host, device_cache
        self.h = vp()
        _check(lib().pa_kv_bind(host.h, device_cache.handle, C.byref(self.h)))

    def close(self):
        if self.h:
            lib().pa_kv_unbind(self.h)
            self.h = vp()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def update(self, keys, values, slot_mapping_dev, num_tokens, layer=0, stream=0):
        _check(lib().pa_kv_update(self.h, layer, _dev(keys), _dev(values), _dev(slot_mapping_dev), num_tokens,
                                  stream))

    def update_with_slots(self, keys, values, slot_mapping, layer=0, stream=0):
        s, n = _arr(slot_mapping, i64)
        _check(lib().pa_kv_update_with_slots(self.h, layer, _dev(keys), _dev(values), s, n, stream))

    def attention(self, out, queries, seq_ids, num_query_heads, scale, layer=0, stream=0):
        s, n = _arr(seq_ids)
        _check(lib().pa_kv_attention(self.h, layer, _dev(out), _dev(queries), s, n, num_query_heads, scale,
                                     stream))

    def attention_with_context(self, out, queries, seq_ids, context_lens, num_query_heads, scale, layer=0,
                               stream=0):
        s, n = _arr(seq_ids)
        c, _ = _arr(context_lens)
        _check(lib().pa_kv_attention_with_context(self.h, layer, _dev(out), _dev(queries), s, c, n,
                                                  num_query_heads, scale, stream))

    def decode_step(self, out, queries, keys, values, seq_ids, num_query_heads, scale, layer=0, stream=0):
        s, n = seq_ids if isinstance(seq_ids, tuple) else _arr(seq_ids)
        _check(lib().pa_kv_decode_step(self.h, layer, _dev(out), _dev(queries), _dev(keys), _dev(values), s, n,
                                       num_query_heads, scale, stream))

    def decode_step_host(self, out_host, q_host, k_host, v_host, seq_ids, num_query_heads, scale, layer=0):
        s, n = seq_ids if isinstance(seq_ids, tuple) else _arr(seq_ids)
        _check(lib().pa_kv_decode_step_host(self.h, layer, _dev(out_host), _dev(q_host), _dev(k_host),
                                            _dev(v_host), s, n, num_query_heads, scale))

    def stats(self):
        e, c, r = u64(), u64(), u32()
        lib().pa_kv_binding_stats(self.h, C.byref(e), C.byref(c), C.byref(r))
        return {"table_entries_sent": int(e.value), "calls": int(c.value), "rows_in_use": int(r.value)}

    def scale_manager(self):
        h = lib().pa_kv_scale_manager(self.h)
        return KvScaleManager(0, handle=h) if h else None

    # -- FP8 scale methods of PagedKVCache (paged_kv_cache.rs:226-309) ---------------------
    def get_layer_scales(self, layer):
        m = self.scale_manager()
        return (m.k_scale(layer), m.v_scale(layer)) if m else (1.0, 1.0)

    def is_fp8_calibrated(self):
        m = self.scale_manager()
        return bool(m and m.is_calibrated())

    def get_scale_stats(self):
        m = self.scale_manager()
        return m.stats() if m else None

    def set_layer_scales(self, layer, k, v):
        m = self.scale_manager()
        if m:
            m.set_scales(layer, k, v)

    def load_scales(self, k_scales, v_scales):
        m = self.scale_manager()
        if m:
            m.load_scales(k_scales, v_scales)

    def get_all_scales(self):
        m = self.scale_manager()
        return m.get_all_scales() if m else None

    def calibrate_layer_scales(self, layer, keys, values, count, dtype=1, stream=0):
        m = self.scale_manager()
        if not m:
            raise PagedAttnError(1, "FP8 scale calibration requires use_fp8 to be enabled in config")
        return m.calibrate_layer(layer, keys, values, count, dtype, stream=stream)

    def update_layer_scales_ema(self, layer, keys, values, count, dtype=1, stream=0):
        m = self.scale_manager()
        if not m:
            raise PagedAttnError(1, "FP8 scale update requires use_fp8 to be enabled in config")
        return m.update_layer_ema(layer, keys, values, count, dtype, stream=stream)


def seq_id_array(seq_ids):
    """A reusable ctypes array of sequence ids (saves the conversion on every step)."""
    return _arr(seq_ids)
