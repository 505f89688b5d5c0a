"""The reference's host-side unit tests for the paged cache, re-expressed against
the C ABI of this library (same test names, same asserted values).  Sources:
crates/mlx-paged-attn/src/{block_allocator,block_table,config,paged_kv_cache,
scheduler,token_tracker}.rs `mod tests`, and metal/kv_scale.rs for the scale rule."""
import struct

import numpy as np

import pytest

import paged_attn_b200 as pa
from paged_attn_b200 import host
from paged_attn_b200.host import (BlockAllocator, PagedKVCacheHost, Scheduler, TokenTracker,
                                  compute_token_hash, hash_tokens, host_config, lib)


# ---- block_allocator.rs:255-434 -----------------------------------------------------
def test_allocate_and_free():
    a = BlockAllocator(10, 32)
    assert a.num_free_blocks() == 10
    b = a.allocate()
    assert a.num_free_blocks() == 9 and b == 0
    a.free(b)
    assert a.num_free_blocks() == 10


def test_reference_counting():
    a = BlockAllocator(10, 32)
    b = a.allocate()
    assert a.ref_count(b) == 1
    a.incref(b)
    assert a.ref_count(b) == 2
    a.free(b)
    assert a.num_free_blocks() == 9
    a.free(b)
    assert a.num_free_blocks() == 10


def test_copy_on_write():
    a = BlockAllocator(10, 32)
    b = a.allocate()
    assert a.copy_on_write(b) is None
    a.incref(b)
    new = a.copy_on_write(b)
    assert new is not None and new != b
    assert a.ref_count(b) == 1 and a.ref_count(new) == 1
    a.free(b)
    a.free(new)


def test_prefix_cache():
    a = BlockAllocator(10, 32)
    b = a.allocate()
    h = hash_tokens([1, 2, 3], 0)
    a.register_prefix(b, h)
    assert a.lookup_prefix(h) == b
    assert a.ref_count(b) == 2
    assert a.lookup_prefix(12345) is None


def test_prefix_cache_cleanup_on_free():
    a = BlockAllocator(10, 32)
    b = a.allocate()
    h = hash_tokens([1, 2, 3], 0)
    a.register_prefix(b, h)
    assert a.lookup_prefix(h) == b
    a.free(b)
    a.free(b)
    assert a.lookup_prefix(h) is None
    assert a.num_free_blocks() == 10


def test_prefix_cache_eviction_cleanup():
    a = BlockAllocator(10, 32)
    a.set_max_prefix_cache_entries(2)
    b1, b2 = a.allocate(), a.allocate()
    h1, h2, h3 = hash_tokens([1], 0), hash_tokens([2], 0), hash_tokens([3], 0)
    a.register_prefix(b1, h1)
    a.register_prefix(b2, h2)
    assert a.prefix_cache_len() == 2
    b3 = a.allocate()
    a.register_prefix(b3, h3)
    assert a.lookup_prefix(h1) is None
    assert a.lookup_prefix(h2) is not None and a.lookup_prefix(h3) is not None
    assert not a.has_block_hash(b1) and a.has_block_hash(b2) and a.has_block_hash(b3)


def test_prefix_cache_disabled():
    a = BlockAllocator(10, 32)
    a.set_max_prefix_cache_entries(0)
    b = a.allocate()
    h = hash_tokens([1, 2, 3], 0)
    a.register_prefix(b, h)
    assert a.prefix_cache_len() == 0 and a.lookup_prefix(h) is None


def test_prefix_cache_eviction_safety():
    a = BlockAllocator(10, 32)
    a.set_max_prefix_cache_entries(1)
    b1 = a.allocate()
    a.register_prefix(b1, hash_tokens([1], 0))
    a.clear_lru_order()
    b2 = a.allocate()
    a.register_prefix(b2, hash_tokens([2], 0))   # must return, not spin
    assert a.prefix_cache_len() > 0


def test_hash_tokens_is_siphash_1_3_zero_key():
    # Rust's DefaultHasher over parent_hash (u64) then each token (u32), zero key.
    M = (1 << 64) - 1

    def rotl(x, b): return ((x << b) | (x >> (64 - b))) & M

    def sip13(data):
        v = [0x736f6d6570736575, 0x646f72616e646f6d, 0x6c7967656e657261, 0x7465646279746573]

        def rnd():
            v[0] = (v[0] + v[1]) & M; v[1] = rotl(v[1], 13); v[1] ^= v[0]; v[0] = rotl(v[0], 32)
            v[2] = (v[2] + v[3]) & M; v[3] = rotl(v[3], 16); v[3] ^= v[2]
            v[0] = (v[0] + v[3]) & M; v[3] = rotl(v[3], 21); v[3] ^= v[0]
            v[2] = (v[2] + v[1]) & M; v[1] = rotl(v[1], 17); v[1] ^= v[2]; v[2] = rotl(v[2], 32)
        n = len(data)
        for i in range(0, n - n % 8, 8):
            m = int.from_bytes(data[i:i + 8], "little")
            v[3] ^= m; rnd(); v[0] ^= m
        b = ((n & 0xFF) << 56) | int.from_bytes(data[n - n % 8:], "little")
        v[3] ^= b; rnd(); v[0] ^= b; v[2] ^= 0xFF
        rnd(); rnd(); rnd()
        return v[0] ^ v[1] ^ v[2] ^ v[3]
    for tokens, parent in (([1, 2, 3], 0), ([], 7), (list(range(40)), 0xDEADBEEFCAFEF00D)):
        data = struct.pack("<Q", parent) + struct.pack(f"<{len(tokens)}I", *tokens)
        assert hash_tokens(tokens, parent) == sip13(data)
    assert hash_tokens([1, 2, 3], 0) != hash_tokens([1, 2, 3], 1)


# ---- block_table.rs:264-316 -----------------------------------------------------------
def test_sequence_block_table():
    L = lib()
    assert L.pa_table_free_slots_in_last_block(0, 0, 32) == 0          # no blocks yet
    assert not L.pa_table_is_last_block_full(20, 32)
    assert L.pa_table_free_slots_in_last_block(1, 20, 32) == 12
    assert L.pa_table_blocks_needed(1, 20, 32, 10) == 0
    assert L.pa_table_blocks_needed(1, 20, 32, 15) == 1
    assert L.pa_table_is_last_block_full(32, 32)
    assert L.pa_table_free_slots_in_last_block(1, 32, 32) == 0


def test_slot_index():
    import ctypes as C
    for pos, want in ((0, (0, 0)), (31, (0, 31)), (32, (1, 0)), (50, (1, 18))):
        b, o = C.c_uint32(), C.c_uint32()
        lib().pa_table_slot_index(pos, 32, C.byref(b), C.byref(o))
        assert (b.value, o.value) == want


def test_block_table():
    cache = PagedKVCacheHost(host_config(gpu_memory_mb=1024))
    s1, s2 = cache.add_sequence(1), cache.add_sequence(1)
    assert cache.num_sequences() == 2 and set(cache.get_seq_ids()) == {s1, s2}
    cache.remove_sequence(s1)
    assert cache.num_sequences() == 1 and cache.get_seq_ids() == [s2]
    with pytest.raises(pa.PagedAttnError):
        cache.remove_sequence(s1)


# ---- config.rs:144-236 -------------------------------------------------------------------
def test_config_validation():
    import ctypes as C
    cfg = host_config()
    assert lib().pa_host_config_validate(C.byref(cfg)) == 0
    cfg.block_size = 64
    assert lib().pa_host_config_validate(C.byref(cfg)) != 0
    assert "Invalid block_size: 64" in pa.last_error()
    cfg.block_size = 32
    cfg.head_size = 100
    assert lib().pa_host_config_validate(C.byref(cfg)) != 0
    cfg.head_size = 128
    assert lib().pa_host_config_validate(C.byref(cfg)) == 0


def test_block_calculation():
    import ctypes as C
    cfg = host_config(block_size=32, gpu_memory_mb=1024, head_size=128, num_kv_heads=4, num_layers=28)
    n = lib().pa_host_config_num_blocks(C.byref(cfg))
    assert 500 < n < 700 and n == 1073741824 // (2 * 4 * 128 * 32 * 2 * 28)


def test_fp8_doubles_capacity():
    import ctypes as C
    a = host_config(block_size=32, gpu_memory_mb=1024, num_kv_heads=4, num_layers=28)
    b = host_config(block_size=32, gpu_memory_mb=1024, num_kv_heads=4, num_layers=28, use_fp8_cache=1)
    na, nb = lib().pa_host_config_num_blocks(C.byref(a)), lib().pa_host_config_num_blocks(C.byref(b))
    assert na * 2 - 1 <= nb <= na * 2 + 1


def test_fp8_validation():
    import ctypes as C
    for bs in (32, 16):
        assert lib().pa_host_config_validate(C.byref(host_config(use_fp8_cache=1, block_size=bs))) == 0
    assert lib().pa_host_config_validate(C.byref(host_config(use_fp8_cache=1, block_size=8))) != 0
    assert "block_size 16 or 32" in pa.last_error()


# ---- paged_kv_cache.rs:1669-2024 --------------------------------------------------------------
def small_cache(**kw):
    base = dict(block_size=32, gpu_memory_mb=1024, head_size=128, num_kv_heads=4, num_layers=28)
    base.update(kw)
    return PagedKVCacheHost(host_config(**base))


def test_paged_kv_cache():
    cache = small_cache()
    sid = cache.add_sequence(100)
    assert cache.num_sequences() == 1 and cache.get_memory_stats().allocated_blocks == 4
    cache.remove_sequence(sid)
    assert cache.num_sequences() == 0 and cache.get_memory_stats().allocated_blocks == 0


def test_extend_sequence():
    cache = small_cache()
    sid = cache.add_sequence(30)
    blocks = [cache.get_memory_stats().allocated_blocks]
    for n in (2, 1, 30, 2):
        cache.extend_sequence(sid, n)
        blocks.append(cache.get_memory_stats().allocated_blocks)
    assert blocks == [1, 1, 2, 2, 3]
    assert cache.get_context_lens() == [65]
    cache.remove_sequence(sid)


def test_slot_mapping():
    cache = small_cache()
    sid = cache.add_sequence(64)
    slots = cache.get_slot_mapping(sid, 0, 5)
    assert slots == [0, 1, 2, 3, 4]       # a fresh pool hands out block 0 first
    slots = cache.get_slot_mapping(sid, 32, 3)
    assert len(slots) == 3 and slots[0] >= 32
    with pytest.raises(pa.PagedAttnError):
        cache.get_slot_mapping(sid, 64, 1)    # position beyond the allocated blocks
    cache.remove_sequence(sid)


def test_block_tables():
    cache = small_cache(max_seq_len=256)
    s1, s2 = cache.add_sequence(64), cache.add_sequence(96)
    assert cache.num_sequences() == 2 and cache.get_memory_stats().allocated_blocks == 5
    tables, mb = cache.build_block_tables(), cache.get_max_blocks_per_seq()
    assert mb == 8 and len(tables) == 2 * mb
    assert tables[:2] == [0, 1] and tables[2:8] == [0] * 6 and tables[8:11] == [2, 3, 4]
    cache.remove_sequence(s1)
    cache.remove_sequence(s2)


def test_fork_sequence():
    cache = small_cache()
    parent = cache.add_sequence(64)
    assert cache.get_memory_stats().allocated_blocks == 2
    child = cache.fork_sequence(parent)
    assert cache.num_sequences() == 2 and cache.get_memory_stats().allocated_blocks == 2
    lens = cache.get_context_lens()
    assert len(lens) == 2 and lens[0] == lens[1]
    cache.remove_sequence(parent)
    assert cache.num_sequences() == 1 and cache.get_memory_stats().allocated_blocks == 2
    cache.remove_sequence(child)
    assert cache.num_sequences() == 0 and cache.get_memory_stats().allocated_blocks == 0


def test_handle_cow_after_fork():
    # handle_cow (paged_kv_cache.rs:1476-1523): a shared block is replaced by a fresh one
    cache = small_cache()
    parent = cache.add_sequence(40)
    child = cache.fork_sequence(parent)
    assert cache.handle_cow(child, 1) == (1, 2)
    assert cache.sequence_blocks(child) == [0, 2] and cache.sequence_blocks(parent) == [0, 1]
    assert cache.handle_cow(child, 1) is None          # no longer shared
    assert cache.get_memory_stats().allocated_blocks == 3
    with pytest.raises(pa.PagedAttnError):
        cache.handle_cow(child, 9)


def test_token_tracking_integration():
    cache = small_cache(block_size=8, num_layers=2)
    tokens = list(range(100, 108)) + list(range(200, 208)) + list(range(300, 308))
    s1 = cache.add_sequence(len(tokens))
    cache.track_sequence_tokens(s1, tokens, 0)
    assert cache.get_sequence_tokens(s1) == tokens
    tokens2 = list(range(100, 108)) + list(range(500, 508))
    s2 = cache.add_sequence(len(tokens2))
    cache.track_sequence_tokens(s2, tokens2, 0)
    assert len(cache.find_prefix_matches(list(range(100, 108)))) == 1
    blocks, matched = cache.find_longest_prefix(list(range(100, 108)) + list(range(200, 208)) + [999] * 8)
    assert matched == 16 and len(blocks) == 2
    assert cache.get_token_tracker_memory() > 0
    st = cache.get_token_tracker_stats()
    assert st.num_tracked_blocks > 0 and st.total_tracked_tokens >= 40
    cache.remove_sequence(s1)
    assert cache.get_sequence_tokens(s2) == tokens2


def test_token_tracking_prefix_caching_workflow():
    cache = small_cache(block_size=8, num_layers=2)
    system = list(range(1, 25))
    s1 = cache.add_sequence(32)
    cache.track_sequence_tokens(s1, system + list(range(100, 108)), 0)
    blocks, matched = cache.find_longest_prefix(system)
    assert matched == 24 and len(blocks) == 3
    for b in blocks:
        assert cache.get_block_tokens(b)


def test_metadata_for_the_kernels():
    # build_input_metadata (paged_kv_cache.rs:646-704): int32 tables zero-padded to
    # max_seq_len/block_size columns, int32 lens, int64 slots; decode slot = context_len-1
    cache = small_cache(block_size=16, max_seq_len=128)
    a, b = cache.add_sequence(20), cache.add_sequence(33)
    m = cache.build_prefill_metadata([a, b], [20, 33])
    assert m["is_prefill"] and m["max_blocks_per_seq"] == 8 and m["max_context_len"] == 33
    assert m["block_tables"] == [0, 1] + [0] * 6 + [2, 3, 4] + [0] * 5
    assert m["context_lens"] == [20, 33]
    assert m["slot_mappings"] == list(range(20)) + [2 * 16 + i for i in range(33)]
    cache.extend_sequence(a, 1)
    cache.extend_sequence(b, 1)
    d = cache.build_decode_metadata([b, a])
    assert not d["is_prefill"] and d["context_lens"] == [34, 21]
    assert d["slot_mappings"] == [4 * 16 + 1, 1 * 16 + 4]
    assert cache.get_slot_mapping_decode([a], [21]) == [20]
    with pytest.raises(pa.PagedAttnError) as e:
        cache.get_slot_mapping_decode([a], [0])
    assert "context_len=0" in str(e.value)


def test_pool_exhaustion_is_an_error_not_a_crash():
    cache = small_cache(gpu_memory_mb=256, num_layers=28)
    total = cache.total_blocks()
    with pytest.raises(pa.PagedAttnError) as e:
        cache.add_sequence((total + 1) * 32)
    assert "Not enough memory" in str(e.value)
    sid = cache.add_sequence(total * 32)
    assert cache.num_free_blocks() == 0 and not cache.can_allocate(1)
    with pytest.raises(pa.PagedAttnError):
        cache.extend_sequence(sid, 1)


# ---- token_tracker.rs:405-702 ----------------------------------------------------------------
def test_token_tracker_creation():
    assert TokenTracker(32).is_enabled() and not TokenTracker(0, enabled=False).is_enabled()


def test_track_tokens():
    t = TokenTracker(32)
    assert t.track_tokens(0, [1, 2, 3, 4, 5], 0) != 0
    assert t.get_block_tokens(0) == [1, 2, 3, 4, 5] and t.get_block_token_count(0) == 5


def test_track_tokens_with_offset():
    t = TokenTracker(32)
    t.track_tokens(0, [1, 2, 3], 0)
    t.track_tokens(0, [4, 5], 3)
    assert t.get_block_tokens(0) == [1, 2, 3, 4, 5]


def test_remove_block():
    t = TokenTracker(32)
    t.track_tokens(0, [1, 2, 3], 0)
    t.track_tokens(1, [4, 5, 6], 0)
    t.remove_block(0)
    assert t.get_block_token_count(0) == 0 and t.get_block_token_count(1) == 3


def test_copy_block():
    t = TokenTracker(32)
    t.track_tokens(0, [1, 2, 3, 4, 5], 0)
    t.copy_block(0, 1)
    assert t.get_block_tokens(0) == t.get_block_tokens(1) == [1, 2, 3, 4, 5]


def test_find_prefix_matches():
    t = TokenTracker(4)
    t.track_tokens(0, [1, 2, 3, 4], 0)
    t.track_tokens(1, [5, 6, 7, 8], 0)
    t.track_tokens(2, [1, 2, 3, 4], 0)
    m = t.find_prefix_matches([1, 2, 3, 4])
    assert m and m[0][1] == 4


def test_find_longest_prefix():
    t = TokenTracker(4)
    t.track_tokens(0, [1, 2, 3, 4], 0)
    t.track_tokens(1, [5, 6, 7, 8], 0)
    assert t.find_longest_prefix([1, 2, 3, 4, 5, 6, 7, 8]) == ([0, 1], 8)
    blocks, n = t.find_longest_prefix([1, 2, 3, 4, 9, 9, 9, 9])
    assert (len(blocks), n) == (1, 4)
    assert t.find_longest_prefix([9, 9, 9, 9]) == ([], 0)


def test_stats():
    t = TokenTracker(32)
    t.track_tokens(0, [1, 2, 3], 0)
    t.track_tokens(1, [4, 5, 6, 7], 0)
    s = t.stats()
    assert s.num_tracked_blocks == 2 and s.total_tracked_tokens == 7
    assert abs(s.avg_tokens_per_block - 3.5) < 0.01


def test_disabled_tracker():
    t = TokenTracker(0, enabled=False)
    assert t.track_tokens(0, [1, 2, 3], 0) == 0 and t.get_block_token_count(0) == 0
    assert t.find_prefix_matches([1, 2, 3]) == []


def test_hash_consistency():
    assert compute_token_hash([1, 2, 3, 4, 5]) == compute_token_hash([1, 2, 3, 4, 5])
    assert compute_token_hash([1, 2, 3, 4, 5]) != compute_token_hash([1, 2, 3, 4, 6])
    # FNV-1a, constants of token_tracker.rs:370-371, over the little-endian bytes
    h = 0xCBF29CE484222325
    for b in struct.pack("<2I", 7, 300):
        h = ((h ^ b) * 0x100000001B3) & ((1 << 64) - 1)
    assert compute_token_hash([7, 300]) == h
    assert compute_token_hash([]) == 0xCBF29CE484222325


def test_memory_usage():
    t = TokenTracker(32)
    before = t.memory_usage()
    t.track_tokens(0, [1, 2, 3, 4, 5], 0)
    assert t.memory_usage() >= before


def test_clear():
    t = TokenTracker(32)
    t.track_tokens(0, [1, 2, 3], 0)
    t.track_tokens(1, [4, 5, 6], 0)
    assert t.stats().num_tracked_blocks == 2
    t.clear()
    assert t.stats().num_tracked_blocks == 0


def test_shared_hash_after_copy_block_track_tokens():
    t = TokenTracker(4)
    t.track_tokens(0, [1, 2, 3, 4], 0)
    t.copy_block(0, 1)
    assert t.find_prefix_matches([1, 2, 3, 4])[0][0] == 1
    t.track_tokens(0, [5, 6, 7, 8], 0)
    assert t.find_prefix_matches([1, 2, 3, 4])[0][0] == 1


def test_shared_hash_after_copy_block_remove_block():
    t = TokenTracker(4)
    t.track_tokens(0, [1, 2, 3, 4], 0)
    t.copy_block(0, 1)
    t.remove_block(0)
    assert t.find_prefix_matches([1, 2, 3, 4])[0][0] == 1


def test_shared_hash_copy_block_overwrites():
    t = TokenTracker(4)
    t.track_tokens(0, [1, 2, 3, 4], 0)
    t.track_tokens(1, [5, 6, 7, 8], 0)
    assert t.find_prefix_matches([1, 2, 3, 4]) and t.find_prefix_matches([5, 6, 7, 8])
    t.copy_block(0, 1)
    assert t.find_prefix_matches([5, 6, 7, 8]) == []
    assert t.find_prefix_matches([1, 2, 3, 4])[0][0] == 1


def test_copy_block_nonexistent_source_preserves_destination():
    t = TokenTracker(4)
    t.track_tokens(1, [5, 6, 7, 8], 0)
    t.copy_block(99, 1)
    assert t.get_block_tokens(1) == [5, 6, 7, 8]
    assert t.find_prefix_matches([5, 6, 7, 8])[0][0] == 1


# ---- scheduler.rs:502-764 ----------------------------------------------------------------------
def sched_cache():
    return PagedKVCacheHost(host_config(block_size=16, gpu_memory_mb=1024, head_size=128,
                                        num_kv_heads=4, num_layers=2))


def test_scheduler_creation():
    s = Scheduler(16)
    assert s.is_empty() and s.num_waiting() == 0 and s.num_running() == 0


def test_add_request():
    s = Scheduler(16)
    s.add_request("req1", [1, 2, 3, 4], 10)
    assert s.num_waiting() == 1 and not s.is_empty()


def test_priority_ordering():
    cache, s = sched_cache(), Scheduler(16)
    s.add_request("low", [1], 10, priority=0)
    s.add_request("high", [2], 10, priority=10)
    s.add_request("medium", [3], 10, priority=5)
    assert s.schedule_step(cache)["request_ids"][0] == "high"


def test_schedule_step():
    cache, s = sched_cache(), Scheduler(16)
    s.add_request("req1", [1, 2, 3, 4], 10)
    b = s.schedule_step(cache)
    assert b is not None and len(b["seq_ids"]) == 1
    assert b["num_prefill"] == 1 and b["num_decode"] == 0 and b["is_prefill"][0]
    assert b["input_tokens"] == [[1, 2, 3, 4]] and b["context_lens"] == [4]
    assert s.num_waiting() == 0 and s.num_running() == 1


def test_process_outputs():
    cache, s = sched_cache(), Scheduler(16)
    s.add_request("req1", [1, 2, 3, 4], 3)
    sid = s.schedule_step(cache)["seq_ids"][0]
    s.process_outputs([(sid, 100, False)], cache)
    assert s.num_running() == 1 and s.running_is_prefill(sid) == 0
    s.process_outputs([(sid, 101, False)], cache)
    s.process_outputs([(sid, 102, False)], cache)
    assert s.num_running() == 0 and s.num_completed() == 1
    done = s.get_completed()
    assert len(done) == 1 and done[0]["request_id"] == "req1"
    assert done[0]["finish_reason"] == "length" and done[0]["generated_tokens"] == [100, 101, 102]
    assert done[0]["total_tokens"] == 7 and cache.num_sequences() == 0


def test_eos_stops_generation():
    cache, s = sched_cache(), Scheduler(16, eos_token_id=999)
    s.add_request("req1", [1, 2, 3, 4], 100)
    sid = s.schedule_step(cache)["seq_ids"][0]
    s.process_outputs([(sid, 999, True)], cache)
    assert s.num_running() == 0 and s.get_completed()[0]["finish_reason"] == "stop"


def test_abort_request():
    cache, s = sched_cache(), Scheduler(16)
    s.add_request("req1", [1, 2], 10)
    s.add_request("req2", [3, 4], 10)
    assert s.abort_request("req2", cache) and s.num_waiting() == 1
    s.schedule_step(cache)
    assert s.num_running() == 1
    assert s.abort_request("req1", cache) and s.num_running() == 0
    assert not s.abort_request("req999", cache)


def test_multiple_sequences():
    cache, s = sched_cache(), Scheduler(16, max_batch_size=4, max_prefill_per_step=2)
    for i in range(3):
        s.add_request(f"req{i}", [1, 2, 3, 4], 5)
    b = s.schedule_step(cache)
    assert b["num_prefill"] == 2 and s.num_running() == 2 and s.num_waiting() == 1
    for sid in b["seq_ids"]:
        s.process_outputs([(sid, 100, False)], cache)
    b = s.schedule_step(cache)
    assert b["num_decode"] >= 2 and b["num_prefill"] >= 1
    # the decode entries carry the position that already counts the generated token
    for sid, pf, ctx in zip(b["seq_ids"], b["is_prefill"], b["context_lens"]):
        assert ctx == (4 if pf else 5)


def test_scheduler_backpressure_when_the_pool_is_full():
    # scheduler.rs:258-261: a request that does not fit stays queued
    cache = PagedKVCacheHost(host_config(block_size=16, gpu_memory_mb=256, num_kv_heads=4, num_layers=28))
    s = Scheduler(16, max_tokens_per_step=1 << 30, max_prefill_per_step=4)
    s.add_request("big", [1] * (cache.total_blocks() * 16), 4)
    s.add_request("next", [1] * 16, 4)
    b = s.schedule_step(cache)
    assert b["request_ids"] == ["big"] and s.num_waiting() == 1
    assert s.schedule_step(cache) is None or "next" not in s.schedule_step(cache)["request_ids"]


# ---- metal/kv_scale.rs:373-386 ------------------------------------------------------------------
def test_compute_scale():
    f = lib().pa_kv_compute_scale
    assert abs(f(448.0) - 1.0) < 1e-6 and abs(f(224.0) - 2.0) < 1e-6 and abs(f(896.0) - 0.5) < 1e-6
    assert f(0.0) == 1.0


# ---- metal/kv_scale.rs:341-448 (the other seven; compute_scale is above) ------------------------
from paged_attn_b200.host import (AttentionLayer, AttentionLayers, InputMetadata,  # noqa: E402
                                  InputMetadataBuilder, KvScaleManager)


def test_scale_manager_creation():
    m = KvScaleManager(28)
    assert m.num_layers == 28 and not m.is_calibrated()
    assert m.k_scale(0) == 1.0 and m.v_scale(0) == 1.0


def test_default_scales():
    m = KvScaleManager(4)
    m.init_default_scales()
    for i in range(4):
        assert m.k_scale(i) == 1.0 and m.v_scale(i) == 1.0


def test_set_scales():
    m = KvScaleManager(4)
    m.set_scales(0, 0.5, 0.25)
    m.set_scales(1, 2.0, 1.5)
    assert (m.k_scale(0), m.v_scale(0), m.k_scale(1), m.v_scale(1)) == (0.5, 0.25, 2.0, 1.5)
    assert m.is_calibrated()


def test_serialization():
    m = KvScaleManager(4)
    for i, (k, v) in enumerate([(0.5, 0.25), (2.0, 1.5), (1.0, 1.0), (0.8, 0.9)]):
        m.set_scales(i, k, v)
    ks, vs = m.get_all_scales()
    f = lambda xs: [np.float32(x) for x in xs]
    assert ks == f([0.5, 2.0, 1.0, 0.8]) and vs == f([0.25, 1.5, 1.0, 0.9])
    m2 = KvScaleManager(4)
    m2.load_scales(ks, vs)
    for i in range(4):
        assert m2.k_scale(i) == m.k_scale(i) and m2.v_scale(i) == m.v_scale(i)


def test_scale_stats():
    m = KvScaleManager(4)
    for i, (k, v) in enumerate([(0.5, 0.25), (2.0, 1.5), (1.0, 1.0), (0.5, 0.25)]):
        m.set_scales(i, k, v)
    s = m.stats()
    assert s.num_layers_calibrated == 4 and s.k_scale_min == 0.5 and s.k_scale_max == 2.0
    assert abs(s.k_scale_mean - 1.0) < 1e-6


def test_scale_reset():
    m = KvScaleManager(4)
    m.set_scales(0, 0.5, 0.25)
    assert m.is_calibrated()
    m.reset()
    assert not m.is_calibrated() and m.k_scale(0) == 1.0


def test_with_alpha():
    assert KvScaleManager.with_alpha(4, 0.5).alpha == 0.5
    assert KvScaleManager.with_alpha(4, -0.5).alpha == 0.0   # clamped
    assert KvScaleManager.with_alpha(4, 1.5).alpha == 1.0
    assert abs(KvScaleManager(4).alpha - 0.1) < 1e-7          # DEFAULT_ALPHA


def test_scale_calibration_arithmetic():
    # kv_scale.rs:108-180: one-shot = 448 / max; running maximum m = a*obs + (1-a)*m,
    # the first observation seeding m (and then being averaged with itself)
    m = KvScaleManager.with_alpha(2, 0.5)
    assert m.calibrate_layer_max(0, 224.0, 896.0) == (2.0, 0.5) and m.is_calibrated()
    k, v = m.update_layer_ema_max(1, 448.0, 448.0)
    assert (k, v) == (1.0, 1.0)
    k, v = m.update_layer_ema_max(1, 896.0, 224.0)       # m_k = 672, m_v = 336
    assert abs(k - 448.0 / 672.0) < 1e-6 and abs(v - 448.0 / 336.0) < 1e-6


# ---- attention_layer.rs:484-546 -----------------------------------------------------------------------
def test_layer_creation():
    layer = AttentionLayer(0, 32, 8, 128, block_size=16)
    assert (layer.layer_idx(), layer.num_heads(), layer.num_kv_heads(), layer.head_size()) == (0, 32, 8, 128)
    assert abs(layer.scale() - 0.0884) < 0.001
    p = layer.params()
    assert p.softcap == 1.0 and p.k_scale == 1.0 and p.v_scale == 1.0 and p.use_fp8 == 0


def test_layers_collection():
    layers = AttentionLayers(28, 32, 8, 128, 16, False)
    assert layers.num_layers() == 28
    assert layers.get(0) is not None and layers.get(27) is not None and layers.get(28) is None
    for i, layer in enumerate(layers):
        assert layer.layer_idx() == i


def test_from_cache_config():
    cfg = host_config(block_size=32, gpu_memory_mb=4096, head_size=128, num_kv_heads=4, num_layers=28)
    layer = AttentionLayer.from_cache_config(5, 32, cfg)
    assert (layer.layer_idx(), layer.num_heads(), layer.num_kv_heads(), layer.head_size()) == (5, 32, 4, 128)
    layers = AttentionLayers.from_cache_config(32, cfg)
    assert layers.num_layers() == 28 and layers.get(3).params().block_size == 32


# ---- input_metadata.rs:284-321 ------------------------------------------------------------------------
def test_input_metadata_creation():
    m = InputMetadata([0, 1, 2, 3], [32, 64], [0, 1, 2], 64, False, 2)
    assert m.num_seqs() == 2 and m.num_tokens() == 3 and not m.is_prefill() and m.max_context_len == 64


def test_builder():
    m = (InputMetadataBuilder().block_tables([0, 1]).context_lens([16]).slot_mappings([0])
         .max_context_len(16).is_prefill(True).max_blocks_per_seq(2).build())
    assert m.num_seqs() == 1 and m.is_prefill()


def test_dummy():
    m = InputMetadata.dummy()
    assert m.num_seqs() == 1 and m.is_prefill()


# ---- cache_engine.rs:222-236 (the host half; the device half is in tests/test_gpu_bound_cache.py) ---------
def test_cache_engine_manager_host():
    cfg = host_config(block_size=32, gpu_memory_mb=1024, head_size=128, num_kv_heads=4, num_layers=28)
    cache = PagedKVCacheHost(cfg)
    assert cfg.num_layers == 28 and cache.num_free_blocks() > 0


# ---- metal/copy_blocks.rs:185-195 ---------------------------------------------------------------------------
def test_copy_blocks_params():
    # numel_per_block = num_kv_heads * head_size * block_size; the library's copy moves that
    # many elements of K and of V per pair (pa_swap_block_bytes reports the same figure in bytes)
    import ctypes as ct
    kb, vb = ct.c_uint64(), ct.c_uint64()
    pa.load_library().pa_swap_block_bytes(4, 128, 16, 0, ct.byref(kb), ct.byref(vb))
    assert kb.value == 4 * 128 * 16 * 2 and vb.value == 4 * 128 * 16 * 2


def test_metadata_buffers_are_bounded():
    # a caller buffer sized for a narrower table is refused, not overrun
    cache = PagedKVCacheHost(host_config(block_size=16, gpu_memory_mb=256, num_kv_heads=4, num_layers=28,
                                         max_seq_len=256))
    a = cache.add_sequence(40)
    mb = cache.get_max_blocks_per_seq()
    import ctypes as ct
    s = (ct.c_uint32 * 1)(a)
    l = (ct.c_uint32 * 1)(1)
    p = (ct.c_uint8 * 1)(0)
    tables, lens, slots = (ct.c_int32 * (mb - 1))(), (ct.c_int32 * 1)(), (ct.c_int64 * 4)()
    cnt = ct.c_size_t()
    rc = lib().pa_kv_build_input_metadata(cache.h, s, l, p, 1, tables, mb - 1, lens, 1, slots, 4, ct.byref(cnt),
                                          None, None)
    assert rc == 1
