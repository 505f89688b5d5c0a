"""Host tests of the hybrid scheduler (chunked prefill + speculative verify + decode in
one batch).  The reference has no such scheduler (crates/mlx-paged-attn/src/
scheduler.rs:237-242), so these pin this library's own contract: the metadata a
batch carries is what pa_paged_attention_varlen needs, and the pool bookkeeping
stays consistent through chunking, accepted and rejected draft tokens."""
import pytest

import paged_attn_b200 as pa
from paged_attn_b200.host import HybridScheduler, PagedKVCacheHost, host_config


def make_cache(**kw):
    base = dict(block_size=16, gpu_memory_mb=256, head_size=128, num_kv_heads=8, num_layers=1, max_seq_len=512)
    base.update(kw)
    return PagedKVCacheHost(host_config(**base))


def test_prompt_is_chunked_and_sampled_only_after_the_last_chunk():
    cache, s = make_cache(), HybridScheduler(16, prefill_chunk_size=40)
    s.add_request("r", list(range(100)), 4)
    seen = []
    for want_q, want_kv, want_sample in ((40, 40, False), (40, 80, False), (20, 100, True)):
        b = s.schedule_step(cache)
        e = b["entries"][0]
        assert (e["kind"], e["q_len"], e["kv_len"], e["needs_sample"]) == ("prefill", want_q, want_kv, want_sample)
        assert e["tokens"] == list(range(want_kv - want_q, want_kv))
        assert b["cu_q_lens"] == [0, want_q] and b["context_lens"] == [want_kv]
        # the chunk's slots are the positions [kv_len - q_len, kv_len) of the sequence
        assert b["slot_mapping"] == cache.get_slot_mapping(e["seq_id"], want_kv - want_q, want_q)
        seen.append(e["seq_id"])
        s.process_outputs([(e["seq_id"], 0, 7, False)] if want_sample else [], cache)
    assert len(set(seen)) == 1
    b = s.schedule_step(cache)
    e = b["entries"][0]
    assert (e["kind"], e["q_len"], e["kv_len"], e["tokens"]) == ("decode", 1, 101, [7])
    assert cache.get_context_lens() == [101]


def test_verify_accept_and_reject_keep_the_pool_consistent():
    cache, s = make_cache(), HybridScheduler(16, prefill_chunk_size=0)
    s.add_request("r", list(range(30)), 50)
    b = s.schedule_step(cache)
    sid = b["entries"][0]["seq_id"]
    s.process_outputs([(sid, 0, 100, False)], cache)            # first token
    assert cache.get_context_lens() == [31]
    s.set_draft_tokens(sid, [201, 202, 203, 204])
    b = s.schedule_step(cache)
    e = b["entries"][0]
    assert (e["kind"], e["q_len"], e["kv_len"]) == ("verify", 5, 35)
    assert e["tokens"] == [100, 201, 202, 203, 204]
    assert b["slot_mapping"] == cache.get_slot_mapping(sid, 30, 5)
    assert cache.get_context_lens() == [35] and len(cache.sequence_blocks(sid)) == 3
    # two drafts accepted, then a different token: 3 new tokens, 2 speculative slots dropped
    s.process_outputs([(sid, 2, 300, False)], cache)
    assert cache.get_context_lens() == [34] and len(cache.sequence_blocks(sid)) == 3
    b = s.schedule_step(cache)
    e = b["entries"][0]
    assert (e["kind"], e["q_len"], e["kv_len"], e["tokens"]) == ("decode", 1, 34, [300])
    s.process_outputs([(sid, 0, 301, False)], cache)
    # all drafts accepted
    s.set_draft_tokens(sid, [401, 402])
    b = s.schedule_step(cache)
    assert b["entries"][0]["kv_len"] == 37
    s.process_outputs([(sid, 2, 403, False)], cache)
    assert cache.get_context_lens() == [38]
    # rejected drafts that had opened a new block give the block back
    s.set_draft_tokens(sid, list(range(500, 512)))
    free_before = cache.num_free_blocks()
    b = s.schedule_step(cache)
    assert b["entries"][0]["kv_len"] == 50 and cache.num_free_blocks() == free_before - 1
    s.process_outputs([(sid, 0, 600, False)], cache)
    assert cache.get_context_lens() == [39] and cache.num_free_blocks() == free_before


def test_mixed_batch_and_token_budget():
    cache = make_cache()
    s = HybridScheduler(16, prefill_chunk_size=64, max_tokens_per_step=80, max_prefill_per_step=2)
    s.add_request("a", list(range(20)), 10)
    b = s.schedule_step(cache)
    a = b["entries"][0]["seq_id"]
    s.process_outputs([(a, 0, 1, False)], cache)
    s.add_request("b", list(range(200)), 10)
    s.set_draft_tokens(a, [2, 3, 4])
    b = s.schedule_step(cache)
    kinds = [e["kind"] for e in b["entries"]]
    assert kinds == ["verify", "prefill"] and (b["num_verify"], b["num_prefill"]) == (1, 1)
    assert [e["q_len"] for e in b["entries"]] == [4, 64]
    assert b["total_tokens"] == 68 <= 80
    assert b["cu_q_lens"] == [0, 4, 68] and b["context_lens"] == [24, 64]
    mb = b["max_blocks_per_seq"]
    assert len(b["block_tables"]) == 2 * mb and len(b["slot_mapping"]) == 68
    s.process_outputs([(a, 3, 5, False)], cache)
    b = s.schedule_step(cache)
    assert [(e["kind"], e["q_len"]) for e in b["entries"]] == [("decode", 1), ("prefill", 64)]


def test_completion_by_length_and_eos_frees_the_blocks():
    cache, s = make_cache(), HybridScheduler(16, eos_token_id=999)
    free0 = cache.num_free_blocks()
    s.add_request("len", [1, 2, 3], 2)
    s.add_request("eos", [4, 5, 6], 100)
    b = s.schedule_step(cache)                                  # prefill of "len" (one prefill per step)
    assert [e["request_id"] for e in b["entries"]] == ["len"]
    len_id = b["entries"][0]["seq_id"]
    s.process_outputs([(len_id, 0, 10, False)], cache)
    b = s.schedule_step(cache)                                  # decode of "len" + prefill of "eos"
    assert [(e["request_id"], e["kind"]) for e in b["entries"]] == [("len", "decode"), ("eos", "prefill")]
    eos_id = b["entries"][1]["seq_id"]
    s.process_outputs([(len_id, 0, 20, False), (eos_id, 0, 10, False)], cache)
    done = s.get_completed()
    assert len(done) == 1 and done[0]["request_id"] == "len"
    assert done[0]["finish_reason"] == "length" and done[0]["generated_tokens"] == [10, 20]
    assert done[0]["total_tokens"] == 5
    s.set_draft_tokens(eos_id, [11, 999, 12])
    b = s.schedule_step(cache)
    assert b["entries"][0]["kind"] == "verify" and b["entries"][0]["tokens"] == [10, 11, 999, 12]
    s.process_outputs([(eos_id, 3, 13, False)], cache)          # the accepted drafts contain EOS
    done = s.get_completed()
    assert done[0]["finish_reason"] == "stop" and done[0]["generated_tokens"] == [10, 11, 999]
    assert s.is_empty() and cache.num_sequences() == 0 and cache.num_free_blocks() == free0


def test_truncate_sequence():
    cache = make_cache()
    sid = cache.add_sequence(50)
    assert len(cache.sequence_blocks(sid)) == 4
    cache.truncate_sequence(sid, 33)
    assert len(cache.sequence_blocks(sid)) == 3 and cache.get_context_lens() == [33]
    cache.truncate_sequence(sid, 32)
    assert len(cache.sequence_blocks(sid)) == 2
    with pytest.raises(pa.PagedAttnError):
        cache.truncate_sequence(sid, 40)
