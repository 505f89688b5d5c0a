"""The host cache bound to a device cache: PagedKVCache::{update, update_with_slots,
attention, attention_with_context} (crates/mlx-paged-attn/src/paged_kv_cache.rs:753-1347),
PagedAttentionLayer::forward (attention_layer.rs:217-416), the FP8 scale manager on
device tensors, the resident block tables and the per-layer host copies of swapped
blocks.  Results against the CPU oracle: KV bytes bit-exact, attention within the
parity rule of pa_testlib.check_attention."""
import ctypes as C

import numpy as np
import pytest
import torch

import paged_attn_b200 as pa
from gpu_util import to_bits, to_dev
from paged_attn_b200.host import (AttentionLayer, BoundCache, InputMetadata, PagedKVCacheHost,
                                  PaHostConfig, host_config, lib)
from pa_testlib import (BS, CANARY, D, X, attention_oracle_rows, bf16_to_f32, check_attention,
                        normal_bf16, write_oracle)

pytestmark = pytest.mark.gpu

HKV, HQ = 4, 16


class World:
    """A host cache + device cache + binding, and numpy pools that follow every write."""

    def __init__(self, prompt_lens, layers=1, seed=3):
        self.cfg = host_config(block_size=BS, gpu_memory_mb=256, head_size=D, num_kv_heads=HKV,
                               num_layers=layers, max_seq_len=2048)
        self.host = PagedKVCacheHost(self.cfg)
        self.NB = self.host.total_blocks()
        self.k_np = [np.full((self.NB, HKV, D // X, BS, X), CANARY, dtype=np.uint16) for _ in range(layers)]
        self.v_np = [np.full((self.NB, HKV, D, BS), CANARY, dtype=np.uint16) for _ in range(layers)]
        self.kd = [to_dev(k) for k in self.k_np]
        self.vd = [to_dev(v) for v in self.v_np]
        self.dev = pa.PagedCache(BS, self.NB, D, HKV, num_layers=layers, key_pools=self.kd, value_pools=self.vd)
        self.bound = BoundCache(self.host, self.dev)
        self.seed = seed
        self.step_no = 0
        self.seqs = [self.host.add_sequence(n) for n in prompt_lens]
        for sid, n in zip(self.seqs, prompt_lens):   # prefill through update_with_slots
            slots = self.host.get_slot_mapping(sid, 0, n)
            for layer in range(layers):
                self.write(layer, slots)

    def fresh(self, shape):
        self.step_no += 1
        return normal_bf16(shape, self.seed, 100 + self.step_no)

    def write(self, layer, slots):
        n = len(slots)
        k, v = self.fresh((n, HKV, D)), self.fresh((n, HKV, D))
        self.bound.update_with_slots(to_dev(k), to_dev(v), slots, layer=layer)
        write_oracle(self.k_np[layer], self.v_np[layer], k, v, np.asarray(slots, dtype=np.int64), HKV)

    def oracle(self, layer, q_bits, seq_ids, ctx=None):
        mb = self.host.get_max_blocks_per_seq()
        tables = np.zeros((len(seq_ids), mb), dtype=np.int32)
        lens = np.zeros(len(seq_ids), dtype=np.int32)
        all_lens = dict(zip(self.host.get_seq_ids(), self.host.get_context_lens()))
        for i, sid in enumerate(seq_ids):
            blocks = self.host.sequence_blocks(sid)
            tables[i, :len(blocks)] = blocks
            lens[i] = all_lens[sid] if ctx is None else ctx[i]
        rows = [(s, 0, h) for s in range(len(seq_ids)) for h in range(HQ)]
        ref = attention_oracle_rows(rows, q_bits, self.k_np[layer], self.v_np[layer], tables, lens, None, HQ,
                                    HKV, mb, 1.0 / np.sqrt(D))
        return ref.reshape(len(seq_ids), HQ, D)

    def pools_match(self, layer=0):
        return (to_bits(self.kd[layer]) == self.k_np[layer]).all() and \
               (to_bits(self.vd[layer]) == self.v_np[layer]).all()


def test_two_decode_steps_through_update_and_attention_only(cuda_device):
    w = World([300, 16, 31, 1029])
    scale = 1.0 / np.sqrt(D)
    sent_before = w.bound.stats()["table_entries_sent"]
    assert sent_before == 0   # update_with_slots needs no tables
    for step in range(2):
        for sid in w.seqs:
            w.host.extend_sequence(sid, 1)
        lens = dict(zip(w.host.get_seq_ids(), w.host.get_context_lens()))
        slots = w.host.get_slot_mapping_decode(w.seqs, [lens[s] for s in w.seqs])
        w.write(0, slots)
        order = w.seqs if step == 0 else w.seqs[::-1]   # batch order is the caller's
        q = w.fresh((len(order), HQ, D))
        out = torch.full((len(order), HQ, D), float("nan"), dtype=torch.bfloat16, device="cuda")
        w.bound.attention(out, to_dev(q), order, HQ, scale)
        torch.cuda.synchronize()
        w.dev.check_errors()
        assert w.pools_match()
        check_attention(bf16_to_f32(to_bits(out)), w.oracle(0, q, order), f"bound attention step {step}")
        st = w.bound.stats()
        if step == 0:   # first attention: every block of every sequence goes over once
            assert st["table_entries_sent"] == sum(len(w.host.sequence_blocks(s)) for s in w.seqs)
            first = st["table_entries_sent"]
        else:           # second: only the blocks the step appended (16 -> 17 and 31 -> 32 + 1 crossed none here)
            new_blocks = sum(len(w.host.sequence_blocks(s)) for s in w.seqs) - first
            assert st["table_entries_sent"] - first == new_blocks
    assert st["rows_in_use"] == 4


def test_attention_with_context_and_missing_sequence(cuda_device):
    w = World([200, 77])
    scale = 1.0 / np.sqrt(D)
    q = w.fresh((2, HQ, D))
    out = torch.zeros(2, HQ, D, dtype=torch.bfloat16, device="cuda")
    w.bound.attention_with_context(out, to_dev(q), w.seqs, [150, 40], HQ, scale)
    torch.cuda.synchronize()
    check_attention(bf16_to_f32(to_bits(out)), w.oracle(0, q, w.seqs, ctx=[150, 40]), "with context")
    with pytest.raises(pa.PagedAttnError) as e:
        w.bound.attention(out, to_dev(q), [w.seqs[0], 999], HQ, scale)
    assert "Sequence 999 not found" in str(e.value)


def test_decode_step_one_launch_device_and_host_buffers(cuda_device):
    w = World([300, 16, 31, 1029, 5])
    scale = 1.0 / np.sqrt(D)
    for use_host in (False, True):
        for sid in w.seqs:
            w.host.extend_sequence(sid, 1)
        lens = dict(zip(w.host.get_seq_ids(), w.host.get_context_lens()))
        slots = np.asarray(w.host.get_slot_mapping_decode(w.seqs, [lens[s] for s in w.seqs]), dtype=np.int64)
        n = len(w.seqs)
        q, k, v = w.fresh((n, HQ, D)), w.fresh((n, HKV, D)), w.fresh((n, HKV, D))
        write_oracle(w.k_np[0], w.v_np[0], k, v, slots, HKV)
        before = pa.kernel_launch_count()
        if use_host:
            pin = lambda a: torch.from_numpy(a.view(np.int16)).pin_memory()
            out_h = torch.zeros(n, HQ, D, dtype=torch.int16).pin_memory()
            w.bound.decode_step_host(out_h, pin(q), pin(k), pin(v), w.seqs, HQ, scale)
            got = bf16_to_f32(out_h.numpy().view(np.uint16))
            # pageable buffers take the copy-engine route to the same result
            out_p = np.zeros((n, HQ, D), dtype=np.uint16)
            w.bound.decode_step_host(out_p, q, k, v, w.seqs, HQ, scale)
            assert np.array_equal(bf16_to_f32(out_p), got)
        else:
            out = torch.zeros(n, HQ, D, dtype=torch.bfloat16, device="cuda")
            w.bound.decode_step(out, to_dev(q), to_dev(k), to_dev(v), w.seqs, HQ, scale)
            torch.cuda.synchronize()
            got = bf16_to_f32(to_bits(out))
            assert pa.kernel_launch_count() - before == 2   # ingest + the fused step
        w.dev.check_errors()
        assert w.pools_match(), "the fused step's KV write differs from the oracle's"
        check_attention(got, w.oracle(0, q, w.seqs), "bound decode step")


def test_rows_are_reclaimed_and_tables_follow_copy_on_write(cuda_device):
    w = World([40, 40])
    scale = 1.0 / np.sqrt(D)
    q = w.fresh((2, HQ, D))
    out = torch.zeros(2, HQ, D, dtype=torch.bfloat16, device="cuda")
    w.bound.attention(out, to_dev(q), w.seqs, HQ, scale)
    # fork, then copy-on-write of the child's last block: its table row must follow
    child = w.host.fork_sequence(w.seqs[0])
    pair = w.host.handle_cow(child, 2)
    assert pair is not None
    src, dst = pair
    pairs = torch.tensor([[src, dst]], dtype=torch.int64, device="cuda")
    w.dev.copy_blocks(pairs, 1)
    for pool in (w.k_np[0], w.v_np[0]):
        pool[dst] = pool[src]
    q1 = w.fresh((1, HQ, D))
    out1 = torch.zeros(1, HQ, D, dtype=torch.bfloat16, device="cuda")
    w.bound.attention(out1, to_dev(q1), [child], HQ, scale)
    torch.cuda.synchronize()
    check_attention(bf16_to_f32(to_bits(out1)), w.oracle(0, q1, [child]), "forked child")
    assert w.bound.stats()["rows_in_use"] == 3


def test_layer_forward_prefill_returns_none_decode_attends(cuda_device):
    # attention_layer.rs:217-384
    w = World([], layers=2)
    layer = AttentionLayer.from_cache_config(1, HQ, w.cfg)
    sid = w.host.add_sequence(70)
    meta_d = w.host.build_prefill_metadata([sid], [70])
    meta = InputMetadata(meta_d["block_tables"], meta_d["context_lens"], meta_d["slot_mappings"],
                         meta_d["max_context_len"], meta_d["is_prefill"], meta_d["max_blocks_per_seq"])
    k, v, q = w.fresh((70, HKV, D)), w.fresh((70, HKV, D)), w.fresh((70, HQ, D))
    out = torch.full((70, HQ, D), 7.0, dtype=torch.bfloat16, device="cuda")
    assert layer.forward(w.bound, out, to_dev(q), to_dev(k), to_dev(v), meta) is False
    torch.cuda.synchronize()
    assert (out == 7.0).all(), "a prefill batch must not write the output"
    write_oracle(w.k_np[1], w.v_np[1], k, v, np.asarray(meta_d["slot_mappings"], dtype=np.int64), HKV)
    assert w.pools_match(1) and w.pools_match(0)
    with pytest.raises(pa.PagedAttnError) as e:
        layer.forward_decode(w.bound, out, to_dev(q), to_dev(k), to_dev(v), meta)
    assert "forward_decode called during prefill phase" in str(e.value)
    # decode
    w.host.extend_sequence(sid, 1)
    md = w.host.build_decode_metadata([sid])
    meta = InputMetadata(md["block_tables"], md["context_lens"], md["slot_mappings"], md["max_context_len"],
                         md["is_prefill"], md["max_blocks_per_seq"])
    k, v, q = w.fresh((1, HKV, D)), w.fresh((1, HKV, D)), w.fresh((1, HQ, D))
    out = torch.zeros(1, HQ, D, dtype=torch.bfloat16, device="cuda")
    assert layer.forward(w.bound, out, to_dev(q), to_dev(k), to_dev(v), meta) is True
    torch.cuda.synchronize()
    w.dev.check_errors()
    write_oracle(w.k_np[1], w.v_np[1], k, v, np.asarray(md["slot_mappings"], dtype=np.int64), HKV)
    assert w.pools_match(1)
    check_attention(bf16_to_f32(to_bits(out)), w.oracle(1, q, [sid]), "layer forward decode")


def test_fp8_scale_integration(cuda_device):
    # paged_kv_cache.rs:1848-1904
    w16 = World([])
    assert not w16.bound.is_fp8_calibrated()
    assert w16.bound.get_layer_scales(0) == (1.0, 1.0)
    assert w16.bound.get_scale_stats() is None
    cfg = host_config(block_size=16, gpu_memory_mb=256, head_size=D, num_kv_heads=4, num_layers=4,
                      use_fp8_cache=1)
    host = PagedKVCacheHost(cfg)
    dev = pa.PagedCache(16, host.total_blocks(), D, 4, num_layers=4, fp8=True)
    b = BoundCache(host, dev)
    for i in range(4):
        assert b.get_layer_scales(i) == (1.0, 1.0)
    b.set_layer_scales(0, 0.5, 0.25)
    b.set_layer_scales(1, 2.0, 1.5)
    assert b.get_layer_scales(0) == (0.5, 0.25) and b.get_layer_scales(1) == (2.0, 1.5)
    assert b.get_scale_stats().num_layers_calibrated == 4
    assert b.is_fp8_calibrated()
    ks, vs = b.get_all_scales()
    assert ks == [0.5, 2.0, 1.0, 1.0] and vs == [0.25, 1.5, 1.0, 1.0]
    b.load_scales([1.0, 1.0, 4.0, 1.0], [1.0, 1.0, 8.0, 1.0])
    assert b.get_layer_scales(2) == (4.0, 8.0)
    # calibrate_layer on device tensors: 448 / max |x| (kv_scale.rs:108-135)
    k = torch.randn(1000, 4, D, device="cuda").to(torch.bfloat16)
    v = (3.0 * torch.randn(1000, 4, D, device="cuda")).to(torch.bfloat16)
    k_s, v_s = b.calibrate_layer_scales(3, k, v, k.numel())
    assert abs(k_s - 448.0 / float(k.abs().max())) < 1e-4 * k_s
    assert abs(v_s - 448.0 / float(v.abs().max())) < 1e-4 * v_s
    assert b.get_layer_scales(3) == (k_s, v_s)
    # the scales reach the kernels: a write through the binding uses the manager's factors
    b.set_layer_scales(0, 1 / 32, 1 / 16)
    sid = host.add_sequence(3)
    slots = host.get_slot_mapping(sid, 0, 3)
    kk, vv = normal_bf16((3, 4, D), 9, 1), normal_bf16((3, 4, D), 9, 2)
    b.update_with_slots(to_dev(kk), to_dev(vv), slots, layer=0)
    torch.cuda.synchronize()
    assert dev.kv_scales(0) == (1 / 32, 1 / 16)


def test_cache_engine_manager_device(cuda_device):
    # cache_engine.rs:222-236 with the pools really allocated: 28 layers, 1 GB
    cfg = host_config(block_size=32, gpu_memory_mb=1024, head_size=128, num_kv_heads=4, num_layers=28)
    kv, cache, bind = C.c_void_p(), C.c_void_p(), C.c_void_p()
    rc = lib().pa_kv_create_bound(C.byref(cfg), 0, 1, C.byref(kv), C.byref(cache), C.byref(bind))
    assert rc == 0, pa.last_error()
    out = pa.PagedAttnConfig()
    assert pa.load_library().pa_cache_get_config(cache, C.byref(out)) == 0
    assert out.num_layers == 28 and out.num_blocks == lib().pa_kv_total_blocks(kv) > 0
    assert lib().pa_kv_num_free_blocks(kv) > 0
    lib().pa_kv_unbind(bind)
    pa.load_library().pa_cache_free(cache)
    lib().pa_kv_destroy(kv)


def test_cpu_block_cache(cuda_device):
    # metal/swap_blocks.rs:258-263
    cache = pa.PagedCache(16, 8, 128, 4)
    cpu = cache.create_cpu_cache()
    assert cpu.num_swapped() == 0 and not cpu.is_swapped(0)


def test_swap_two_layers_through_one_host_cache(cuda_device):
    Hkv, NB = 2, 16
    pools = [(normal_bf16((NB, Hkv, D // X, BS, X), 80 + l, 1), normal_bf16((NB, Hkv, D, BS), 80 + l, 2))
             for l in range(2)]
    kd, vd = [to_dev(p[0]) for p in pools], [to_dev(p[1]) for p in pools]
    cache = pa.PagedCache(BS, NB, D, Hkv, num_layers=2, key_pools=kd, value_pools=vd)
    cpu = cache.create_cpu_cache()
    ids = [3, 9]
    for layer in range(2):
        cache.swap_out(ids, cpu, layer=layer)
    assert cpu.num_swapped() == 2 and cpu.is_swapped(3, layer=1) and cpu.is_swapped(9, layer=0)
    nbytes = Hkv * D * BS * 2
    for layer in range(2):
        for b in ids:
            kp, vp = cpu.block_ptrs(b, layer=layer)
            assert C.string_at(kp, nbytes) == pools[layer][0][b].tobytes()
            assert C.string_at(vp, nbytes) == pools[layer][1][b].tobytes()
    for layer in range(2):
        kd[layer][torch.tensor(ids).cuda()] = 0
        vd[layer][torch.tensor(ids).cuda()] = 0
    cache.swap_in(ids, cpu, layer=1)
    assert cpu.num_swapped() == 2 and not cpu.is_swapped(3, layer=1) and cpu.is_swapped(3, layer=0)
    with pytest.raises(pa.PagedAttnError):
        cache.swap_in(ids, cpu, layer=1)      # layer 1 has nothing left on the host
    cache.swap_in(ids, cpu, layer=0)
    cache.check_errors()
    assert cpu.num_swapped() == 0
    for layer in range(2):
        assert (to_bits(kd[layer]) == pools[layer][0]).all() and (to_bits(vd[layer]) == pools[layer][1]).all()
