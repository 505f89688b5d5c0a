"""End to end on the GPU: the hybrid scheduler's batches (prefill chunks, decode and
speculative-verify steps mixed) drive the KV write and the variable-length attention
through the C ABI for many steps; every query row that will be kept is compared with
float64 dense causal attention over the sequence's true keys and values.  Rejected draft
tokens write K/V that later steps overwrite, so the test also covers roll-back."""
import numpy as np
import pytest
import torch

import paged_attn_b200 as pa
from gpu_util import to_bits, to_dev
from paged_attn_b200.host import HybridScheduler, PagedKVCacheHost, host_config
from pa_testlib import (BS, D, X, X8, bf16_to_f32, check_attention, fp8_pools, normal_bf16, oracle,
                        write_oracle_fp8)

pytestmark = pytest.mark.gpu


def dense_rows(q, k, v, positions, G, scale):
    """float64 attention of query rows at `positions` over keys [0, position]."""
    out = np.zeros((len(positions), q.shape[1], D))
    for i, pos in enumerate(positions):
        for hq in range(q.shape[1]):
            h = hq // G
            logits = (k[:pos + 1, h] @ q[pos, hq]) * scale
            w = np.exp(logits - logits.max())
            out[i, hq] = (w / w.sum()) @ v[:pos + 1, h]
    return out


def through_fp8(x_bits, scale):
    """[L, Hkv, D] bf16 bits -> float64 values as an FP8 cache with this scale holds them
    (written by the oracle into a scratch pool, decoded by the format's table)."""
    L, Hkv, _ = x_bits.shape
    nb = (L + BS - 1) // BS
    k8, v8 = fp8_pools(nb, Hkv)
    write_oracle_fp8(k8, v8, x_bits, x_bits, np.arange(L, dtype=np.int64), Hkv, scale, scale)
    table = np.array([oracle().oracle_fp8_e4m3_decode(c) for c in range(256)], dtype=np.float64)
    vals = table[v8] * scale                       # [nb, Hkv, D, BS]
    return vals.transpose(0, 3, 1, 2).reshape(nb * BS, Hkv, D)[:L]


@pytest.mark.parametrize("fp8,bs", [(False, 16), (True, 16), (False, 32), (True, 32), (False, 8)])
def test_scheduler_drives_the_kernels(cuda_device, fp8, bs):
    Hq, Hkv, L = 16, 4, 400
    G = Hq // Hkv
    rng = np.random.Generator(np.random.PCG64(5))
    cfg = host_config(block_size=bs, gpu_memory_mb=256, head_size=D, num_kv_heads=Hkv, num_layers=1,
                      max_seq_len=512)
    kv_host = PagedKVCacheHost(cfg)
    NB = kv_host.total_blocks()
    kv_scale = 1.0 / 16
    if fp8:
        # prefill chunks of 64 tokens go to the tile kernel's FP8 path (with 8-token blocks,
        # further down, to the split-KV kernel in pieces of 24/G = 6 tokens)
        k_pool = torch.zeros(NB, Hkv, D // X8, bs, X8, dtype=torch.uint8, device="cuda")
        v_pool = torch.zeros(NB, Hkv, D, bs, dtype=torch.uint8, device="cuda")
    else:
        k_pool = torch.zeros(NB, Hkv, D // X, bs, X, dtype=torch.bfloat16, device="cuda")
        v_pool = torch.zeros(NB, Hkv, D, bs, dtype=torch.bfloat16, device="cuda")
    cache = pa.PagedCache(bs, NB, D, Hkv, key_pools=[k_pool], value_pools=[v_pool], fp8=fp8)
    if fp8:
        cache.set_kv_scales(kv_scale, kv_scale)
        cache.fp8_set_exact_decode(False)   # zero-filled pools, in-range values
    ws = torch.empty(cache.workspace_bytes(), dtype=torch.uint8, device="cuda")
    sched = HybridScheduler(bs, prefill_chunk_size=64, max_tokens_per_step=160, max_prefill_per_step=2,
                            max_batch_size=8, eos_token_id=1 << 30)
    prompts = {"r0": 20, "r1": 150, "r2": 300, "r3": 65, "r4": 33}
    true_q, true_k, true_v, junk_k = {}, {}, {}, {}
    for i, (name, plen) in enumerate(prompts.items()):
        sched.add_request(name, list(range(plen)), 24)
        true_q[name] = normal_bf16((L, Hq, D), 100 + i, 1)
        true_k[name] = normal_bf16((L, Hkv, D), 100 + i, 2)
        true_v[name] = normal_bf16((L, Hkv, D), 100 + i, 3)
        junk_k[name] = normal_bf16((L, Hkv, D), 100 + i, 4)
    # what the cache holds of the true keys and values
    if fp8:
        held_k = {n: through_fp8(true_k[n], kv_scale) for n in prompts}
        held_v = {n: through_fp8(true_v[n], kv_scale) for n in prompts}
    else:
        held_k = {n: bf16_to_f32(true_k[n]).astype(np.float64) for n in prompts}
        held_v = {n: bf16_to_f32(true_v[n]).astype(np.float64) for n in prompts}
    scale = 1.0 / np.sqrt(D)
    checked, kinds, steps = 0, set(), 0
    while not sched.is_empty() and steps < 200:
        steps += 1
        b = sched.schedule_step(kv_host)
        assert b is not None
        n, total = len(b["entries"]), b["total_tokens"]
        q = np.zeros((total, Hq, D), dtype=np.uint16)
        k = np.zeros((total, Hkv, D), dtype=np.uint16)
        v = np.zeros((total, Hkv, D), dtype=np.uint16)
        outputs, keep = [], []     # keep: (row in batch, request, position)
        for i, e in enumerate(b["entries"]):
            name, r0 = e["request_id"], b["cu_q_lens"][i]
            first = e["kv_len"] - e["q_len"]
            accepted = 0
            if e["kind"] == "verify":
                accepted = int(rng.integers(0, e["q_len"]))          # 0 .. k drafts accepted
            for j in range(e["q_len"]):
                pos = first + j
                good = e["kind"] != "verify" or j <= accepted
                q[r0 + j] = true_q[name][pos]
                k[r0 + j] = true_k[name][pos] if good else junk_k[name][pos]
                v[r0 + j] = true_v[name][pos] if good else junk_k[name][pos]
                if good:
                    keep.append((r0 + j, name, pos))
            kinds.add(e["kind"])
            if e["needs_sample"]:
                outputs.append((e["seq_id"], accepted, 1000 + steps, False))
        out = torch.full((total, Hq, D), float("nan"), dtype=torch.bfloat16, device="cuda")
        slots = torch.tensor(b["slot_mapping"], dtype=torch.int64, device="cuda")
        tables = torch.tensor(b["block_tables"], dtype=torch.int32, device="cuda").view(n, -1)
        lens = torch.tensor(b["context_lens"], dtype=torch.int32, device="cuda")
        cu = np.asarray(b["cu_q_lens"], dtype=np.int32)
        cache.reshape_and_cache(to_dev(k), to_dev(v), slots, total, Hkv * D, Hkv * D)
        cache.varlen(out, to_dev(q), tables, lens, cu, n, Hq, b["max_blocks_per_seq"], scale, ws, ws.numel(),
                     max_context_len=b["max_context_len"],
                     context_lens_host=np.asarray(b["context_lens"], dtype=np.int32)
                     if fp8 or bs == 8 else None)
        torch.cuda.synchronize()
        cache.check_errors()
        got = bf16_to_f32(to_bits(out))
        for name in {kname for _, kname, _ in keep}:
            rows = [(r, p_) for r, kname, p_ in keep if kname == name]
            ref = dense_rows(bf16_to_f32(true_q[name]).astype(np.float64), held_k[name],
                             held_v[name], [p_ for _, p_ in rows], G, scale)
            check_attention(np.stack([got[r] for r, _ in rows]), ref, f"step {steps} {name}")
            checked += len(rows)
        sched.process_outputs(outputs, kv_host)
        # next step: propose drafts for some of the sequences now in decode
        for e in b["entries"]:
            if e["needs_sample"] and rng.random() < 0.6:
                try:
                    sched.set_draft_tokens(e["seq_id"], [7] * int(rng.integers(1, 5)))
                except pa.PagedAttnError:
                    pass    # the sequence has just finished
    assert sched.is_empty() and kinds == {"prefill", "decode", "verify"}
    assert kv_host.num_sequences() == 0 and kv_host.num_free_blocks() == NB
    assert len(sched.get_completed()) == len(prompts) and checked > 500
