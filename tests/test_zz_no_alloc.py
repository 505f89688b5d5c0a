"""The decode entry for callers that cannot allocate device memory
(pa_paged_attention_decode_static) must give what the ordinary entry gives.

It keeps its split-KV partial results in an array inside the library image
rather than in a workspace the caller allocates, and every call shares that
array, so the check is made on two different batches back to back: if the
second call picked up anything the first one left behind, it would show.
This file sorts last on purpose, so a failure here cannot hide another test's.
"""
import numpy as np
import pytest
import torch

import paged_attn_b200 as pa
from gpu_util import DeviceCase, to_bits, to_dev
from pa_testlib import (BS, Case, D, attention_oracle, attention_oracle_fp8, bf16_to_f32, check_attention,
                        fp8_pools, write_oracle_fp8)

pytestmark = pytest.mark.gpu


def both_entries(case):
    dc = DeviceCase(case)
    dc.write()
    want = torch.full((case.S, case.Hq, D), float("nan"), dtype=torch.bfloat16, device="cuda")
    got = torch.full_like(want, float("nan"))
    dc.cache.decode(want, dc.q, dc.tables, dc.lens, case.S, case.Hq, case.MB, case.scale, dc.ws,
                    dc.ws_bytes)
    dc.cache.decode_static(got, dc.q, dc.tables, dc.lens, case.S, case.Hq, case.MB, case.scale)
    torch.cuda.synchronize()
    dc.cache.check_errors()
    # and against the fp64 oracle, by the parity rule every attention test uses
    k_ref, v_ref = case.pools_after_write()
    check_attention(bf16_to_f32(to_bits(got)), attention_oracle(case, k_ref, v_ref, varlen=False),
                    "static-scratch entry vs oracle")
    return bf16_to_f32(to_bits(got)), bf16_to_f32(to_bits(want))


def test_static_scratch_entry_matches_workspace_entry(cuda_device):
    # first batch: long contexts, so that items are split across CTAs and the
    # partial slots are really used
    first = Case([9000, 300, 4100, 17, 2500, 12000], [1] * 6, 32, 8, 2048, seed=101)
    got, want = both_entries(first)
    assert np.isfinite(want).all()
    # same kernel, same partition, same merge order: the results are identical,
    # which is well inside the 2e-2 / 1e-2 tolerance the parity tests use
    assert np.array_equal(got, want)
    # second batch right after, different shapes and lengths, same shared scratch
    second = Case([700, 16000, 33, 5000], [1] * 4, 64, 8, 2048, seed=102)
    got2, want2 = both_entries(second)
    assert np.isfinite(want2).all()
    assert np.array_equal(got2, want2)
    assert np.abs(want2).max() > 0


def test_static_scratch_entry_on_an_fp8_cache(cuda_device):
    """On an E4M3 cache the workspace entry runs its narrow kernel on two CTAs per SM;
    the library-resident scratch has slots for one per SM, so this entry takes the other
    partition of the same work: not the same bits, the same parity bound."""
    case = Case([9000, 300, 4100, 17, 2500, 12000], [1] * 6, 32, 8, 2048, seed=103)
    k8, v8 = fp8_pools(case.NB, case.Hkv)
    ks, vs = 1 / 32, 1 / 16
    write_oracle_fp8(k8, v8, case.k_all, case.v_all, case.slots_all, case.Hkv, ks, vs)
    ref = attention_oracle_fp8(case, k8, v8, ks, vs, varlen=False)
    kd, vd = torch.from_numpy(k8).cuda(), torch.from_numpy(v8).cuda()
    cache = pa.PagedCache(BS, case.NB, D, case.Hkv, key_pools=[kd], value_pools=[vd], fp8=True)
    cache.set_kv_scales(ks, vs)
    q = to_dev(case.q)
    tables, lens = torch.from_numpy(case.block_tables).cuda(), torch.from_numpy(case.kv_lens).cuda()
    ws = torch.empty(cache.workspace_bytes(), dtype=torch.uint8, device="cuda")
    for call in range(2):   # twice in a row on the shared scratch
        got = torch.full((case.S, case.Hq, D), float("nan"), dtype=torch.bfloat16, device="cuda")
        want = torch.full_like(got, float("nan"))
        cache.decode_static(got, q, tables, lens, case.S, case.Hq, case.MB, case.scale)
        cache.decode(want, q, tables, lens, case.S, case.Hq, case.MB, case.scale, ws, ws.numel())
        torch.cuda.synchronize()
        cache.check_errors()
        check_attention(bf16_to_f32(to_bits(got)), ref, f"static entry, FP8 cache, call {call}")
        check_attention(bf16_to_f32(to_bits(want)), ref, f"workspace entry, FP8 cache, call {call}")


def test_static_scratch_entry_with_small_heads(cuda_device):
    """Head size 64: the workspace entry runs its narrow kernel on two CTAs per SM, this entry
    on one (the scratch has slots for one per SM): another partition of the same work, the
    same parity bound, twice in a row on the shared scratch."""
    case = Case([9000, 300, 4100, 17, 2500, 12000], [1] * 6, 32, 8, 2048, seed=104, head_size=64)
    dc = DeviceCase(case)
    dc.write()
    k_ref, v_ref = case.pools_after_write()
    ref = attention_oracle(case, k_ref, v_ref, varlen=False)
    for call in range(2):
        got = torch.full((case.S, case.Hq, 64), float("nan"), dtype=torch.bfloat16, device="cuda")
        dc.cache.decode_static(got, dc.q, dc.tables, dc.lens, case.S, case.Hq, case.MB, case.scale)
        torch.cuda.synchronize()
        dc.cache.check_errors()
        check_attention(bf16_to_f32(to_bits(got)), ref, f"static entry, head size 64, call {call}")
