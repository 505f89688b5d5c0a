"""GPU parity tests of the producer (QK norm + rotary embedding + KV write in one
launch) against the CPU oracle: values bit-exact, rotated queries and keys within one
unit in the last place with at least 99 % identical (pa_testlib.check_rotated), the
pool untouched elsewhere, and the producer -> attention chain within the attention
tolerance of the oracle chain."""
import numpy as np
import pytest
import torch

import paged_attn_b200 as pa
from gpu_util import DeviceCase, to_bits, to_dev
from pa_testlib import (BS, CANARY, D, Case, attention_oracle, bf16_to_f32, check_attention,
                        check_rotated, f32_to_bf16, normal_bf16, normal_f16, qk_norm_rope_oracle,
                        write_oracle)

pytestmark = pytest.mark.gpu


def norm_weight(seed, f16):
    wf = 1.0 + 0.25 * bf16_to_f32(normal_bf16((D,), seed, 9))
    return wf.astype(np.float16).view(np.uint16) if f16 else f32_to_bf16(wf)


def positions_of(case):
    """Rotary position of each new token: its index in its sequence."""
    pos = np.empty(case.total_q, dtype=np.int32)
    for s in range(case.S):
        q0, q1 = case.cu_q[s], case.cu_q[s + 1]
        pos[q0:q1] = case.kv_lens[s] - (q1 - q0) + np.arange(q1 - q0)
    return pos


def token_rows(k_pool_bits, slots, Hkv):
    """[T, Hkv, D] rows of the K pool [NB, Hkv, D/8, BS, 8] at `slots`."""
    blk, off = slots // BS, slots % BS
    return np.ascontiguousarray(k_pool_bits[blk, :, :, off, :].reshape(len(slots), Hkv, D))


def run_producer(case, wq, wk, eps, base, dims, in_place, q_pad=0):
    f16 = case.f16
    dc = DeviceCase(case)
    T = case.total_q
    pos = positions_of(case)
    q_row = case.Hq * D + q_pad
    q_buf = torch.zeros((T, q_row), dtype=torch.float16 if f16 else torch.bfloat16, device="cuda")
    q_buf[:, :case.Hq * D] = to_dev(case.q, f16).view(T, -1)
    q_out = q_buf if in_place else torch.full_like(q_buf, float("nan"))
    wq_d = to_dev(wq, f16) if wq is not None else None
    wk_d = to_dev(wk, f16) if wk is not None else None
    pos_d = torch.from_numpy(pos).cuda()
    dc.cache.qk_norm_rope_and_cache(q_out, q_buf, dc.k_new, dc.v_new, wq_d, wk_d, eps, pos_d, base,
                                    dims, dc.slots, T, case.Hq, q_row, q_row, case.Hkv * D,
                                    case.Hkv * D)
    torch.cuda.synchronize()
    dc.cache.check_errors()
    # oracle side
    q_ref, q_bound = qk_norm_rope_oracle(case.q, wq, eps, pos, base, dims, f16)
    k_ref, k_bound = qk_norm_rope_oracle(case.k_new, wk, eps, pos, base, dims, f16)
    q_got = to_bits(q_out).reshape(T, q_row)[:, :case.Hq * D].reshape(T, case.Hq, D)
    check_rotated(q_got, q_ref, q_bound, f16, "rotated queries")
    k_pool_got, v_pool_got = to_bits(dc.k_pool), to_bits(dc.v_pool)
    check_rotated(token_rows(k_pool_got, case.slot_mapping, case.Hkv), k_ref, k_bound, f16,
                  "rotated keys in the pool")
    # values bit-exact, and nothing outside the written slots moved
    k_exp, v_exp = case.k_pool.copy(), case.v_pool.copy()
    write_oracle(k_exp, v_exp, k_ref, case.v_new, case.slot_mapping, case.Hkv)
    assert (v_pool_got == v_exp).all(), "V pool differs from the oracle"
    blk, off = case.slot_mapping // BS, case.slot_mapping % BS
    untouched = np.ones(k_exp.shape, dtype=bool)
    untouched[blk, :, :, off, :] = False
    assert (k_pool_got[untouched] == case.k_pool[untouched]).all(), "K pool changed off the slots"
    return dc, q_out, q_row, k_exp, v_exp, q_ref


@pytest.mark.parametrize("f16", [False, True])
def test_decode_batch_norm_and_rope(cuda_device, f16):
    kv = [1, 17, 300, 4097, 33000, 16, 2049]
    case = Case(kv, [1] * len(kv), 16, 4, 4096, seed=61, f16=f16)
    run_producer(case, norm_weight(1, f16), norm_weight(2, f16), 1e-6, 1.0e6, D, in_place=True)


def test_prefill_chunks_in_place_and_strided(cuda_device):
    # two chunks that start and end inside blocks, one decode token, padded query rows
    case = Case([150, 77, 40], [100, 77, 1], 8, 2, 64, seed=62)
    run_producer(case, norm_weight(3, False), norm_weight(4, False), 1e-5, 1.0e4, D, in_place=True,
                 q_pad=64)


def test_partial_rotary_without_norm(cuda_device):
    case = Case([90, 12], [20, 12], 4, 4, 32, seed=63)
    dc, q_out, q_row, *_ = run_producer(case, None, None, 1e-6, 1.0e4, 64, in_place=False)
    # elements beyond rope_dims pass through bit for bit when there is no norm
    got = to_bits(q_out).reshape(case.total_q, q_row)[:, :case.Hq * D].reshape(-1, case.Hq, D)
    assert (got[..., 64:] == case.q[..., 64:]).all()


def test_only_query_norm(cuda_device):
    case = Case([64, 65], [1, 1], 8, 1, 16, seed=64)
    run_producer(case, norm_weight(5, False), None, 1e-6, 1.0e6, D, in_place=False)


def test_negative_slots_are_skipped(cuda_device):
    case = Case([40, 41, 42], [1, 1, 1], 4, 2, 16, seed=65)
    case.slot_mapping = case.slot_mapping.copy()
    case.slot_mapping[1] = -1
    dc = DeviceCase(case)
    pos = torch.from_numpy(positions_of(case)).cuda()
    q = to_dev(case.q)
    dc.cache.qk_norm_rope_and_cache(q, q, dc.k_new, dc.v_new, None, None, 1e-6, pos, 1e6, D,
                                    dc.slots, 3, case.Hq, case.Hq * D, case.Hq * D, case.Hkv * D,
                                    case.Hkv * D)
    torch.cuda.synchronize()
    dc.cache.check_errors()
    blk, off = int(case.slots_all[case.cu_kv[2] - 1]) // BS, int(case.slots_all[case.cu_kv[2] - 1]) % BS
    assert (to_bits(dc.v_pool)[blk, :, :, off] == CANARY).all(), "skipped token was written"


def test_producer_then_attention_matches_oracle_chain(cuda_device):
    """The pair the producer feeds: rotated queries attend the pool that holds rotated
    keys (the prefix rotated by the oracle, the new tokens by the kernel)."""
    kv = [513, 64, 1000, 2048, 31]
    ql = [1, 1, 5, 1, 31]
    case = Case(kv, ql, 16, 4, 512, seed=66, prefill=False)
    wq, wk = norm_weight(6, False), norm_weight(7, False)
    # prefix keys rotated by the oracle at their own positions, written to the pool
    old = np.ones(len(case.slots_all), dtype=bool)
    pos_all = np.empty(len(case.slots_all), dtype=np.int32)
    for s in range(case.S):
        pos_all[case.cu_kv[s]:case.cu_kv[s + 1]] = np.arange(kv[s])
        old[case.cu_kv[s + 1] - ql[s]:case.cu_kv[s + 1]] = False
    k_rot_all, _ = qk_norm_rope_oracle(case.k_all, wk, 1e-6, pos_all, 1e6, D)
    write_oracle(case.k_pool, case.v_pool, np.ascontiguousarray(k_rot_all[old]),
                 np.ascontiguousarray(case.v_all[old]), np.ascontiguousarray(case.slots_all[old]),
                 case.Hkv)
    dc, q_out, q_row, k_exp, v_exp, q_ref = run_producer(case, wq, wk, 1e-6, 1.0e6, D, in_place=True)
    out = torch.full((case.total_q, case.Hq, D), float("nan"), dtype=torch.bfloat16, device="cuda")
    dc.cache.varlen(out, q_out, dc.tables, dc.lens, case.cu_q, case.S, case.Hq, case.MB, case.scale,
                    dc.ws, dc.ws_bytes, context_lens_host=case.kv_lens)
    torch.cuda.synchronize()
    dc.cache.check_errors()
    case.q = q_ref
    ref = attention_oracle(case, k_exp, v_exp)
    check_attention(bf16_to_f32(to_bits(out)), ref, "producer -> attention")


def test_producer_rejects_bad_arguments(cuda_device):
    case = Case([20], [1], 4, 2, 16, seed=67)
    dc = DeviceCase(case)
    q = to_dev(case.q)
    pos = torch.zeros(1, dtype=torch.int32, device="cuda")

    def call(**kw):
        a = dict(dims=D, hq=case.Hq, q_stride=case.Hq * D, base=1e6)
        a.update(kw)
        dc.cache.qk_norm_rope_and_cache(q, q, dc.k_new, dc.v_new, None, None, 1e-6, pos, a["base"],
                                        a["dims"], dc.slots, 1, a["hq"], a["q_stride"],
                                        case.Hq * D, case.Hkv * D, case.Hkv * D)
    for bad in (dict(dims=63), dict(dims=D + 2), dict(hq=3), dict(q_stride=case.Hq * D - 8),
                dict(base=0.0)):
        with pytest.raises(pa.PagedAttnError) as e:
            call(**bad)
        assert e.value.status == 1, bad
    call()  # and the good call still works afterwards
    torch.cuda.synchronize()
    dc.cache.check_errors()
