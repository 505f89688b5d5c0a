"""GPU parity tests with the other block sizes PagedAttentionConfig accepts
(crates/mlx-paged-attn/src/config.rs:40-45; 32 is its default, :128): 32-token and 8-token
pool blocks.  The KV write bit-exact, decode / verify / chunked-prefill attention within
the attention tolerance of the oracle, on 16-bit and (32-token blocks) FP8 pools, plus the
producer, block copy and swap.  One case also runs with 16-token blocks on the same tokens:
the block size is a layout choice and must not change a result beyond rounding."""
import numpy as np
import pytest
import torch

import paged_attn_b200 as pa
from gpu_util import DeviceCase, to_bits, to_dev
from pa_testlib import (D, X, Case, attention_oracle, attention_oracle_fp8, check_attention,
                        normal_bf16, oracle, p, qk_norm_rope_oracle, check_rotated, write_oracle)
from test_gpu_fp8 import Fp8DeviceCase
from test_gpu_producer import norm_weight, positions_of

pytestmark = pytest.mark.gpu
BS32 = 32
SIZES = [8, 32]


def pool(n32, bs):
    """Pool size in blocks of `bs` tokens that holds what n32 32-token blocks hold."""
    return n32 * 32 // bs


def run_case(case, varlen=True, softcap=1.0):
    dc = DeviceCase(case)
    dc.write()
    torch.cuda.synchronize()
    dc.cache.check_errors()
    k_ref, v_ref = case.pools_after_write()
    assert (to_bits(dc.k_pool) == k_ref).all(), "K pool differs from the oracle"
    assert (to_bits(dc.v_pool) == v_ref).all(), "V pool differs from the oracle"
    got = dc.attend(varlen=varlen, softcap=softcap)
    ref = attention_oracle(case, k_ref, v_ref, softcap=softcap, varlen=varlen)
    return got, ref


@pytest.mark.parametrize("f16", [False, True])
@pytest.mark.parametrize("G,Hkv", [(1, 2), (4, 8), (8, 2), (16, 1), (5, 8), (6, 2)])
@pytest.mark.parametrize("bs", SIZES)
def test_decode_edge_lengths(cuda_device, G, Hkv, f16, bs):
    # lengths around both the 16-token unit and the 32-token block boundaries
    kv = [1, 15, 16, 17, 31, 32, 33, 47, 48, 49, 64, 255, 256, 257, 1000, 4097]
    case = Case(kv, [1] * len(kv), G * Hkv, Hkv, pool(512, bs), seed=131 + G, f16=f16, bs=bs)
    got, ref = run_case(case, varlen=False)
    check_attention(got, ref, f"decode G={G} f16={f16}")


@pytest.mark.parametrize("bs", SIZES)
def test_same_tokens_give_the_same_bits_as_16_token_blocks(cuda_device, bs):
    kv, ql = [700, 64, 1029, 300, 6, 2500, 17], [1, 2, 3, 6, 6, 5, 1]
    c32 = Case(kv, ql, 8, 2, pool(256, bs), seed=132, bs=bs)
    c16 = Case(kv, ql, 8, 2, 512, seed=132)
    assert (c32.q == c16.q).all() and (c32.k_all == c16.k_all).all()
    got32, ref32 = run_case(c32)
    got16, _ = run_case(c16)
    check_attention(got32, ref32, f"verify widths, {bs}-token blocks")
    if bs == 8:
        # the same 16-token units are multiplied in the same order: the same bits
        assert (got32 == got16).all()
    else:
        # a warp takes a whole 32-token block (both 16-token halves) from one stage, so the
        # units are shared out among the warps differently: not the same bits as with
        # 16-token blocks, the same parity bound (above) and the same bits run to run
        again, _ = run_case(c32)
        assert (again == got32).all()
    got_cap, ref_cap = run_case(c32, softcap=30.0)
    check_attention(got_cap, ref_cap, f"softcap, {bs}-token blocks")


@pytest.mark.parametrize("bs", SIZES)
def test_long_contexts_are_split_across_ctas(cuda_device, bs):
    kv = [20000, 9000, 33, 15000]
    case = Case(kv, [1] * 4, 32, 8, pool(2048, bs), seed=133, bs=bs)
    got, ref = run_case(case, varlen=False)
    check_attention(got, ref, f"long decode, {bs}-token blocks")


@pytest.mark.parametrize("bs", SIZES)
def test_chunked_prefill_with_decode_and_verify(cuda_device, bs):
    # chunks that start and end inside blocks and units; a decode token and a verify
    # sequence in the same call (tile kernel side by side with 32-token blocks; chunks in
    # pieces through the split-KV kernel with 8-token blocks)
    kv = [1500, 300, 77, 2049, 40, 33]
    ql = [700, 300, 50, 1, 3, 33]
    case = Case(kv, ql, 16, 4, pool(256, bs), seed=134, bs=bs)
    launches = pa.load_library().pa_kernel_launch_count()
    got, ref = run_case(case)
    check_attention(got, ref, f"chunked prefill, {bs}-token blocks")
    assert pa.load_library().pa_kernel_launch_count() - launches >= 4  # write, tile, split-KV, merge
    got_cap, ref_cap = run_case(case, softcap=50.0)
    check_attention(got_cap, ref_cap, f"chunked prefill softcap, {bs}-token blocks")


@pytest.mark.parametrize("bs", SIZES)
def test_prefill_longer_than_the_staged_table(cuda_device, bs):
    # more than 2048 units per sequence: ids beyond the staged table are read from memory
    case = Case([40000], [300], 8, 1, pool(1280, bs), seed=135, bs=bs)
    got, ref = run_case(case)
    check_attention(got, ref, f"40k-token context prefill chunk, {bs}-token blocks")


@pytest.mark.parametrize("bs", SIZES)
def test_out_of_range_block_and_slot_are_reported(cuda_device, bs):
    case = Case([100, 50], [1, 1], 4, 2, pool(16, bs), seed=136, bs=bs)
    dc = DeviceCase(case)
    dc.write()
    torch.cuda.synchronize()
    dc.cache.check_errors()
    bad = dc.slots.clone()
    bad[0] = case.NB * bs  # first slot past the pool
    dc.cache.reshape_and_cache(dc.k_new, dc.v_new, bad, 2, case.Hkv * D, case.Hkv * D)
    torch.cuda.synchronize()
    with pytest.raises(pa.PagedAttnError) as e:
        dc.cache.check_errors()
    assert e.value.status == 4
    ok = dc.slots.clone()
    ok[0] = case.NB * bs - 1
    dc.cache.reshape_and_cache(dc.k_new, dc.v_new, ok, 2, case.Hkv * D, case.Hkv * D)
    torch.cuda.synchronize()
    dc.cache.check_errors()
    dc.tables[0, 1] = case.NB
    out = torch.empty((2, case.Hq, D), dtype=torch.bfloat16, device="cuda")
    dc.cache.decode(out, dc.q, dc.tables, dc.lens, 2, case.Hq, case.MB, case.scale, dc.ws, dc.ws_bytes)
    torch.cuda.synchronize()
    with pytest.raises(pa.PagedAttnError) as e:
        dc.cache.check_errors()
    assert e.value.status == 4


@pytest.mark.parametrize("f16", [False, True])
def test_fp8_pools(cuda_device, f16):
    kv = [1, 16, 17, 32, 33, 49, 255, 1000, 4097, 700, 64]
    ql = [1, 1, 1, 1, 1, 1, 1, 1, 1, 3, 6]
    case = Case(kv, ql, 8, 2, 256, seed=137, f16=f16, bs=BS32)
    for exact in (False, True):
        dc = Fp8DeviceCase(case, 0.37, 0.6, exact=exact)
        k_ref, v_ref = dc.write_and_check()
        got = dc.attend()
        ref = attention_oracle_fp8(case, k_ref, v_ref, 0.37, 0.6)
        check_attention(got, ref, f"fp8, 32-token blocks, f16={f16} exact={exact}")


def test_fp8_long_chunk_on_32_token_blocks(cuda_device):
    case = Case([900, 130, 40], [200, 130, 1], 8, 2, 64, seed=138, bs=BS32)
    dc = Fp8DeviceCase(case, 0.5, 0.5, exact=False)
    k_ref, v_ref = dc.write_and_check()
    got = dc.attend()
    ref = attention_oracle_fp8(case, k_ref, v_ref, 0.5, 0.5)
    check_attention(got, ref, "fp8 long chunk, 32-token blocks")


@pytest.mark.parametrize("bs", SIZES)
def test_producer_writes_the_blocks(cuda_device, bs):
    case = Case([150, 77, 40, 33], [100, 77, 1, 1], 8, 2, pool(32, bs), seed=139, bs=bs)
    dc = DeviceCase(case)
    wq, wk = norm_weight(8, False), norm_weight(9, False)
    pos = positions_of(case)
    q = to_dev(case.q)
    dc.cache.qk_norm_rope_and_cache(q, q, dc.k_new, dc.v_new, to_dev(wq), to_dev(wk), 1e-6,
                                    torch.from_numpy(pos).cuda(), 1.0e6, D, dc.slots, case.total_q,
                                    case.Hq, case.Hq * D, case.Hq * D, case.Hkv * D, case.Hkv * D)
    torch.cuda.synchronize()
    dc.cache.check_errors()
    q_ref, q_bound = qk_norm_rope_oracle(case.q, wq, 1e-6, pos, 1.0e6, D)
    k_ref, k_bound = qk_norm_rope_oracle(case.k_new, wk, 1e-6, pos, 1.0e6, D)
    check_rotated(to_bits(q).reshape(case.total_q, case.Hq, D), q_ref, q_bound, False, "rotated queries")
    k_got, v_got = to_bits(dc.k_pool), to_bits(dc.v_pool)
    blk, off = case.slot_mapping // bs, case.slot_mapping % bs
    rows = np.ascontiguousarray(k_got[blk, :, :, off, :].reshape(case.total_q, case.Hkv, D))
    check_rotated(rows, k_ref, k_bound, False, "rotated keys in the pool")
    k_exp, v_exp = case.k_pool.copy(), case.v_pool.copy()
    write_oracle(k_exp, v_exp, k_ref, case.v_new, case.slot_mapping, case.Hkv)
    assert (v_got == v_exp).all(), "V pool differs from the oracle"
    untouched = np.ones(k_exp.shape, dtype=bool)
    untouched[blk, :, :, off, :] = False
    assert (k_got[untouched] == case.k_pool[untouched]).all(), "K pool changed off the slots"


@pytest.mark.parametrize("bs", SIZES)
def test_copy_and_swap_move_whole_blocks(cuda_device, bs):
    import ctypes as C
    Hkv, NB = 4, 32
    k_pool = normal_bf16((NB, Hkv, D // X, bs, X), 140, 1)
    v_pool = normal_bf16((NB, Hkv, D, bs), 140, 2)
    kd, vd = to_dev(k_pool), to_dev(v_pool)
    cache = pa.PagedCache(bs, NB, D, Hkv, key_pools=[kd], value_pools=[vd])
    pairs = np.array([[0, 9], [5, 31], [7, 8]], dtype=np.int64)
    cache.copy_blocks(torch.from_numpy(pairs).cuda(), 3)
    torch.cuda.synchronize()
    cache.check_errors()
    oracle().oracle_copy_blocks(p(k_pool), p(v_pool), p(pairs), 3, Hkv * D * bs)
    assert (to_bits(kd) == k_pool).all() and (to_bits(vd) == v_pool).all()
    cpu = cache.create_cpu_cache()
    ids = [3, 31, 0]
    cache.swap_out(ids, cpu)
    nbytes = Hkv * D * bs * 2
    for b in ids:
        kp, vp = cpu.block_ptrs(b)
        assert C.string_at(kp, nbytes) == k_pool[b].tobytes()
        assert C.string_at(vp, nbytes) == v_pool[b].tobytes()
    kd[torch.tensor(ids).cuda()] = 0
    vd[torch.tensor(ids).cuda()] = 0
    cache.swap_in(ids, cpu)
    cache.check_errors()
    assert (to_bits(kd) == k_pool).all() and (to_bits(vd) == v_pool).all()


def test_fp8_with_8_token_blocks_is_refused_like_the_reference(cuda_device):
    # crates/mlx-paged-attn/src/config.rs:71-76, test_fp8_validation (:218-236)
    with pytest.raises(pa.PagedAttnError) as e:
        pa.PagedCache(8, 16, D, 2, fp8=True)
    assert e.value.status == 1 and "block_size 16 or 32" in str(e.value)


def test_long_chunk_on_8_token_blocks_needs_host_lengths(cuda_device):
    case = Case([200], [100], 8, 2, 32, seed=141, bs=8)
    dc = DeviceCase(case)
    dc.write()
    out = torch.empty((100, 8, D), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(pa.PagedAttnError) as e:
        dc.cache.varlen(out, dc.q, dc.tables, dc.lens, case.cu_q, 1, 8, case.MB, case.scale, dc.ws,
                        dc.ws_bytes)
    assert e.value.status == 1 and "context_lens_host" in str(e.value)
    torch.cuda.synchronize()
