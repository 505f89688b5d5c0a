"""The decode step in one launch (pa_decode_step): KV write of the step's tokens by
the attention kernel itself, and the combine of split items by the last CTA to
arrive.  Pool bytes: bit-exact against the oracle's reshape_and_cache over the whole
pool.  Attention: the parity rule of pa_testlib.check_attention against the fp64
oracle."""
import numpy as np
import pytest
import torch

import paged_attn_b200 as pa
from gpu_util import DeviceCase, to_bits
from pa_testlib import BS, D, Case, attention_oracle, bf16_to_f32, check_attention, elems_to_f32

pytestmark = pytest.mark.gpu


def fused_step(dc, case, slots=None):
    f16 = getattr(case, "f16", False)
    out = torch.full((case.S, case.Hq, D), float("nan"),
                     dtype=torch.float16 if f16 else torch.bfloat16, device="cuda")
    dc.cache.decode_step(out, dc.q, dc.k_new, dc.v_new, dc.slots if slots is None else slots,
                         dc.tables, dc.lens, case.S, case.Hq, case.MB, case.scale, dc.ws, dc.ws_bytes)
    torch.cuda.synchronize()
    return elems_to_f32(to_bits(out), f16)


@pytest.mark.parametrize("G,Hkv,f16", [(1, 2, False), (4, 8, False), (8, 8, False), (8, 1, False),
                                       (4, 8, True), (5, 8, False), (7, 4, True), (3, 2, False)])
def test_fused_step_pool_bit_exact_and_attention_parity(cuda_device, G, Hkv, f16):
    # contexts 1, block edges +-1, several long ones that are split across CTAs
    kv = [1, 15, 16, 17, 31, 32, 33, 255, 256, 257, 1000, 4097, 9000, 12001, 5, 700]
    case = Case(kv, [1] * len(kv), G * Hkv, Hkv, 2048, seed=70 + G, f16=f16)
    dc = DeviceCase(case)
    got = fused_step(dc, case)
    dc.cache.check_errors()
    k_ref, v_ref = case.pools_after_write()
    assert (to_bits(dc.k_pool) == k_ref).all(), "K pool differs from the oracle's write"
    assert (to_bits(dc.v_pool) == v_ref).all(), "V pool differs from the oracle's write"
    check_attention(got, attention_oracle(case, k_ref, v_ref, varlen=False), f"fused step G={G}")
    # the same step through write + attention gives the same bits (same kernel, same order)
    dc2 = DeviceCase(case)
    dc2.write()
    two = dc2.attend(varlen=False)
    assert np.array_equal(got, two)


def test_fused_step_negative_slot_and_wrong_slot(cuda_device):
    case = Case([40, 70, 300], [1, 1, 1], 8, 2, 64, seed=61)
    dc = DeviceCase(case)
    slots = dc.slots.clone()
    slots[1] = -1  # no write for sequence 1
    fused_step(dc, case, slots)
    dc.cache.check_errors()
    k_ref, v_ref = case.k_pool.copy(), case.v_pool.copy()
    from pa_testlib import write_oracle
    keep = np.array([0, 2])
    write_oracle(k_ref, v_ref, np.ascontiguousarray(case.k_new[keep]),
                 np.ascontiguousarray(case.v_new[keep]),
                 np.ascontiguousarray(case.slot_mapping[keep]), case.Hkv)
    assert (to_bits(dc.k_pool) == k_ref).all() and (to_bits(dc.v_pool) == v_ref).all()
    # a slot that is not the sequence's last position is refused, not written
    dc = DeviceCase(case)
    slots = dc.slots.clone()
    slots[2] = slots[2] - 1
    fused_step(dc, case, slots)
    with pytest.raises(pa.PagedAttnError) as e:
        dc.cache.check_errors()
    assert e.value.status == 1
    keep = np.array([0, 1])
    k_ref, v_ref = case.k_pool.copy(), case.v_pool.copy()
    write_oracle(k_ref, v_ref, np.ascontiguousarray(case.k_new[keep]),
                 np.ascontiguousarray(case.v_new[keep]),
                 np.ascontiguousarray(case.slot_mapping[keep]), case.Hkv)
    assert (to_bits(dc.k_pool) == k_ref).all() and (to_bits(dc.v_pool) == v_ref).all()


@pytest.mark.parametrize("kind", ["fp8", "block32", "block8", "g16"])
def test_step_falls_back_to_two_launches(cuda_device, kind):
    """Caches the attention kernel cannot write itself: the same entry runs the write
    kernel and then attention; results as through the separate calls."""
    if kind == "fp8":
        from pa_testlib import attention_oracle_fp8, fp8_pools, write_oracle_fp8
        case = Case([300, 33, 2049], [1, 1, 1], 32, 8, 256, seed=5)
        k8, v8 = fp8_pools(case.NB, case.Hkv)
        old = np.ones(len(case.slots_all), dtype=bool)
        old[case.cu_kv[1:] - 1] = False
        ks, vs = 1 / 32, 1 / 16
        write_oracle_fp8(k8, v8, np.ascontiguousarray(case.k_all[old]),
                         np.ascontiguousarray(case.v_all[old]),
                         np.ascontiguousarray(case.slots_all[old]), case.Hkv, ks, vs)
        kd, vd = torch.from_numpy(k8.copy()).cuda(), torch.from_numpy(v8.copy()).cuda()
        cache = pa.PagedCache(BS, case.NB, D, case.Hkv, key_pools=[kd], value_pools=[vd], fp8=True)
        cache.set_kv_scales(ks, vs)
        from gpu_util import to_dev
        out = torch.zeros(case.S, case.Hq, D, dtype=torch.bfloat16, device="cuda")
        ws = torch.empty(cache.workspace_bytes(), dtype=torch.uint8, device="cuda")
        before = pa.kernel_launch_count()
        cache.decode_step(out, to_dev(case.q), to_dev(case.k_new), to_dev(case.v_new),
                          torch.from_numpy(case.slot_mapping).cuda(),
                          torch.from_numpy(case.block_tables).cuda(),
                          torch.from_numpy(case.kv_lens).cuda(), case.S, case.Hq, case.MB,
                          case.scale, ws, ws.numel())
        torch.cuda.synchronize()
        cache.check_errors()
        assert pa.kernel_launch_count() - before == 2
        write_oracle_fp8(k8, v8, case.k_new, case.v_new, case.slot_mapping, case.Hkv, ks, vs)
        assert (kd.cpu().numpy() == k8).all() and (vd.cpu().numpy() == v8).all()
        ref = attention_oracle_fp8(case, k8, v8, ks, vs, varlen=False)
        check_attention(bf16_to_f32(to_bits(out)), ref, "fp8 step")
        return
    if kind == "g16":
        case = Case([300, 33, 2049], [1, 1, 1], 16, 1, 256, seed=6)
    else:
        case = Case([300, 33, 2049, 9], [1, 1, 1, 1], 32, 8, 512, seed=7, bs=32 if kind == "block32" else 8)
    dc = DeviceCase(case)
    before = pa.kernel_launch_count()
    got = fused_step(dc, case)
    dc.cache.check_errors()
    assert pa.kernel_launch_count() - before == 2
    k_ref, v_ref = case.pools_after_write()
    assert (to_bits(dc.k_pool) == k_ref).all() and (to_bits(dc.v_pool) == v_ref).all()
    check_attention(got, attention_oracle(case, k_ref, v_ref, varlen=False), kind)


def test_one_launch_per_decode_step_and_counters_return_to_zero(cuda_device):
    case = Case([9000, 300, 4100, 17, 2500, 12000], [1] * 6, 32, 8, 2048, seed=11)
    dc = DeviceCase(case)
    before = pa.kernel_launch_count()
    a = fused_step(dc, case)
    assert pa.kernel_launch_count() - before == 1
    # twice more on the same handle: the arrival counters must have come back to zero,
    # or split items would be combined too early (garbage) or never (stale rows)
    for _ in range(2):
        b = fused_step(dc, case)
        assert np.array_equal(a, b)
    dc.cache.check_errors()
