"""GPU parity tests of the FP8 (E4M3) KV cache: the write bit-exact against the oracle
(the reference's own byte format, out-of-range inputs included), attention over the FP8
pools within the attention tolerance of the fp64 oracle on the same bytes, every byte
code decoded the way the format defines, block copy and swap on the smaller blocks."""
import numpy as np
import pytest
import torch

import paged_attn_b200 as pa
from gpu_util import to_bits, to_dev
from pa_testlib import (BS, D, X8, Case, attention_oracle_fp8, check_attention, elems_to_f32,
                        fp8_pools, normal_bf16, oracle, write_oracle_fp8)

pytestmark = pytest.mark.gpu


class Fp8DeviceCase:
    def __init__(self, case, k_scale, v_scale, k8=None, v8=None, exact=True):
        """`exact`: decoding variant of the attention kernels.  Wrapped pools start exact
        (their contents are unknown to the library); False states that they hold no byte
        with exponent field 15, which is true of every pool the oracle filled from
        in-range values."""
        self.case, self.ks, self.vs = case, k_scale, v_scale
        if k8 is None:
            k8, v8 = fp8_pools(case.NB, case.Hkv, fill=0x7F, bs=case.bs)  # NaN codes where nothing was written
            old = np.ones(len(case.slots_all), dtype=bool)
            for s in range(case.S):
                old[case.cu_kv[s + 1] - case.q_lens[s]:case.cu_kv[s + 1]] = False
            write_oracle_fp8(k8, v8, np.ascontiguousarray(case.k_all[old]),
                             np.ascontiguousarray(case.v_all[old]),
                             np.ascontiguousarray(case.slots_all[old]), case.Hkv, k_scale, v_scale,
                             case.f16)
        self.k8_host, self.v8_host = k8, v8
        self.k_pool = torch.from_numpy(k8).cuda()
        self.v_pool = torch.from_numpy(v8).cuda()
        self.cache = pa.PagedCache(case.bs, case.NB, D, case.Hkv, dtype=0 if case.f16 else 1,
                                   key_pools=[self.k_pool], value_pools=[self.v_pool], fp8=True)
        self.cache.set_kv_scales(k_scale, v_scale)
        if not exact:
            self.cache.fp8_set_exact_decode(False)
        self.q = to_dev(case.q, case.f16)
        self.k_new, self.v_new = to_dev(case.k_new, case.f16), to_dev(case.v_new, case.f16)
        self.slots = torch.from_numpy(case.slot_mapping).cuda()
        self.tables = torch.from_numpy(case.block_tables).cuda()
        self.lens = torch.from_numpy(case.kv_lens).cuda()
        self.ws_bytes = self.cache.workspace_bytes()
        self.ws = torch.empty(self.ws_bytes, dtype=torch.uint8, device="cuda")
        self.ws.view(torch.int16).fill_(0x7FFF)

    def write_and_check(self):
        c = self.case
        self.cache.reshape_and_cache(self.k_new, self.v_new, self.slots, len(c.slot_mapping),
                                     c.Hkv * D, c.Hkv * D)
        torch.cuda.synchronize()
        self.cache.check_errors()
        k_ref, v_ref = self.k8_host.copy(), self.v8_host.copy()
        write_oracle_fp8(k_ref, v_ref, c.k_new, c.v_new, c.slot_mapping, c.Hkv, self.ks, self.vs,
                         c.f16)
        assert (self.k_pool.cpu().numpy() == k_ref).all(), "FP8 K pool differs from the oracle"
        assert (self.v_pool.cpu().numpy() == v_ref).all(), "FP8 V pool differs from the oracle"
        return k_ref, v_ref

    def attend(self, varlen=True, softcap=1.0):
        c = self.case
        out = torch.full((max(c.total_q, 1), c.Hq, D), float("nan"),
                         dtype=torch.float16 if c.f16 else torch.bfloat16, device="cuda")
        if varlen:
            self.cache.varlen(out, self.q, self.tables, self.lens, c.cu_q, c.S, c.Hq, c.MB, c.scale,
                              self.ws, self.ws_bytes, softcap=softcap, context_lens_host=c.kv_lens)
        else:
            self.cache.decode(out, self.q, self.tables, self.lens, c.S, c.Hq, c.MB, c.scale,
                              self.ws, self.ws_bytes, softcap=softcap)
        torch.cuda.synchronize()
        self.cache.check_errors()
        return elems_to_f32(to_bits(out), c.f16)[:c.total_q]


def run(case, ks, vs, varlen=True, softcap=1.0, exact=False):
    dc = Fp8DeviceCase(case, ks, vs, exact=exact)
    k_ref, v_ref = dc.write_and_check()
    got = dc.attend(varlen=varlen, softcap=softcap)
    ref = attention_oracle_fp8(case, k_ref, v_ref, ks, vs, softcap=softcap, varlen=varlen)
    return got, ref


@pytest.mark.parametrize("f16", [False, True])
@pytest.mark.parametrize("G,Hkv", [(1, 2), (4, 8), (8, 2), (16, 1), (5, 8), (7, 4), (12, 2)])
def test_fp8_decode_edge_lengths(cuda_device, G, Hkv, f16):
    kv = [1, 15, 16, 17, 31, 32, 33, 255, 256, 257, 1000, 4097]
    case = Case(kv, [1] * len(kv), G * Hkv, Hkv, 512, seed=81 + G, f16=f16)
    for exact in (False, True):
        got, ref = run(case, 0.37, 0.6, varlen=False, exact=exact)
        check_attention(got, ref, f"fp8 decode G={G} f16={f16} exact={exact}")


def test_fp8_verify_and_mixed_widths(cuda_device):
    # 1, 2, 3 and 6 query tokens x 4 heads: all three width classes, split items included
    kv = [700, 64, 1029, 300, 6, 2500]
    ql = [1, 2, 3, 6, 6, 5]
    case = Case(kv, ql, 8, 2, 512, seed=82)
    got, ref = run(case, 0.5, 0.25)
    check_attention(got, ref, "fp8 verify")
    got_cap, ref_cap = run(case, 0.5, 0.25, softcap=30.0, exact=True)
    check_attention(got_cap, ref_cap, "fp8 verify softcap")


def test_fp8_long_contexts_are_split_across_ctas(cuda_device):
    kv = [20000, 9000, 33, 15000]
    case = Case(kv, [1] * 4, 32, 8, 4096, seed=83)
    got, ref = run(case, 1.0, 1.0, varlen=False)
    check_attention(got, ref, "fp8 long decode")


def test_fp8_write_out_of_range_values_bit_exact(cuda_device):
    """Values beyond the format's range, below its smallest step, infinities and NaN go
    through the same encoder as the reference's."""
    case = Case([40, 41], [8, 9], 4, 2, 16, seed=84)
    special = np.array([250.0, 256.0, 300.0, 1000.0, 16383.0, 16384.0, 1e9, -248.0, 0.0019, 0.00195,
                        0.0146, 0.0147, 0.0156, -0.0, np.inf, -np.inf, np.nan, 239.0, 240.0, 247.0],
                       dtype=np.float32)
    from pa_testlib import f32_to_bf16
    case.k_new.reshape(-1)[:len(special)] = f32_to_bf16(special)
    case.v_new.reshape(-1)[5:5 + len(special)] = f32_to_bf16(-special)
    dc = Fp8DeviceCase(case, 1.0, 1.0)
    dc.write_and_check()
    dc2 = Fp8DeviceCase(case, 3.0, 0.01)
    dc2.write_and_check()


def test_fp8_every_byte_code_decodes_as_the_format_defines(cuda_device):
    """Single-token contexts: the output row is the value row itself, so all 256 codes can
    be read back through the attention kernel (infinity and NaN codes included)."""
    Hkv, G = 2, 1
    case = Case([1], [1], G * Hkv, Hkv, 16, seed=85)
    k8, v8 = fp8_pools(case.NB, Hkv)
    write_oracle_fp8(k8, v8, case.k_all, case.v_all, case.slots_all, Hkv, 1.0, 1.0)
    blk = int(case.block_tables[0, 0])
    v8[blk, :, :, 0] = np.arange(256, dtype=np.uint8).reshape(Hkv, D)
    v8[blk, :, :, 1:] = 0x7F   # other tokens of the block: NaN codes, must not leak
    case.q_lens[:] = 0          # nothing new to write
    case.slot_mapping = case.slot_mapping[:0]
    dc = Fp8DeviceCase(case, 1.0, 0.5, k8=k8, v8=v8)
    case.q_lens[:] = 1
    got = dc.attend(varlen=False).reshape(256)
    want = np.array([oracle().oracle_fp8_e4m3_decode(c) for c in range(256)], dtype=np.float64) * 0.5
    assert np.array_equal(np.isnan(got), np.isnan(want))
    ok = ~np.isnan(want)
    assert (got[ok].astype(np.float64) == want[ok]).all()


class _RawBytes:
    def __init__(self, ptr, shape):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": "|u1",
                                         "data": (int(ptr), False), "version": 2}


def test_fp8_overflow_in_a_write_switches_to_exact_decoding(cuda_device):
    """A library-owned cache decodes with the fast variant until a write produces an
    exponent-15 byte; from then on the infinity it stands for must come out."""
    Hkv, Hq, NB = 2, 4, 8
    case = Case([3], [1], Hq, Hkv, NB, seed=88, prefill=False)
    from pa_testlib import f32_to_bf16
    case.v_all[2, 1, 5] = f32_to_bf16(np.array([250.0], dtype=np.float32))[0]   # rounds past 240
    cache = pa.PagedCache(BS, NB, D, Hkv, fp8=True)
    k_all, v_all = to_dev(case.k_all), to_dev(case.v_all)
    slots = torch.from_numpy(case.slots_all).cuda()
    tables, lens = torch.from_numpy(case.block_tables).cuda(), torch.from_numpy(case.kv_lens).cuda()
    ws = torch.empty(cache.workspace_bytes(), dtype=torch.uint8, device="cuda")
    q = to_dev(case.q)
    k8, v8 = fp8_pools(NB, Hkv)
    kp = torch.as_tensor(_RawBytes(cache.key_ptr(), k8.shape), device="cuda")
    vp = torch.as_tensor(_RawBytes(cache.value_ptr(), v8.shape), device="cuda")

    def attend(n):
        out = torch.full((1, Hq, D), float("nan"), dtype=torch.bfloat16, device="cuda")
        cache.decode(out, q, tables, torch.full_like(lens, n), 1, Hq, case.MB, case.scale, ws,
                     cache.workspace_bytes())
        torch.cuda.synchronize()
        cache.check_errors()
        case.kv_lens[:] = n
        ref = attention_oracle_fp8(case, k8, v8, 1.0, 1.0, varlen=False)
        case.kv_lens[:] = 3
        return elems_to_f32(to_bits(out), False), ref

    # first two tokens only: in range, fast variant
    cache.reshape_and_cache(k_all, v_all, slots, 2, Hkv * D, Hkv * D)
    write_oracle_fp8(k8, v8, case.k_all[:2], case.v_all[:2], case.slots_all[:2], Hkv, 1.0, 1.0)
    torch.cuda.synchronize()
    assert (kp.cpu().numpy() == k8).all() and (vp.cpu().numpy() == v8).all()
    got, ref = attend(2)
    check_attention(got, ref, "before the overflow")
    # third token carries the overflowing value
    cache.reshape_and_cache(k_all[2:], v_all[2:], slots[2:], 1, Hkv * D, Hkv * D)
    write_oracle_fp8(k8, v8, case.k_all[2:], case.v_all[2:], case.slots_all[2:], Hkv, 1.0, 1.0)
    torch.cuda.synchronize()
    assert (vp.cpu().numpy() == v8).all() and (v8 == 0x78).sum() == 1
    got, ref = attend(3)
    assert np.array_equal(np.isinf(got), np.isinf(ref)) and np.isinf(ref).sum() == 2  # heads 2, 3
    fin = np.isfinite(ref)
    check_attention(np.where(fin, got, 0), np.where(fin, ref, 0), "finite part")


@pytest.mark.parametrize("f16", [False, True])
def test_fp8_long_chunks_run_on_the_tile_kernel(cuda_device, f16):
    """Prefill chunks over an FP8 cache: the tcgen05 tile kernel converts the cache bytes to
    f16 on their way into shared memory.  Chunks that start and end inside blocks, contexts
    that end inside a block (the pool holds NaN codes where nothing was written), a decode
    and an empty sequence ride along; with and without host context lengths."""
    case = Case([200, 64, 33, 700, 1500, 129], [100, 30, 1, 0, 600, 129], 8, 2, 256, seed=86, f16=f16)
    got, ref = run(case, 0.5, 0.25)
    check_attention(got, ref, f"fp8 chunk on the tile kernel f16={f16}")
    got_cap, ref_cap = run(case, 0.5, 0.25, softcap=30.0)
    check_attention(got_cap, ref_cap, f"fp8 chunk on the tile kernel, softcap, f16={f16}")
    dc = Fp8DeviceCase(case, 0.5, 0.25, exact=False)
    k_ref, v_ref = dc.write_and_check()
    out = torch.full((case.total_q, case.Hq, D), float("nan"),
                     dtype=torch.float16 if f16 else torch.bfloat16, device="cuda")
    dc.cache.varlen(out, dc.q, dc.tables, dc.lens, case.cu_q, case.S, case.Hq, case.MB,
                    case.scale, dc.ws, dc.ws_bytes)   # no host lengths: kernels back to back
    torch.cuda.synchronize()
    dc.cache.check_errors()
    check_attention(elems_to_f32(to_bits(out), f16), got, "without host lengths")


def test_fp8_tile_kernel_wide_groups_and_long_context(cuda_device):
    # G = 16 (16 queries per 256-row CTA) and G = 1; a context beyond the staged block table
    for G, Hkv, kv, ql in ((16, 1, [3000, 500], [40, 500]), (1, 2, [36000, 300], [260, 300])):
        case = Case(kv, ql, G * Hkv, Hkv, 2400, seed=87 + G)
        got, ref = run(case, 0.37, 0.6)
        check_attention(got, ref, f"fp8 tile kernel G={G}")


def test_fp8_copy_blocks_and_swap(cuda_device):
    case = Case([64, 48], [1, 1], 4, 2, 16, seed=87)
    dc = Fp8DeviceCase(case, 1.0, 1.0)
    dc.write_and_check()
    before_k, before_v = dc.k_pool.cpu().numpy().copy(), dc.v_pool.cpu().numpy().copy()
    src = int(case.block_tables[0, 0])
    free = sorted(set(range(case.NB)) - set(case.block_tables.ravel().tolist()))
    dst = free[0]
    mapping = torch.tensor([[src, dst]], dtype=torch.int64, device="cuda")
    dc.cache.copy_blocks(mapping, 1)
    torch.cuda.synchronize()
    k_now, v_now = dc.k_pool.cpu().numpy(), dc.v_pool.cpu().numpy()
    assert (k_now[dst] == before_k[src]).all() and (v_now[dst] == before_v[src]).all()
    keep = np.ones(case.NB, dtype=bool)
    keep[dst] = False
    assert (k_now[keep] == before_k[keep]).all() and (v_now[keep] == before_v[keep]).all()
    cpu = dc.cache.create_cpu_cache()
    dc.cache.swap_out([src], cpu)
    torch.cuda.synchronize()
    dc.k_pool[src].fill_(0)
    dc.v_pool[src].fill_(0)
    dc.cache.swap_in([src], cpu)
    torch.cuda.synchronize()
    assert (dc.k_pool.cpu().numpy()[src] == before_k[src]).all()
    assert (dc.v_pool.cpu().numpy()[src] == before_v[src]).all()


def test_fp8_scales_are_per_layer_and_validated(cuda_device):
    cache = pa.PagedCache(BS, 8, D, 2, num_layers=2, fp8=True)
    assert cache.kv_scales(0) == (1.0, 1.0)
    cache.set_kv_scales(0.5, 0.25, layer=1)
    assert cache.kv_scales(1) == (0.5, 0.25) and cache.kv_scales(0) == (1.0, 1.0)
    for bad in ((0.0, 1.0), (1.0, -1.0), (float("inf"), 1.0), (float("nan"), 1.0)):
        with pytest.raises(pa.PagedAttnError):
            cache.set_kv_scales(*bad)
    plain = pa.PagedCache(BS, 8, D, 2)
    with pytest.raises(pa.PagedAttnError):
        plain.set_kv_scales(0.5, 0.5)
