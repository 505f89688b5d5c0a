"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU
oracle on the same seeded inputs.  KV write: bit-exact.  Attention: bf16 output
with fp32 accumulation within max-abs 2e-2 and 1e-2 relative (RMS-floored) of
the fp64-accumulated oracle (pa_testlib.check_attention)."""
import os

import numpy as np
import pytest
import torch

import paged_attn_b200 as pa
from golden import make_golden
from gpu_util import DeviceCase, device_view, to_bits, to_dev
from pa_testlib import (BS, CANARY, D, X, Case, attention_oracle, attention_oracle_rows,
                        bf16_to_f32, check_attention, config_lengths, normal_bf16, oracle, p,
                        write_oracle)

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def run_case(case, varlen=True, softcap=1.0):
    dc = DeviceCase(case)
    dc.write()
    torch.cuda.synchronize()
    k_ref, v_ref = case.pools_after_write()
    assert (to_bits(dc.k_pool) == k_ref).all(), "K pool differs from the oracle"
    assert (to_bits(dc.v_pool) == v_ref).all(), "V pool differs from the oracle"
    got = dc.attend(varlen=varlen, softcap=softcap)
    ref = attention_oracle(case, k_ref, v_ref, softcap=softcap, varlen=varlen)
    return got, ref


@pytest.mark.parametrize("name", sorted(make_golden.CASES))
def test_golden_cases(cuda_device, name):
    case = make_golden.build(name)
    g = np.load(os.path.join(GOLDEN, name + ".npz"))
    got, ref = run_case(case)
    check_attention(got, g["out"], name + " vs golden")
    check_attention(got, ref, name + " vs oracle")
    got_cap, _ = run_case(case, softcap=30.0)
    check_attention(got_cap, g["out_softcap30"], name + " softcap vs golden")


@pytest.mark.parametrize("G,Hkv", [(1, 2), (2, 8), (4, 8), (8, 8), (16, 1),
                                   (3, 4), (5, 8), (6, 2), (7, 4), (12, 2), (24, 1)])
def test_decode_edge_lengths(cuda_device, G, Hkv):
    # (group sizes that are not powers of two too: 40 query / 8 kv heads and 28 / 4 are shapes
    # of the Qwen family, 12 / 2 is the one the reference's parameter test uses,
    # crates/mlx-paged-attn/src/metal/paged_attention.rs:998-1016)
    # context 1, one block exactly, k*BS +- 1, a long one, and an empty sequence
    kv = [1, 15, 16, 17, 31, 32, 33, 0, 255, 256, 257, 1000, 4097]
    ql = [1 if n > 0 else 0 for n in kv]
    case = Case(kv, ql, G * Hkv, Hkv, 512, seed=31 + G)
    # decode entry: one query per sequence, including the empty one
    case.q = normal_bf16((len(kv), G * Hkv, D), 31 + G, 7)
    case.total_q = len(kv)
    case.cu_q = np.arange(len(kv) + 1, dtype=np.int32)
    got, ref = run_case(case, varlen=False)
    assert (got[7] == 0).all(), "empty context must give a zero row"
    check_attention(got, ref, f"decode edges G={G}")


def test_decode_wide_table_and_row_strides(cuda_device):
    # block-table width as the crate builds it (max_seq_len / block_size, zero padded)
    case = Case([300, 45, 1029], [1, 1, 1], 32, 8, 256, seed=40, mb_extra=190)
    dc = DeviceCase(case)
    # strided new K/V rows and strided q/out rows
    ks = torch.zeros(case.S, case.Hkv * D + 64, dtype=torch.bfloat16, device="cuda")
    vs = torch.zeros_like(ks)
    ks[:, :case.Hkv * D] = to_dev(case.k_new).view(case.S, -1)
    vs[:, :case.Hkv * D] = to_dev(case.v_new).view(case.S, -1)
    dc.cache.reshape_and_cache(ks, vs, dc.slots, case.S, ks.stride(0), vs.stride(0))
    k_ref, v_ref = case.pools_after_write()
    torch.cuda.synchronize()
    assert (to_bits(dc.k_pool) == k_ref).all() and (to_bits(dc.v_pool) == v_ref).all()
    qs = torch.zeros(case.S, case.Hq * D + 128, dtype=torch.bfloat16, device="cuda")
    qs[:, :case.Hq * D] = dc.q.view(case.S, -1)
    outs = torch.zeros_like(qs)
    dc.cache.decode(outs, qs, dc.tables, dc.lens, case.S, case.Hq, case.MB, case.scale, dc.ws,
                    dc.ws_bytes, q_stride=qs.stride(0), out_stride=outs.stride(0))
    torch.cuda.synchronize()
    dc.cache.check_errors()
    got = bf16_to_f32(to_bits(outs[:, :case.Hq * D].contiguous())).reshape(case.S, case.Hq, D)
    check_attention(got, attention_oracle(case, k_ref, v_ref), "wide table, strided rows")
    assert (outs[:, case.Hq * D:] == 0).all(), "wrote outside the output rows"


@pytest.mark.parametrize("kv,ql,Hq,Hkv", [
    ([1, 15, 16, 17, 100, 4097, 700], [1] * 7, 32, 8),          # decode
    ([37, 70, 21, 2000], [5, 5, 1, 3], 16, 4),                  # verify-shaped
    ([640 + 200, 333, 77], [200, 333, 77], 32, 8),              # prefill chunks (tcgen05 path)
])
def test_f16_cache(cuda_device, kv, ql, Hq, Hkv):
    # The reference's default cache dtype is f16 (dtype code 0,
    # crates/mlx-core/src/transformer/paged_attention.rs:85-92).
    case = Case(kv, ql, Hq, Hkv, 512, seed=90, f16=True)
    got, ref = run_case(case)
    print("f16", check_attention(got, ref, "f16 cache"))


def test_write_edges(cuda_device):
    # negative slots skipped, ragged token count, untouched slots unchanged
    Hkv, NB, T = 8, 64, 37
    rng = np.random.Generator(np.random.PCG64(5))
    slots = rng.permutation(NB * BS)[:T].astype(np.int64)
    slots[[3, 20]] = -1
    key, val = normal_bf16((T, Hkv, D), 50, 1), normal_bf16((T, Hkv, D), 50, 2)
    k_pool = np.full((NB, Hkv, D // X, BS, X), CANARY, dtype=np.uint16)
    v_pool = np.full((NB, Hkv, D, BS), CANARY, dtype=np.uint16)
    kd, vd = to_dev(k_pool), to_dev(v_pool)
    cache = pa.PagedCache(BS, NB, D, Hkv, key_pools=[kd], value_pools=[vd])
    cache.reshape_and_cache(to_dev(key), to_dev(val), torch.from_numpy(slots).cuda(), T, Hkv * D,
                            Hkv * D)
    torch.cuda.synchronize()
    cache.check_errors()
    oracle().oracle_reshape_and_cache(p(key), p(val), p(k_pool), p(v_pool), p(slots), T, Hkv * D,
                                      Hkv * D, Hkv, D, BS, X)
    assert (to_bits(kd) == k_pool).all() and (to_bits(vd) == v_pool).all()
    # zero tokens is a no-op
    cache.reshape_and_cache(to_dev(key), to_dev(val), torch.from_numpy(slots).cuda(), 0, Hkv * D,
                            Hkv * D)


def test_out_of_range_ids_are_reported_not_followed(cuda_device):
    case = Case([40, 70], [1, 1], 8, 2, 16, seed=60)
    dc = DeviceCase(case)
    dc.write()
    bad_slots = torch.tensor([16 * BS + 3, 5], dtype=torch.int64, device="cuda")
    dc.cache.reshape_and_cache(dc.k_new, dc.v_new, bad_slots, 2, case.Hkv * D, case.Hkv * D)
    with pytest.raises(pa.PagedAttnError) as e:
        dc.cache.check_errors()
    assert e.value.status == 4
    dc.cache.check_errors()  # the error word is cleared once reported
    dc.tables[0, 1] = 1 << 20
    out = torch.zeros(case.S, case.Hq, D, dtype=torch.bfloat16, device="cuda")
    dc.cache.decode(out, dc.q, dc.tables, dc.lens, case.S, case.Hq, case.MB, case.scale, dc.ws,
                    dc.ws_bytes)
    with pytest.raises(pa.PagedAttnError) as e:
        dc.cache.check_errors()
    assert e.value.status == 4


def test_copy_blocks(cuda_device):
    Hkv, NB = 8, 32
    k_pool, v_pool = normal_bf16((NB, Hkv, D // X, BS, X), 70, 1), normal_bf16((NB, Hkv, D, BS), 70, 2)
    kd, vd = to_dev(k_pool), to_dev(v_pool)
    cache = pa.PagedCache(BS, NB, D, Hkv, key_pools=[kd], value_pools=[vd])
    pairs = np.array([[0, 9], [5, 31], [7, 8]], dtype=np.int64)
    cache.copy_blocks(torch.from_numpy(pairs).cuda(), 3)
    torch.cuda.synchronize()
    cache.check_errors()
    oracle().oracle_copy_blocks(p(k_pool), p(v_pool), p(pairs), 3, Hkv * D * BS)
    assert (to_bits(kd) == k_pool).all() and (to_bits(vd) == v_pool).all()


def test_swap_out_and_in(cuda_device):
    # PagedKVCache::swap_out / swap_in (crates/mlx-paged-attn/src/paged_kv_cache.rs:1542-1637)
    import ctypes as C
    Hkv, NB = 8, 64
    k_pool, v_pool = normal_bf16((NB, Hkv, D // X, BS, X), 71, 1), normal_bf16((NB, Hkv, D, BS), 71, 2)
    kd, vd = to_dev(k_pool), to_dev(v_pool)
    cache = pa.PagedCache(BS, NB, D, Hkv, key_pools=[kd], value_pools=[vd])
    cpu = cache.create_cpu_cache()
    assert cpu.num_swapped() == 0 and not cpu.is_swapped(0)
    ids = [3, 17, 63, 0]
    cache.swap_out(ids, cpu)
    cache.swap_out([17], cpu)                      # already out: skipped
    assert cpu.num_swapped() == 4 and cpu.is_swapped(63)
    nbytes = Hkv * D * BS * 2
    for b in ids:
        kp, vp = cpu.block_ptrs(b)
        assert C.string_at(kp, nbytes) == k_pool[b].tobytes()
        assert C.string_at(vp, nbytes) == v_pool[b].tobytes()
    # the device blocks are reused by someone else, then the originals come back
    kd[torch.tensor(ids).cuda()] = 0
    vd[torch.tensor(ids).cuda()] = 0
    with pytest.raises(pa.PagedAttnError) as e:
        cache.swap_in([3, 5], cpu)
    assert "Block 5 not found in CPU cache" in str(e.value)
    assert (to_bits(kd)[3] == 0).all()             # nothing moved by the failed call
    cache.swap_in(ids, cpu)
    cache.check_errors()
    assert cpu.num_swapped() == 0
    assert (to_bits(kd) == k_pool).all() and (to_bits(vd) == v_pool).all()


def test_config1_full(cuda_device):
    # Qwen3-0.6B-shaped decode: the whole configuration against the whole oracle.
    kv, ql, Hq, Hkv, NB = config_lengths("c1")
    case = Case(kv, ql, Hq, Hkv, NB, seed=0)
    got, ref = run_case(case, varlen=False)
    stats = check_attention(got, ref, "config 1")
    got2, _ = run_case(case, varlen=True)
    assert (got == got2).all(), "decode and varlen(q_len=1) entries must agree bit for bit"
    print("config1", stats)


@pytest.mark.parametrize("name,n_seq", [("c2", 12), ("c3", 10)])
def test_decode_configs_reduced(cuda_device, name, n_seq):
    # Same head shapes and length distribution, fewer sequences and a smaller pool so
    # the full oracle finishes in seconds.
    kv, ql, Hq, Hkv, _ = config_lengths(name)
    order = np.argsort(kv)
    pick = np.concatenate([order[:2], order[-2:], order[len(order) // 2:len(order) // 2 + n_seq - 4]])
    kv, ql = kv[pick], ql[pick]
    NB = int(((kv + BS - 1) // BS).sum()) + 64
    case = Case(kv, ql, Hq, Hkv, NB, seed=0)
    got, ref = run_case(case, varlen=False)
    print(name, check_attention(got, ref, name + " reduced"))


def test_mixed_batch_reduced(cuda_device):
    # config-5-shaped: decode + 5-token verify + prefill chunks in ONE call
    kv = [1500, 9000, 3333, 16, 2053, 4101, 700, 1024 + 300, 512 + 1024]
    ql = [1, 1, 1, 1, 5, 5, 5, 300, 1024]
    case = Case(kv, ql, 32, 8, 2048, seed=3)
    got, ref = run_case(case)
    print("mixed", check_attention(got, ref, "mixed batch"))
    # without host context lengths the kernels run back to back on every SM instead of
    # side by side on shares of them: another partition of the same work, so not
    # necessarily the same bits, but the same parity bound - and the same bits run to run
    dc = DeviceCase(case)
    dc.write()
    serial = dc.attend(host_lens=False)
    check_attention(serial, ref, "mixed batch, kernels back to back")
    assert (dc.attend(host_lens=False) == serial).all()
    assert (dc.attend(host_lens=True) == got).all()


def test_all_width_classes_and_a_chunk_side_by_side(cuda_device):
    """Decode (4 columns), 3-token verify (12), 5-token verify (20) and a prefill chunk, long
    enough that the call runs its three split-KV launches and the tile kernel at the same
    time, each split-KV launch on its own range of partial slots and counters."""
    kv = [9000, 6000, 500, 7000, 2500, 8000, 1200, 3000 + 512]
    ql = [1, 1, 1, 3, 3, 5, 5, 512]
    case = Case(kv, ql, 32, 8, 2400, seed=9)
    got, ref = run_case(case)
    print("classes", check_attention(got, ref, "three width classes + chunk"))
    dc = DeviceCase(case)
    dc.write()
    assert (dc.attend() == got).all()          # same shares, same partitions: same bits
    # and with a soft cap (the tile kernel's other variant)
    got_cap, ref_cap = run_case(case, softcap=30.0)
    check_attention(got_cap, ref_cap, "three width classes + chunk, soft cap")


@pytest.mark.parametrize("G,Hkv,fp8", [(5, 8, False), (7, 4, False), (6, 2, False), (3, 4, False)])
def test_mixed_batch_with_odd_group_sizes(cuda_device, G, Hkv, fp8):
    """Decode, verify and prefill chunks in one call with 5, 7, 6 and 3 query heads per kv
    head: columns and tile rows are (query token, head) pairs by plain division, so a
    query's heads may straddle column tiles and the two 128-row halves of a tile CTA."""
    kv = [1500, 3333, 16, 2053, 4101, 700, 300 + 77, 512 + 300, 9000]
    ql = [1, 1, 1, 2, 4, 5, 77, 300, 1]
    case = Case(kv, ql, G * Hkv, Hkv, 1600, seed=40 + G)
    got, ref = run_case(case)
    print("G", G, check_attention(got, ref, f"mixed batch, {G} query heads per kv head"))
    got_cap, ref_cap = run_case(case, softcap=30.0)
    check_attention(got_cap, ref_cap, f"mixed batch with soft cap, {G} query heads per kv head")


def test_prefill_chunk_reduced(cuda_device):
    # config-4-shaped: cached prefix + causal chunk, including a chunk that is not a
    # multiple of the tile and a prefix that is not a multiple of the block
    kv = [2048 + 512, 1000 + 333, 77]
    ql = [512, 333, 77]
    case = Case(kv, ql, 32, 8, 512, seed=4)
    got, ref = run_case(case)
    print("prefill", check_attention(got, ref, "prefill chunk"))


def test_more_sequences_than_one_launch_covers(cuda_device):
    """The split-KV kernel keeps per-launch prefix sums for 2048 sequences; a larger batch is
    cut into several launches that share the workspace one after the other."""
    rng = np.random.Generator(np.random.PCG64(41))
    S = 2048 + 77
    kv = rng.integers(0, 40, size=S)          # includes empty contexts
    kv[5] = 700                                 # and one item that is split across CTAs
    ql = (kv > 0).astype(np.int64)
    case = Case(kv, ql, 8, 2, 4096, seed=41)
    case.q = normal_bf16((S, 8, D), 41, 7)      # one query per sequence, empty ones included
    case.total_q = S
    case.cu_q = np.arange(S + 1, dtype=np.int32)
    got, ref = run_case(case, varlen=False)
    assert (got[kv == 0] == 0).all()
    check_attention(got, ref, "2125 sequences")


def test_fewer_units_than_ctas(cuda_device):
    """Three one-block sequences: most CTAs own nothing, the merge kernel must skip them."""
    case = Case([3, 16, 9], [1, 1, 1], 4, 1, 8, seed=42)
    got, ref = run_case(case, varlen=False)
    check_attention(got, ref, "tiny batch")
    got_v, ref_v = run_case(Case([3, 16, 9], [2, 1, 3], 4, 1, 8, seed=43))
    check_attention(got_v, ref_v, "tiny varlen batch")


def test_layers_of_a_library_owned_cache_are_independent(cuda_device):
    """pa_cache_create allocates zero-filled pools per layer; a write and an attention call
    on one layer neither read nor disturb the others."""
    L = 3
    cases = [Case([70, 33, 129], [1, 1, 1], 8, 2, 32, seed=50 + i, prefill=False) for i in range(L)]
    cache = pa.PagedCache(BS, 32, D, 2, num_layers=L)
    ws = torch.empty(cache.workspace_bytes(), dtype=torch.uint8, device="cuda")
    for i, c in enumerate(cases):
        k_view = device_view(cache.key_ptr(i), (c.NB, c.Hkv, D // X, BS, X))
        assert (k_view.view(torch.int16) == 0).all(), "pools start zero-filled"
        slots = torch.from_numpy(c.slots_all).cuda()
        cache.reshape_and_cache(to_dev(c.k_all), to_dev(c.v_all), slots, len(c.slots_all),
                                c.Hkv * D, c.Hkv * D, layer=i)
    torch.cuda.synchronize()
    for i, c in enumerate(cases):
        k_ref = np.zeros_like(c.k_pool)
        v_ref = np.zeros_like(c.v_pool)
        write_oracle(k_ref, v_ref, c.k_all, c.v_all, c.slots_all, c.Hkv)
        k_got = to_bits(device_view(cache.key_ptr(i), k_ref.shape))
        v_got = to_bits(device_view(cache.value_ptr(i), v_ref.shape))
        assert (k_got == k_ref).all() and (v_got == v_ref).all(), f"layer {i} pools"
        out = torch.full((c.S, c.Hq, D), float("nan"), dtype=torch.bfloat16, device="cuda")
        cache.decode(out, to_dev(c.q), torch.from_numpy(c.block_tables).cuda(),
                     torch.from_numpy(c.kv_lens).cuda(), c.S, c.Hq, c.MB, c.scale, ws, ws.numel(),
                     layer=i)
        torch.cuda.synchronize()
        cache.check_errors()
        check_attention(bf16_to_f32(to_bits(out)), attention_oracle(c, k_ref, v_ref, varlen=False),
                        f"layer {i}")
    with pytest.raises(pa.PagedAttnError):
        cache.decode(out, to_dev(cases[0].q), torch.from_numpy(cases[0].block_tables).cuda(),
                     torch.from_numpy(cases[0].kv_lens).cuda(), 3, 8, cases[0].MB, 0.1, ws, ws.numel(),
                     layer=L)


def test_determinism_and_placement_invariance(cuda_device):
    # Same logical KV under two physical placements: outputs must be bit-identical,
    # and two runs of the same call must be bit-identical.
    kv, ql = [5000, 123, 2047, 800], [1, 1, 1, 1]
    a = Case(kv, ql, 32, 8, 1024, seed=9)
    b = Case(kv, ql, 32, 8, 1024, seed=9)
    rng = np.random.Generator(np.random.PCG64(77))
    perm = rng.permutation(1024).astype(np.int32)
    b.block_tables = np.zeros_like(a.block_tables)
    nblk = (np.asarray(kv) + BS - 1) // BS
    for s in range(len(kv)):
        b.block_tables[s, :nblk[s]] = perm[a.block_tables[s, :nblk[s]]]
        b.block_tables[s, nblk[s]:] = 0
    b.k_pool = np.full_like(a.k_pool, CANARY)
    b.v_pool = np.full_like(a.v_pool, CANARY)
    b.k_pool[perm] = a.k_pool
    b.v_pool[perm] = a.v_pool
    b.slot_mapping = perm[a.slot_mapping // BS].astype(np.int64) * BS + a.slot_mapping % BS
    got_a, _ = run_case(a, varlen=False)
    got_a2, _ = run_case(a, varlen=False)
    got_b, _ = run_case(b, varlen=False)
    assert (got_a == got_a2).all()
    assert (got_a == got_b).all()


@pytest.mark.parametrize("bs", [16, 32])
def test_tier1_reference_named_entry_points(cuda_device, bs):
    # create_cache -> reshape_and_cache -> get_*_cache -> forward -> copy_blocks, as
    # crates/mlx-core/src/transformer/paged_attention.rs:85-230 drives them.
    import ctypes as C
    lib = pa.load_library()
    case = Case([100, 37, 256], [1, 1, 1], 16, 8, 64, seed=12, prefill=False, bs=bs)
    cfg = pa.PagedAttnConfig(bs, case.NB, D, case.Hkv, 2, 1)
    cache = lib.mlx_paged_attn_create_cache(C.byref(cfg))
    assert cache

    def arr(t, dtype):
        shape = (C.c_int64 * t.dim())(*t.shape)
        return lib.pa_array_from_device(t.data_ptr(), dtype, shape, t.dim())
    k_all, v_all = to_dev(case.k_all), to_dev(case.v_all)
    slots = torch.from_numpy(case.slots_all).cuda()
    ka, va, sa = arr(k_all, 1), arr(v_all, 1), arr(slots, 4)
    lib.mlx_paged_attn_reshape_and_cache(cache, 1, ka, va, sa)
    q, tables, lens = to_dev(case.q), torch.from_numpy(case.block_tables).cuda(), \
        torch.from_numpy(case.kv_lens).cuda()
    qa, ta, la = arr(q, 1), arr(tables, 3), arr(lens, 3)
    kc, vc = lib.mlx_paged_attn_get_key_cache(cache, 1), lib.mlx_paged_attn_get_value_cache(cache, 1)
    assert lib.mlx_array_ndim(kc) == 5 and lib.mlx_array_ndim(vc) == 4
    out = lib.mlx_paged_attn_forward(qa, kc, vc, ta, la, case.scale, bs, int(case.kv_lens.max()))
    assert out, pa.last_error()
    shape = (C.c_int64 * 3)()
    lib.mlx_array_shape(out, shape)
    assert list(shape) == [case.S, case.Hq, D]
    got_dev = device_view(lib.pa_array_data(out), (case.S, case.Hq, D)).clone()
    k_ref = np.zeros((case.NB, case.Hkv, D // X, bs, X), dtype=np.uint16)
    v_ref = np.zeros((case.NB, case.Hkv, D, bs), dtype=np.uint16)
    oracle().oracle_reshape_and_cache(p(case.k_all), p(case.v_all), p(k_ref), p(v_ref),
                                      p(case.slots_all), len(case.slots_all), case.Hkv * D,
                                      case.Hkv * D, case.Hkv, D, bs, X)
    check_attention(bf16_to_f32(to_bits(got_dev)), attention_oracle(case, k_ref, v_ref, varlen=False),
                    "tier-1 forward")
    # layer 0 was never written and the pools start zeroed (crates/mlx-sys/src/mlx.cpp:3847)
    k0 = lib.mlx_paged_attn_get_key_cache(cache, 0)
    assert (device_view(lib.pa_array_data(k0), (case.NB, case.Hkv * D * bs)).view(torch.int16) == 0).all()
    for h in (ka, va, sa, qa, ta, la, kc, vc, k0, out):
        lib.mlx_array_delete(h)
    lib.mlx_paged_attn_free_cache(cache)


def test_decode_step_from_host_buffers(cuda_device):
    case = Case([513, 64, 2000, 31], [1, 1, 1, 1], 32, 8, 256, seed=13)
    dc = DeviceCase(case)
    out = np.zeros((case.S, case.Hq, D), dtype=np.uint16)
    dc.cache.decode_step_host(out, case.q, case.k_new, case.v_new, case.slot_mapping,
                              case.block_tables, case.kv_lens, case.S, case.Hq, case.MB, case.scale)
    k_ref, v_ref = case.pools_after_write()
    assert (to_bits(dc.k_pool) == k_ref).all() and (to_bits(dc.v_pool) == v_ref).all()
    check_attention(bf16_to_f32(out), attention_oracle(case, k_ref, v_ref), "host step")


def test_decode_step_from_pinned_host_buffers(cuda_device):
    """Pinned (device-mapped) buffers take the path where the kernels read host memory
    themselves; results and error reporting must be the same as with pageable memory."""
    case = Case([513, 64, 2000, 31, 17, 4096], [1] * 6, 32, 8, 512, seed=14)
    dc = DeviceCase(case)
    pin = lambda a: torch.from_numpy(a.view(np.int16) if a.dtype == np.uint16 else a).pin_memory()
    q, k, v = pin(case.q), pin(case.k_new), pin(case.v_new)
    slots, tables, lens = pin(case.slot_mapping), pin(case.block_tables), pin(case.kv_lens)
    out = torch.zeros(case.S, case.Hq, D, dtype=torch.int16).pin_memory()
    for _ in range(2):  # twice: the second call reuses the staging area
        out.zero_()
        dc.cache.decode_step_host(out, q, k, v, slots, tables, lens, case.S, case.Hq, case.MB,
                                  case.scale)
        k_ref, v_ref = case.pools_after_write()
        assert (to_bits(dc.k_pool) == k_ref).all() and (to_bits(dc.v_pool) == v_ref).all()
        check_attention(bf16_to_f32(out.numpy().view(np.uint16)),
                        attention_oracle(case, k_ref, v_ref), "pinned host step")
    # an out-of-range block id is reported by the same call
    bad = tables.clone().pin_memory()
    bad[2, 0] = case.NB + 5
    with pytest.raises(pa.PagedAttnError) as e:
        dc.cache.decode_step_host(out, q, k, v, slots, bad, lens, case.S, case.Hq, case.MB,
                                  case.scale)
    assert e.value.status == 4
    dc.cache.decode_step_host(out, q, k, v, slots, tables, lens, case.S, case.Hq, case.MB,
                              case.scale)  # and the handle stays usable
