"""CPU tests of the oracle itself: pinned against the committed golden fixtures
(made by an independent numpy implementation), against dense causal attention,
and against its own row-restricted and baseline variants."""
import hashlib
import os

import numpy as np
import pytest

import numpy_reference
from golden import make_golden
from pa_testlib import (BS, CANARY, D, X, Case, attention_oracle, attention_oracle_rows,
                        bf16_to_f32, f32_to_bf16, normal_bf16, oracle, p, write_oracle)

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


@pytest.mark.parametrize("name", sorted(make_golden.CASES))
def test_oracle_matches_golden(name):
    g = np.load(os.path.join(GOLDEN, name + ".npz"))
    case = make_golden.build(name)
    assert make_golden.digest(case.q, case.k_all, case.v_all, case.block_tables) == \
        str(g["inputs_sha256"]), "seeded inputs changed"
    k_pool, v_pool = case.pools_after_write()
    assert make_golden.digest(k_pool, v_pool) == str(g["pools_sha256"])
    b0 = case.block_tables[0, 0]
    assert (k_pool[b0] == g["k_pool_block0"]).all() and (v_pool[b0] == g["v_pool_block0"]).all()
    out = attention_oracle(case, k_pool, v_pool)
    np.testing.assert_allclose(out, g["out"], rtol=0, atol=2e-6)
    out_cap = attention_oracle(case, k_pool, v_pool, softcap=30.0)
    np.testing.assert_allclose(out_cap, g["out_softcap30"], rtol=0, atol=2e-6)


def test_write_index_formula_small():
    # One token, slot 50 in a 16-token-block pool: block 3, offset 2.  Element (h, d) lands at
    # K[3, h, d//8, 2, d%8] and V[3, h, d, 2]
    # (crates/mlx-paged-attn/metal/cache/reshape_and_cache.metal:65-85).
    Hkv, NB = 2, 5
    k_pool = np.zeros((NB, Hkv, D // X, BS, X), dtype=np.uint16)
    v_pool = np.zeros((NB, Hkv, D, BS), dtype=np.uint16)
    key = np.arange(1, Hkv * D + 1, dtype=np.uint16).reshape(1, Hkv, D)
    val = (key + 1000).astype(np.uint16)
    write_oracle(k_pool, v_pool, key, val, np.array([50], dtype=np.int64), Hkv)
    for h in range(Hkv):
        for d in (0, 7, 8, 127):
            assert k_pool[3, h, d // 8, 2, d % 8] == key[0, h, d]
            assert v_pool[3, h, d, 2] == val[0, h, d]
    assert np.count_nonzero(k_pool) == Hkv * D and np.count_nonzero(v_pool) == Hkv * D


def test_write_skips_negative_slots_and_honours_strides():
    Hkv, NB, T = 2, 4, 5
    stride = Hkv * D + 64
    key = normal_bf16((T, stride), 3, 1)
    val = normal_bf16((T, stride), 3, 2)
    slots = np.array([5, -1, 17, 63, -7], dtype=np.int64)
    k_pool = np.full((NB, Hkv, D // X, BS, X), CANARY, dtype=np.uint16)
    v_pool = np.full((NB, Hkv, D, BS), CANARY, dtype=np.uint16)
    write_oracle(k_pool, v_pool, key, val, slots, Hkv, stride, stride)
    k_exp, v_exp = np.full_like(k_pool, CANARY), np.full_like(v_pool, CANARY)
    for t, s in enumerate(slots):
        if s < 0:
            continue
        k_exp[s // BS, :, :, s % BS, :] = key[t, :Hkv * D].reshape(Hkv, D // X, X)
        v_exp[s // BS, :, :, s % BS] = val[t, :Hkv * D].reshape(Hkv, D)
    assert (k_pool == k_exp).all() and (v_pool == v_exp).all()


def test_copy_blocks_oracle():
    Hkv, NB = 2, 6
    k_pool = normal_bf16((NB, Hkv, D // X, BS, X), 4, 1)
    v_pool = normal_bf16((NB, Hkv, D, BS), 4, 2)
    k0, v0 = k_pool.copy(), v_pool.copy()
    pairs = np.array([[0, 3], [1, 5]], dtype=np.int64)
    oracle().oracle_copy_blocks(p(k_pool), p(v_pool), p(pairs), 2, Hkv * D * BS)
    assert (k_pool[3] == k0[0]).all() and (v_pool[5] == v0[1]).all()
    assert (k_pool[[0, 1, 2, 4]] == k0[[0, 1, 2, 4]]).all()


def test_rows_variant_equals_full():
    case = Case([70, 33, 16], [3, 1, 16], 8, 2, 16, seed=5)
    k_pool, v_pool = case.pools_after_write()
    full = attention_oracle(case, k_pool, v_pool)
    rows = [(0, 2, 7), (1, 0, 0), (2, 15, 3), (2, 0, 4)]
    got = attention_oracle_rows(rows, case.q, k_pool, v_pool, case.block_tables, case.kv_lens,
                                case.cu_q, case.Hq, case.Hkv, case.MB, case.scale)
    for r, (s, j, hq) in enumerate(rows):
        assert (got[r] == full[case.cu_q[s] + j, hq]).all()


def test_paged_oracle_equals_dense_causal():
    # Prefix + chunk over the paged pool == dense causal attention over the
    # concatenated contiguous tensors.
    case = Case([96, 40, 130], [32, 40, 1], 8, 2, 32, seed=6)
    k_pool, v_pool = case.pools_after_write()
    paged = attention_oracle(case, k_pool, v_pool)
    dense = np.zeros_like(paged)
    oracle().oracle_dense_causal(p(dense), p(case.q), p(case.k_all), p(case.v_all), p(case.cu_q),
                                 p(case.cu_kv), case.S, case.Hq, case.Hkv, D, case.scale)
    np.testing.assert_allclose(paged, dense, rtol=0, atol=1e-6)


def test_empty_context_gives_zero_rows_and_padding_is_not_read():
    case = Case([0, 20, 0], [0, 1, 0], 4, 2, 8, seed=7, mb_extra=3)
    k_pool, v_pool = case.pools_after_write()
    # decode call (no cu_q_lens): sequences 0 and 2 have context 0
    q = normal_bf16((3, 4, D), 7, 9)
    out = np.ones((3, 4, D), dtype=np.float32)
    oracle().oracle_paged_attention_varlen(p(out), p(q), p(k_pool), p(v_pool), p(case.block_tables),
                                           p(case.kv_lens), None, 3, 4, 2, D, BS, case.MB, 4 * D,
                                           case.scale, 1.0)
    assert (out[0] == 0).all() and (out[2] == 0).all() and np.isfinite(out[1]).all()
    assert np.abs(out[1]).max() > 0


def test_cpu_baseline_tracks_oracle():
    case = Case([300, 17, 129, 64], [1, 1, 1, 1], 8, 2, 64, seed=8)
    k_pool, v_pool = case.pools_after_write()
    ref = attention_oracle(case, k_pool, v_pool)
    out = np.zeros((case.S, case.Hq, D), dtype=np.uint16)
    rc = oracle().baseline_mlx_paged_forward(p(out), p(case.q), p(k_pool), p(v_pool),
                                             p(case.block_tables), p(case.kv_lens), case.S,
                                             case.Hq, case.Hkv, D, BS, case.MB, case.scale)
    assert rc == 0
    # bf16 intermediates (scores, weights) as in an MLX graph of bf16 arrays: loose bound
    assert np.abs(bf16_to_f32(out) - ref).max() < 3e-2


def test_generator_is_counter_based_and_matches_numpy_restatement():
    a = normal_bf16((4096,), 0, 5)
    b = np.empty(100, dtype=np.uint16)
    oracle().oracle_fill_normal_bf16(p(b), 100, 0, 5, 1000)
    assert (a[1000:1100] == b).all()

    def splitmix(z):
        z = (z + 0x9E3779B97F4A7C15) & (2**64 - 1)
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & (2**64 - 1)
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & (2**64 - 1)
        return z ^ (z >> 31)
    import math
    base = splitmix((0 * 0x100000001B3 + 5) & (2**64 - 1))
    for i in (0, 1, 17, 4095):
        r = splitmix((base + i) & (2**64 - 1))
        u1 = (((r >> 40) & 0xFFFFFF) + 1.0) / 16777216.0
        u2 = ((r >> 16) & 0xFFFFFF) / 16777216.0
        z = math.sqrt(-2.0 * math.log(u1)) * math.cos(6.283185307179586 * u2)
        assert a[i] == f32_to_bf16(np.array([z], dtype=np.float32))[0]
    f = bf16_to_f32(normal_bf16((1 << 18,), 1, 1))
    assert abs(f.mean()) < 0.01 and abs(f.std() - 1.0) < 0.01


def test_bf16_rounding_helper():
    x = np.array([1.0, 1.00390625, 1.01171875, np.nan, -0.0, 3.3895314e38], dtype=np.float32)
    got = f32_to_bf16(x)
    ref = np.empty(len(x), dtype=np.uint16)
    oracle().oracle_f32_to_bf16(p(x), p(ref), len(x))
    assert (got == ref).all()
    assert got[0] == 0x3F80 and got[1] == 0x3F80 and got[2] == 0x3F82 and got[3] == 0x7FC0


def test_numpy_reference_agrees_on_random_case():
    rng = np.random.Generator(np.random.PCG64(99))
    kv = rng.integers(1, 90, 5)
    ql = np.minimum(rng.integers(1, 8, 5), kv)
    case = Case(kv, ql, 8, 4, 40, seed=21)
    k_pool, v_pool = case.pools_after_write()
    ref = numpy_reference.paged_attention(case.q, k_pool, v_pool, case.block_tables, case.kv_lens,
                                          case.cu_q, case.Hq, case.Hkv, case.scale)
    np.testing.assert_allclose(attention_oracle(case, k_pool, v_pool), ref, rtol=0, atol=2e-6)


@pytest.mark.parametrize("bs", [8, 32])
def test_other_block_sizes_against_numpy_reference_and_index_formula(bs):
    """Block sizes 8 and 32 (32 is the default of PagedAttentionConfig,
    crates/mlx-paged-attn/src/config.rs:128): slot 50 is block 50 // bs, offset 50 % bs;
    attention agrees with the numpy statement."""
    Hkv, NB = 2, 7
    k_pool = np.zeros((NB, Hkv, D // X, bs, X), dtype=np.uint16)
    v_pool = np.zeros((NB, Hkv, D, bs), dtype=np.uint16)
    key = np.arange(1, Hkv * D + 1, dtype=np.uint16).reshape(1, Hkv, D)
    val = (key + 1000).astype(np.uint16)
    write_oracle(k_pool, v_pool, key, val, np.array([50], dtype=np.int64), Hkv)
    blk, off = 50 // bs, 50 % bs
    for h in range(Hkv):
        for d in (0, 7, 8, 127):
            assert k_pool[blk, h, d // 8, off, d % 8] == key[0, h, d]
            assert v_pool[blk, h, d, off] == val[0, h, d]
    assert np.count_nonzero(k_pool) == Hkv * D and np.count_nonzero(v_pool) == Hkv * D

    kv, ql = [70, 33, 16, 5, 32, 97], [3, 1, 16, 5, 1, 40]
    case = Case(kv, ql, 8, 2, 512 // bs, seed=24, bs=bs)
    k_pool, v_pool = case.pools_after_write()
    ref = numpy_reference.paged_attention(case.q, k_pool, v_pool, case.block_tables, case.kv_lens,
                                          case.cu_q, case.Hq, case.Hkv, case.scale)
    np.testing.assert_allclose(attention_oracle(case, k_pool, v_pool), ref, rtol=0, atol=2e-6)
    # the same tokens through 16-token blocks give the same rows: block size is layout only
    case16 = Case(kv, ql, 8, 2, 32, seed=24)
    k16, v16 = case16.pools_after_write()
    assert (case16.q == case.q).all() and (case16.k_all == case.k_all).all()
    np.testing.assert_allclose(attention_oracle(case16, k16, v16), attention_oracle(case, k_pool, v_pool),
                               rtol=0, atol=1e-6)


@pytest.mark.parametrize("hd", [32, 64, 80, 96, 112, 120, 192, 256])
def test_other_head_sizes_against_numpy_reference_and_index_formula(hd):
    """The other head sizes that are built (of those PagedAttentionConfig accepts,
    crates/mlx-paged-attn/src/config.rs:47-50): element (h, d) of the token in slot 50 lands at
    K[3, h, d//8, 2, d%8] and V[3, h, d, 2]; attention agrees with the numpy statement."""
    Hkv, NB = 2, 5
    k_pool = np.zeros((NB, Hkv, hd // X, BS, X), dtype=np.uint16)
    v_pool = np.zeros((NB, Hkv, hd, BS), dtype=np.uint16)
    key = np.arange(1, Hkv * hd + 1, dtype=np.uint16).reshape(1, Hkv, hd)
    val = (key + 1000).astype(np.uint16)
    write_oracle(k_pool, v_pool, key, val, np.array([50], dtype=np.int64), Hkv)
    for h in range(Hkv):
        for d in (0, 7, 8, hd - 1):
            assert k_pool[3, h, d // 8, 2, d % 8] == key[0, h, d]
            assert v_pool[3, h, d, 2] == val[0, h, d]
    assert np.count_nonzero(k_pool) == Hkv * hd and np.count_nonzero(v_pool) == Hkv * hd
    for f16 in (False, True):
        case = Case([70, 33, 16, 5, 32, 97], [3, 1, 16, 5, 1, 40], 8, 2, 32, seed=25, f16=f16, head_size=hd)
        assert case.q.shape[-1] == hd and abs(case.scale - hd ** -0.5) < 1e-12
        k_pool, v_pool = case.pools_after_write()
        ref = numpy_reference.paged_attention(case.q, k_pool, v_pool, case.block_tables, case.kv_lens,
                                              case.cu_q, case.Hq, case.Hkv, case.scale, f16=f16)
        got = attention_oracle(case, k_pool, v_pool)
        assert got.shape == (case.total_q, 8, hd)
        np.testing.assert_allclose(got, ref, rtol=0, atol=2e-6)


def test_f16_inputs_against_numpy_reference():
    case = Case([70, 33, 16, 5], [3, 1, 16, 5], 8, 2, 16, seed=23, f16=True)
    k_pool, v_pool = case.pools_after_write()
    ref = numpy_reference.paged_attention(case.q, k_pool, v_pool, case.block_tables, case.kv_lens,
                                          case.cu_q, case.Hq, case.Hkv, case.scale, f16=True)
    np.testing.assert_allclose(attention_oracle(case, k_pool, v_pool), ref, rtol=0, atol=2e-6)


@pytest.mark.parametrize("name", sorted(make_golden.PRODUCER_CASES))
def test_producer_oracle_matches_golden(name):
    """QK norm + rotary embedding: the C oracle against the numpy-made fixture."""
    from pa_testlib import check_rotated, elems_to_f32, qk_norm_rope_oracle
    g = np.load(os.path.join(GOLDEN, name + ".npz"))
    c = make_golden.build_producer(name)
    assert make_golden.digest(c["x"], c["pos"]) == str(g["inputs_sha256"]), "seeded inputs changed"
    bits, bound = qk_norm_rope_oracle(c["x"], c["w"], c["eps"], c["pos"], c["base"], c["dims"],
                                      f16=c["f16"])
    exp = g["out"]
    exp_bits = exp.astype(np.float16).view(np.uint16) if c["f16"] else f32_to_bf16(exp)
    assert (elems_to_f32(exp_bits, c["f16"]) == exp).all()
    same = check_rotated(bits, exp_bits, bound, c["f16"], name)
    assert same >= 0.999
    # position 0 rotates by nothing: with no norm the row passes through bit for bit
    if c["w"] is None:
        assert (bits[0] == c["x"][0]).all()
    # elements beyond rope_dims are only normalised
    if c["dims"] < D:
        ref = numpy_reference.qk_norm_rope(c["x"], c["w"], c["eps"], np.zeros_like(c["pos"]),
                                           c["base"], c["dims"], f16=c["f16"])
        assert (elems_to_f32(bits, c["f16"])[..., c["dims"]:] == ref[..., c["dims"]:]).mean() >= 0.999


def test_producer_rotation_preserves_pair_norm_and_composes():
    """Size-independent properties: a rotation keeps a^2+b^2 of every pair (to rounding),
    and rotating by position p is the same as what the attention logits need:
    <rot(q,p), rot(k,p')> depends on p-p' only (checked for equal positions)."""
    from pa_testlib import elems_to_f32, qk_norm_rope_oracle
    x = normal_bf16((33, 2, D), 5, 1)
    pos = np.arange(33, dtype=np.int32) * 977
    bits, _ = qk_norm_rope_oracle(x, None, 1e-6, pos, 1e6, D)
    a, r = bf16_to_f32(x).astype(np.float64), bf16_to_f32(bits).astype(np.float64)
    n_in = a[..., :64] ** 2 + a[..., 64:] ** 2
    n_out = r[..., :64] ** 2 + r[..., 64:] ** 2
    np.testing.assert_allclose(n_out, n_in, rtol=2 ** -6, atol=1e-3)
    y = normal_bf16((33, 2, D), 6, 1)
    ybits, _ = qk_norm_rope_oracle(y, None, 1e-6, pos, 1e6, D)
    dot_in = (a * bf16_to_f32(y)).sum(-1)
    dot_out = (r * bf16_to_f32(ybits)).sum(-1)
    np.testing.assert_allclose(dot_out, dot_in, atol=0.25)
