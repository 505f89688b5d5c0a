"""CPU tests of the oracle's FP8 (E4M3) cache functions: the byte format against an
independent numpy statement (decode table, nearest-value encoding in the normal range,
the stated behaviour outside it), the write's index arithmetic against fancy indexing,
and attention over an FP8 pool against float64 numpy on the dequantised values."""
import numpy as np
import pytest

from pa_testlib import (BS, D, X8, Case, attention_oracle_fp8, bf16_to_f32, fp8_pools, normal_bf16,
                        oracle, write_oracle_fp8)


def decode_table():
    """All 256 codes by the format's definition (bias 7; exponent 15 = inf / NaN)."""
    t = np.empty(256, dtype=np.float64)
    for c in range(256):
        s, e, m = c >> 7, (c >> 3) & 15, c & 7
        if e == 0:
            v = m / 8 * 2.0 ** -6
        elif e == 15:
            v = np.nan if m else np.inf
        else:
            v = (1 + m / 8) * 2.0 ** (e - 7)
        t[c] = -v if s else v
    return t


def enc(x):
    return int(oracle().oracle_fp8_e4m3_encode(float(np.float32(x))))


def test_decode_all_codes():
    t = decode_table()
    got = np.array([oracle().oracle_fp8_e4m3_decode(c) for c in range(256)], dtype=np.float64)
    assert np.array_equal(np.isnan(got), np.isnan(t))
    assert (got[~np.isnan(t)] == t[~np.isnan(t)]).all()
    assert t[0x77] == 240.0 and t[0x78] == np.inf and t[0x08] == 2.0 ** -6


def test_encode_round_trips_every_finite_code():
    t = decode_table()
    for c in range(256):
        if np.isfinite(t[c]):
            assert enc(t[c]) == c, hex(c)


def test_encode_normal_range_is_nearest_even():
    t = decode_table()
    pos = np.array([c for c in range(0x08, 0x78)])          # positive normal codes, ascending
    vals = t[pos]
    rng = np.random.Generator(np.random.PCG64(3))
    xs = np.exp(rng.uniform(np.log(2.0 ** -6), np.log(240.0), size=4000)).astype(np.float32)
    # exact midpoints between neighbours too (ties go to the even mantissa)
    mids = ((vals[:-1] + vals[1:]) / 2).astype(np.float32)
    for x in np.concatenate([xs, mids]):
        i = np.searchsorted(vals, x)
        cands = [j for j in (i - 1, i) if 0 <= j < len(vals)]
        best = min(cands, key=lambda j: (abs(vals[j] - float(x)), pos[j] & 1))
        assert enc(x) == pos[best], float(x)
        assert enc(-x) == pos[best] | 0x80


def test_encode_outside_the_normal_range():
    # overflow of the rounding goes to the infinity code; 240 itself is the largest finite
    assert enc(240.0) == 0x77 and enc(247.9) == 0x77 and enc(248.0) == 0x78 and enc(255.0) == 0x78
    assert enc(np.inf) == 0x78 and enc(-np.inf) == 0xF8 and enc(np.nan) & 0x7F == 0x79
    # below normal: spacing 2^-9, round half up
    assert enc(2.0 ** -9) == 0x01 and enc(1.5 * 2.0 ** -9) == 0x02 and enc(1.49 * 2.0 ** -9) == 0x01
    # ... but everything below 2^-9 is cut to zero before any rounding
    assert enc(0.4 * 2.0 ** -9) == 0x00 and enc(0.99 * 2.0 ** -9) == 0x00
    # a value that would round up to the smallest normal number comes out as zero
    assert enc(7.5 * 2.0 ** -9) == 0x00 and enc(7.49 * 2.0 ** -9) == 0x07
    assert enc(0.0) == 0 and enc(-0.0) == 0x80
    # magnitudes of 256 and above take the below-normal branch: low bits of the shifted
    # mantissa, exponent field 0 (kept as the reference computes it)
    for x in (256.0, 300.0, 1000.0, 16383.0):
        bits = np.float32(x).view(np.uint32)
        e8 = int((bits >> 23) & 0xFF) - 120
        rshift = 21 - e8
        want = (((0x800000 | int(bits & 0x7FFFFF)) + (1 << (rshift - 1))) >> rshift) & 7
        assert enc(x) == want, x
    assert enc(16384.0) == 0x78 and enc(-1e9) == 0xF8


@pytest.mark.parametrize("f16", [False, True])
def test_fp8_write_matches_fancy_indexing(f16):
    case = Case([37, 70, 21], [5, 5, 1], 8, 2, 16, seed=71, f16=f16)
    k8, v8 = fp8_pools(case.NB, case.Hkv, fill=0xAA)
    ks, vs = 0.37, 2.5
    write_oracle_fp8(k8, v8, case.k_all, case.v_all, case.slots_all, case.Hkv, ks, vs, f16)

    def quant(bits, scale):
        x = bits.view(np.float16).astype(np.float32) if f16 else bf16_to_f32(bits)
        y = (x / np.float32(scale)).astype(np.float32)
        y = y.astype(np.float16).astype(np.float32) if f16 else bf16_to_f32(
            __import__("pa_testlib").f32_to_bf16(y))
        return np.array([enc(v) for v in y.ravel()], dtype=np.uint8).reshape(y.shape)

    kq, vq = quant(case.k_all, ks), quant(case.v_all, vs)
    blk, off = case.slots_all // BS, case.slots_all % BS
    k_exp, v_exp = fp8_pools(case.NB, case.Hkv, fill=0xAA)
    k_exp[blk, :, :, off, :] = kq.reshape(-1, case.Hkv, D // X8, X8)
    v_exp[blk, :, :, off] = vq
    assert (k_exp == k8).all() and (v_exp == v8).all()


def test_fp8_attention_oracle_against_numpy():
    case = Case([40, 129, 16, 5], [1, 4, 1, 5], 8, 2, 32, seed=72)
    k8, v8 = fp8_pools(case.NB, case.Hkv)
    ks, vs = 0.5, 0.75
    write_oracle_fp8(k8, v8, case.k_all, case.v_all, case.slots_all, case.Hkv, ks, vs)
    got = attention_oracle_fp8(case, k8, v8, ks, vs)
    t = decode_table()
    q = bf16_to_f32(case.q).astype(np.float64)
    G = case.Hq // case.Hkv
    for s in range(case.S):
        n = int(case.kv_lens[s])
        nb = (n + BS - 1) // BS
        blocks = case.block_tables[s, :nb]
        k = t[k8[blocks]].transpose(1, 0, 3, 2, 4).reshape(case.Hkv, nb * BS, D)[:, :n] * ks
        v = t[v8[blocks]].transpose(1, 0, 3, 2).reshape(case.Hkv, nb * BS, D)[:, :n] * vs
        ql = int(case.q_lens[s])
        for j in range(ql):
            lim = n - ql + j + 1
            for hq in range(case.Hq):
                h = hq // G
                logits = (k[h, :lim] @ q[case.cu_q[s] + j, hq]) * case.scale
                w = np.exp(logits - logits.max())
                ref = (w / w.sum()) @ v[h, :lim]
                np.testing.assert_allclose(got[case.cu_q[s] + j, hq], ref, rtol=0, atol=2e-6)
