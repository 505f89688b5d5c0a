"""How far the reference Metal kernels' own arithmetic is from the exact-softmax oracle.

The oracle the parity tests use (oracle/paged_oracle.c) follows the semantics of the
reference's software path with an exact softmax in fp64.  The reference's Metal decode
kernels compute the same thing with their own rounding: 1 / (sum + 1e-6) as normaliser,
probabilities rounded to the storage type and the eight products of a 16-byte V piece
formed in the storage type (crates/mlx-paged-attn/metal/attention/paged_attention.metal
:986-999, 1016-1084, 1191-1259).  oracle/metal_arithmetic.c restates that arithmetic;
these tests measure the distance on every decode fixture and pin it, so that "the oracle
deviates from the Metal kernels by a precision loss only" is a number, not a claim:
    bf16:  |exact - metal| <= 2.5e-2 * rms(row)   (the 1e-2 parity rule is EXCEEDED by the
           reference's own bf16 arithmetic on some elements: up to 1.3 x its bound)
    f16:   |exact - metal| <= 5e-3 * rms(row)
"""
import os

import numpy as np
import pytest

from golden import make_golden
from pa_testlib import D, Case, attention_oracle, attention_oracle_metal

BOUND = {False: 2.5e-2, True: 5e-3}   # of the row's rms, by storage type (bf16, f16)


def distance(case, softcap=1.0):
    k, v = case.pools_after_write()
    exact = attention_oracle(case, k, v, softcap=softcap, varlen=False).reshape(-1, D).astype(np.float64)
    metal = attention_oracle_metal(case, k, v, softcap=softcap).reshape(-1, D).astype(np.float64)
    assert np.isfinite(metal).all()
    rms = np.sqrt((exact ** 2).mean(axis=1, keepdims=True))
    live = rms[:, 0] > 0
    rel = (np.abs(exact - metal)[live] / rms[live]).max()
    return float(rel), float(np.abs(exact - metal).max())


# (the restatement follows the Metal kernel at its head-size-128 template constants)
DECODE_FIXTURES = [n for n in sorted(make_golden.CASES) if n.startswith("decode") and "head" not in n]


@pytest.mark.parametrize("name", DECODE_FIXTURES)
def test_metal_arithmetic_on_the_decode_fixtures(name):
    case = make_golden.build(name)
    rel, mx = distance(case)
    print(name, "max |exact - metal| / rms(row) =", rel, "max abs", mx)
    assert rel <= BOUND[bool(case.f16)]
    assert mx <= 2e-2
    rel_cap, _ = distance(case, softcap=30.0)
    assert rel_cap <= BOUND[bool(case.f16)]


@pytest.mark.parametrize("f16", [False, True])
def test_metal_arithmetic_v1_v2_and_block_edges(f16):
    # contexts around the block size and around the 512-token switch from the one-pass
    # kernel to partitions + reduce
    for kv in ([1, 15, 16, 17, 100, 300, 511, 512], [513, 700, 1029, 4097, 33], [2000, 9000]):
        case = Case(kv, [1] * len(kv), 32, 8, 1024, seed=5, f16=f16)
        rel, mx = distance(case)
        assert rel <= BOUND[f16] and mx <= 2e-2, (kv, rel, mx)


def test_bf16_metal_arithmetic_is_looser_than_the_parity_rule():
    """The parity rule (|a-b| <= 1e-2|ref| + 1e-2 rms) is tighter than what the
    reference's bf16 kernel arithmetic itself achieves against the exact result; the
    CUDA kernels are held to the rule, i.e. to less error than the reference's own."""
    case = Case([513, 700, 1029, 4097, 33], [1] * 5, 32, 8, 1024, seed=5)
    k, v = case.pools_after_write()
    exact = attention_oracle(case, k, v, varlen=False).reshape(-1, D).astype(np.float64)
    metal = attention_oracle_metal(case, k, v).reshape(-1, D).astype(np.float64)
    rms = np.sqrt((exact ** 2).mean(axis=1, keepdims=True))
    over = (np.abs(exact - metal) / (1e-2 * np.abs(exact) + 1e-2 * rms)).max()
    assert 1.0 < over < 2.0
