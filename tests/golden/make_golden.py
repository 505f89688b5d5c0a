"""Regenerates tests/golden/*.npz.

The reference keeps no golden vector for the numerical result of its kernels,
so these fixtures pin the C oracle against an independent implementation
instead: expected outputs come from tests/numpy_reference.py (float64 numpy
following the reference's gather/transposes), inputs from the seeded case
builder.  Stored: the case parameters, a checksum of the inputs, the expected
pool bits after the write (as a checksum plus a sampled slice) and the expected
attention output in float32.

Run from the repository root:  python tests/golden/make_golden.py [case names]
"""
import hashlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))

import numpy_reference  # noqa: E402
from pa_testlib import Case  # noqa: E402

CASES = {
    # name: (kv_lens, q_lens, Hq, Hkv, NB, seed[, tokens per pool block = 16[, head size = 128]])
    "decode_g2": ([1, 15, 16, 17, 100, 33], [1, 1, 1, 1, 1, 1], 4, 2, 32, 11),
    "decode_g4": ([257, 64, 5, 300], [1, 1, 1, 1], 8, 2, 64, 12),
    "decode_g8": ([40, 129], [1, 1], 8, 1, 16, 13),
    "verify_g4": ([37, 70, 21], [5, 5, 1], 8, 2, 16, 14),
    "prefill_g4": ([96, 50], [64, 50], 4, 1, 16, 15),
    "mixed_block32": ([1, 31, 32, 33, 100, 75], [1, 1, 1, 3, 1, 40], 8, 2, 16, 16, 32),
    "mixed_block8": ([1, 7, 8, 9, 100, 75], [1, 1, 1, 3, 1, 40], 8, 2, 64, 17, 8),
    # ... [, head size = 128]: other head sizes and group sizes that are not powers of two
    "decode_g5_head64": ([1, 16, 17, 300, 45], [1, 1, 1, 1, 1], 10, 2, 32, 18, 16, 64),
    "mixed_g3_head256": ([33, 70, 21, 90], [1, 2, 1, 30], 6, 2, 16, 19, 16, 256),
    "decode_g7_head120": ([5, 129, 64], [1, 1, 1], 7, 1, 16, 20, 16, 120),
}


# Producer (QK norm + rotary embedding) fixtures: name -> (T, H, seed, rope_base, rope_dims,
# eps, with_weight, f16).  Positions are seeded, spread over [0, 40000).
PRODUCER_CASES = {
    "producer_bf16_norm": (19, 6, 21, 1.0e6, 128, 1e-6, True, False),
    "producer_bf16_partial": (7, 3, 22, 1.0e4, 64, 1e-5, True, False),
    "producer_f16_nonorm": (9, 4, 23, 1.0e6, 128, 1e-6, False, True),
}


def build_producer(name):
    """Seeded producer inputs: x [T, H, 128], weight [128] (or None), positions [T]."""
    from pa_testlib import normal_bf16, normal_f16, bf16_to_f32, f32_to_bf16
    T, H, seed, base, dims, eps, with_w, f16 = PRODUCER_CASES[name]
    gen = normal_f16 if f16 else normal_bf16
    x = gen((T, H, 128), seed, 1)
    w = None
    if with_w:
        wf = 1.0 + 0.25 * bf16_to_f32(normal_bf16((128,), seed, 2))
        w = wf.astype(np.float16).view(np.uint16) if f16 else f32_to_bf16(wf)
    rng = np.random.Generator(np.random.PCG64(seed))
    pos = rng.integers(0, 40000, size=T).astype(np.int32)
    pos[0] = 0
    return dict(x=x, w=w, pos=pos, base=base, dims=dims, eps=eps, f16=f16)


def digest(*arrays) -> str:
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def build(name):
    kv, ql, Hq, Hkv, NB, seed, *rest = CASES[name]
    return Case(kv, ql, Hq, Hkv, NB, seed=seed, bs=rest[0] if rest else 16,
                head_size=rest[1] if len(rest) > 1 else 128)


def main():
    only = set(sys.argv[1:])  # names to regenerate; none = all
    for name in CASES:
        if only and name not in only:
            continue
        case = build(name)
        k_pool, v_pool = case.pools_after_write()
        # pool after the write, by fancy indexing (no shared index arithmetic)
        k_exp = case.k_pool.copy()
        v_exp = case.v_pool.copy()
        blk, off = case.slots_all // case.bs, case.slots_all % case.bs
        k_exp[blk, :, :, off, :] = case.k_all.reshape(-1, case.Hkv, case.D // 8, 8)
        v_exp[blk, :, :, off] = case.v_all
        assert (k_exp == k_pool).all() and (v_exp == v_pool).all(), name
        out = numpy_reference.paged_attention(case.q, k_exp, v_exp, case.block_tables,
                                              case.kv_lens, case.cu_q, Hq=case.Hq, Hkv=case.Hkv,
                                              scale=case.scale).astype(np.float32)
        out_cap = numpy_reference.paged_attention(case.q, k_exp, v_exp, case.block_tables,
                                                  case.kv_lens, case.cu_q, Hq=case.Hq,
                                                  Hkv=case.Hkv, scale=case.scale,
                                                  softcap=30.0).astype(np.float32)
        np.savez_compressed(
            os.path.join(HERE, name + ".npz"),
            inputs_sha256=digest(case.q, case.k_all, case.v_all, case.block_tables),
            pools_sha256=digest(k_exp, v_exp), k_pool_block0=k_exp[case.block_tables[0, 0]],
            v_pool_block0=v_exp[case.block_tables[0, 0]], out=out, out_softcap30=out_cap)
        print(name, out.shape)
    for name in PRODUCER_CASES:
        if only and name not in only:
            continue
        c = build_producer(name)
        out = numpy_reference.qk_norm_rope(c["x"], c["w"], c["eps"], c["pos"], c["base"], c["dims"],
                                           f16=c["f16"]).astype(np.float32)
        np.savez_compressed(os.path.join(HERE, name + ".npz"),
                            inputs_sha256=digest(c["x"], c["pos"]), out=out)
        print(name, out.shape)


if __name__ == "__main__":
    main()
