"""Shared test infrastructure: the oracle binding, seeded case builders and the
parity rule.  Only tests, the smoke check and the benchmark's CPU-baseline leg
import this module."""
from __future__ import annotations

import ctypes as C
import math
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG_DIR = os.path.join(ROOT, "mlx-node_b200")
if PKG_DIR not in sys.path:
    sys.path.insert(0, PKG_DIR)

ORACLE_DIR = os.path.join(ROOT, "oracle")
ORACLE_LIB = os.path.join(ORACLE_DIR, "liboracle.so")

D = 128
BS = 16
X = 8
CANARY = 0x7FFF  # bf16 NaN pattern in never-written pool slots

_oracle = None


def oracle() -> C.CDLL:
    global _oracle
    if _oracle is not None:
        return _oracle
    if not os.path.exists(ORACLE_LIB):
        subprocess.run(["make", "-C", ORACLE_DIR], check=True, capture_output=True)
    lib = C.CDLL(ORACLE_LIB)
    vp, i32, i64, f32 = C.c_void_p, C.c_int32, C.c_int64, C.c_float
    lib.oracle_num_threads.restype = i32
    lib.oracle_set_num_threads.argtypes = [i32]
    lib.oracle_set_num_threads.restype = None
    lib.oracle_reshape_and_cache.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, i32, i32, i32, i32]
    lib.oracle_reshape_and_cache.restype = None
    lib.oracle_copy_blocks.argtypes = [vp, vp, vp, i64, i64]
    lib.oracle_copy_blocks.restype = None
    lib.oracle_paged_attention_varlen.argtypes = [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32,
                                                  i32, i32, i64, f32, f32]
    lib.oracle_paged_attention_varlen.restype = None
    lib.oracle_paged_attention_varlen_dt.argtypes = [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32,
                                                     i32, i32, i64, f32, f32, i32]
    lib.oracle_paged_attention_varlen_dt.restype = None
    lib.oracle_paged_attention_rows.argtypes = [vp, vp, i32, vp, vp, vp, vp, vp, vp, i32, i32, i32,
                                                i32, i32, i64, f32, f32]
    lib.oracle_paged_attention_rows.restype = None
    lib.oracle_dense_causal.argtypes = [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, f32]
    lib.oracle_dense_causal.restype = None
    lib.baseline_mlx_paged_forward.argtypes = [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32,
                                               i32, f32]
    lib.baseline_mlx_paged_forward.restype = i32
    lib.oracle_fill_normal_bf16.argtypes = [vp, i64, C.c_uint64, C.c_uint64, i64]
    lib.oracle_fill_normal_bf16.restype = None
    lib.oracle_fp8_e4m3_decode.argtypes = [C.c_uint8]
    lib.oracle_fp8_e4m3_decode.restype = f32
    lib.oracle_fp8_e4m3_encode.argtypes = [f32]
    lib.oracle_fp8_e4m3_encode.restype = C.c_uint8
    lib.oracle_reshape_and_cache_fp8.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, i32, i32, i32,
                                                 f32, f32, i32]
    lib.oracle_reshape_and_cache_fp8.restype = None
    lib.oracle_paged_attention_varlen_fp8.argtypes = [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32,
                                                      i32, i32, i64, f32, f32, i32, f32, f32]
    lib.oracle_paged_attention_varlen_fp8.restype = None
    lib.oracle_qk_norm_rope.argtypes = [vp, vp, vp, i64, vp, C.c_double, vp, C.c_double, i32, i64,
                                        i32, i32, i32]
    lib.oracle_qk_norm_rope.restype = None
    lib.oracle_paged_attention_metal.argtypes = [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, f32, f32, i32]
    lib.oracle_paged_attention_metal.restype = None
    lib.oracle_f32_to_bf16.argtypes = [vp, vp, i64]
    lib.oracle_f32_to_bf16.restype = None
    lib.oracle_bf16_to_f32.argtypes = [vp, vp, i64]
    lib.oracle_bf16_to_f32.restype = None
    _oracle = lib
    return lib


def p(a: np.ndarray) -> int:
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data


# ---- bf16 <-> numpy ----------------------------------------------------------------
def bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    """Round to nearest even, NaN -> 0x7FC0 (crates/mlx-paged-attn/metal/utils.metal:14-27)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r = ((u.astype(np.uint64) + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    r[nan] = 0x7FC0
    return r


def normal_bf16(shape, seed: int, stream: int) -> np.ndarray:
    """Seeded N(0,1) bf16 bit patterns from the oracle's counter-based generator."""
    out = np.empty(shape, dtype=np.uint16)
    oracle().oracle_fill_normal_bf16(p(out), out.size, seed, stream, 0)
    return out


def normal_f16(shape, seed: int, stream: int) -> np.ndarray:
    """The same seeded values as f16 bit patterns (bf16 values are exact in f16 here)."""
    return bf16_to_f32(normal_bf16(shape, seed, stream)).astype(np.float16).view(np.uint16)


def elems_to_f32(bits: np.ndarray, f16: bool) -> np.ndarray:
    return bits.view(np.float16).astype(np.float32) if f16 else bf16_to_f32(bits)


# ---- case construction ---------------------------------------------------------------
class Case:
    """One seeded workload: pool pre-filled with every sequence's prefix, the
    step's new tokens and queries held apart for the code under test."""

    def __init__(self, kv_lens, q_lens, Hq, Hkv, NB, seed=0, mb_extra=0, prefill=True, f16=False,
                 bs=BS, head_size=D):
        self.f16 = f16
        self.bs = bs  # tokens per pool block (16 or 32)
        self.D = head_size  # the module constant D (128) unless a test says otherwise
        D_ = head_size
        self.S = len(kv_lens)
        self.Hq, self.Hkv, self.NB = Hq, Hkv, NB
        self.G = Hq // Hkv
        self.kv_lens = np.asarray(kv_lens, dtype=np.int32)
        self.q_lens = np.asarray(q_lens, dtype=np.int32)
        assert (self.q_lens <= self.kv_lens).all()
        self.cu_q = np.zeros(self.S + 1, dtype=np.int32)
        self.cu_q[1:] = np.cumsum(self.q_lens)
        self.total_q = int(self.cu_q[-1])
        nblk = (self.kv_lens + bs - 1) // bs
        assert int(nblk.sum()) <= NB, "pool too small"
        rng = np.random.Generator(np.random.PCG64(seed))
        perm = rng.permutation(NB).astype(np.int32)
        self.MB = max(int(nblk.max()) if self.S else 1, 1) + mb_extra
        self.block_tables = np.zeros((self.S, self.MB), dtype=np.int32)  # zero padded
        pos = 0
        for s in range(self.S):
            self.block_tables[s, :nblk[s]] = perm[pos:pos + nblk[s]]
            pos += nblk[s]
        self.scale = 1.0 / math.sqrt(D_)
        # tensors
        gen = normal_f16 if f16 else normal_bf16
        self.q = gen((self.total_q, Hq, D_), seed, 1)
        tot_kv = int(self.kv_lens.sum())
        self.cu_kv = np.zeros(self.S + 1, dtype=np.int32)
        self.cu_kv[1:] = np.cumsum(self.kv_lens)
        self.k_all = gen((tot_kv, Hkv, D_), seed, 2)  # every token of every sequence
        self.v_all = gen((tot_kv, Hkv, D_), seed, 3)
        slots_all = np.empty(tot_kv, dtype=np.int64)
        is_new = np.zeros(tot_kv, dtype=bool)
        for s in range(self.S):
            t = np.arange(self.kv_lens[s])
            slots_all[self.cu_kv[s]:self.cu_kv[s + 1]] = (
                self.block_tables[s, t // bs].astype(np.int64) * bs + t % bs)
            is_new[self.cu_kv[s + 1] - self.q_lens[s]:self.cu_kv[s + 1]] = True
        self.slots_all = slots_all
        self.k_new = np.ascontiguousarray(self.k_all[is_new])
        self.v_new = np.ascontiguousarray(self.v_all[is_new])
        self.slot_mapping = np.ascontiguousarray(slots_all[is_new])
        self.k_pool = np.full((NB, Hkv, D_ // X, bs, X), CANARY, dtype=np.uint16)
        self.v_pool = np.full((NB, Hkv, D_, bs), CANARY, dtype=np.uint16)
        if prefill:
            old = ~is_new
            write_oracle(self.k_pool, self.v_pool, np.ascontiguousarray(self.k_all[old]),
                         np.ascontiguousarray(self.v_all[old]),
                         np.ascontiguousarray(slots_all[old]), Hkv)

    def pools_after_write(self):
        k, v = self.k_pool.copy(), self.v_pool.copy()
        write_oracle(k, v, self.k_new, self.v_new, self.slot_mapping, self.Hkv)
        return k, v


def write_oracle(k_pool, v_pool, key, value, slots, Hkv, key_stride=None, value_stride=None):
    n = len(slots)
    if n == 0:
        return
    hd = v_pool.shape[2]  # head size
    oracle().oracle_reshape_and_cache(p(key), p(value), p(k_pool), p(v_pool), p(slots), n,
                                      key_stride or Hkv * hd, value_stride or Hkv * hd, Hkv, hd,
                                      k_pool.shape[3], X)


def attention_oracle(case: Case, k_pool, v_pool, softcap=1.0, varlen=True) -> np.ndarray:
    hd = v_pool.shape[2]  # head size
    out = np.zeros((case.total_q, case.Hq, hd), dtype=np.float32)
    cu = p(case.cu_q) if varlen else None
    oracle().oracle_paged_attention_varlen_dt(p(out), p(case.q), p(k_pool), p(v_pool),
                                              p(case.block_tables), p(case.kv_lens), cu, case.S,
                                              case.Hq, case.Hkv, hd, k_pool.shape[3], case.MB,
                                              case.Hq * hd, case.scale, softcap, int(case.f16))
    return out


def attention_oracle_metal(case: Case, k_pool, v_pool, softcap=1.0) -> np.ndarray:
    """The reference Metal kernels' own arithmetic (oracle/metal_arithmetic.c) on a decode
    case with 16-token blocks: T-typed output as float32 [S, Hq, D]."""
    assert (case.q_lens == 1).all() and k_pool.shape[3] == 16
    out = np.zeros((case.S, case.Hq, D), dtype=np.uint16)
    oracle().oracle_paged_attention_metal(p(out), p(case.q), p(k_pool), p(v_pool), p(case.block_tables),
                                          p(case.kv_lens), case.S, case.Hq, case.Hkv, case.MB,
                                          case.scale, softcap, int(case.f16))
    return elems_to_f32(out, case.f16)


def attention_oracle_rows(rows, q, k_pool, v_pool, block_tables, kv_lens, cu_q, Hq, Hkv, MB, scale,
                          softcap=1.0) -> np.ndarray:
    rows = np.ascontiguousarray(rows, dtype=np.int32).reshape(-1, 3)
    out = np.zeros((len(rows), D), dtype=np.float32)
    oracle().oracle_paged_attention_rows(p(out), p(rows), len(rows), p(q), p(k_pool), p(v_pool),
                                         p(block_tables), p(kv_lens),
                                         p(cu_q) if cu_q is not None else None, Hq, Hkv, D,
                                         k_pool.shape[3], MB,
                                         Hq * D, scale, softcap)
    return out


# ---- FP8 (E4M3) cache ----------------------------------------------------------------
X8 = 16  # elements per 16-byte piece of the FP8 key pool


def fp8_pools(NB, Hkv, fill=0, bs=BS):
    return (np.full((NB, Hkv, D // X8, bs, X8), fill, dtype=np.uint8),
            np.full((NB, Hkv, D, bs), fill, dtype=np.uint8))


def write_oracle_fp8(k_pool8, v_pool8, key, value, slots, Hkv, k_scale, v_scale, f16=False):
    n = len(slots)
    if n:
        oracle().oracle_reshape_and_cache_fp8(p(key), p(value), p(k_pool8), p(v_pool8), p(slots), n,
                                              Hkv * D, Hkv * D, Hkv, D, k_pool8.shape[3], k_scale,
                                              v_scale, int(f16))


def attention_oracle_fp8(case, k_pool8, v_pool8, k_scale, v_scale, softcap=1.0, varlen=True):
    out = np.zeros((case.total_q, case.Hq, D), dtype=np.float32)
    cu = p(case.cu_q) if varlen else None
    oracle().oracle_paged_attention_varlen_fp8(p(out), p(case.q), p(k_pool8), p(v_pool8),
                                               p(case.block_tables), p(case.kv_lens), cu, case.S,
                                               case.Hq, case.Hkv, D, k_pool8.shape[3], case.MB,
                                               case.Hq * D, case.scale, softcap, int(case.f16), k_scale,
                                               v_scale)
    return out


def qk_norm_rope_oracle(x_bits, weight_bits, eps, positions, rope_base, rope_dims, f16=False):
    """Oracle for the producer on x [T, H, D]: returns (rotated bits, per-element bound base
    |a|+|b| of the rotated pair)."""
    T, H, _ = x_bits.shape
    x_bits = np.ascontiguousarray(x_bits)
    out = np.empty_like(x_bits)
    bound = np.empty(x_bits.shape, dtype=np.float32)
    positions = np.ascontiguousarray(positions, dtype=np.int32)
    oracle().oracle_qk_norm_rope(p(out), p(bound), p(x_bits), H * D,
                                 p(weight_bits) if weight_bits is not None else None, eps,
                                 p(positions), rope_base, rope_dims, T, H, D, int(f16))
    return out, bound


def check_rotated(got_bits, ref_bits, bound, f16, what=""):
    """The producer's fp32 steps (mean of squares, reciprocal square root, sine and
    cosine) are evaluated by different routines on the two sides, so a value that sits
    on a rounding boundary can land one unit in the last place apart after the norm and
    carry that through the rotation: |a-b| <= 2^-7 (bf16) / 2^-10 (f16) of the pair's
    magnitude |a|+|b|, and at least 99 % of the elements identical."""
    got = elems_to_f32(got_bits, f16).astype(np.float64)
    ref = elems_to_f32(ref_bits, f16).astype(np.float64)
    ulp = 2.0 ** (-10 if f16 else -7)
    floor = np.maximum(bound.astype(np.float64), np.abs(ref))
    bad = np.abs(got - ref) > ulp * floor + 1e-30
    same = float((got_bits == ref_bits).mean())
    assert not bad.any(), f"{what}: {int(bad.sum())} elements beyond one unit in the last place; " \
                          f"worst {np.abs(got - ref).max()}"
    assert same >= 0.99, f"{what}: only {same:.4f} of the elements identical"
    return same


# ---- parity rule ------------------------------------------------------------------------
ATOL = 2e-2   # max-abs bound stated for the path
RTOL = 1e-2   # max-rel bound, applied with a per-row RMS floor


def check_attention(got_f32: np.ndarray, ref_f32: np.ndarray, what: str = "") -> dict:
    """bf16 output with fp32 accumulation vs the fp64-accumulated oracle:
    (i) max|a-b| <= 2e-2;
    (ii) |a-b| <= 1e-2*|ref| + 1e-2*rms(row) element-wise, where a row is the D
    outputs of one (query, head).  The floor is per row because a batch mixes
    short contexts (outputs ~0.3) with long ones (outputs ~0.01): a global floor
    would be loose for the long rows and meaningless for the short ones, and a
    pure relative test would be dominated by elements that happen to be near 0."""
    hd = ref_f32.shape[-1] if ref_f32.ndim > 1 else D  # a row = the outputs of one (query, head)
    got = got_f32.astype(np.float64).reshape(-1, hd)
    ref = ref_f32.astype(np.float64).reshape(-1, hd)
    assert got.shape == ref.shape
    assert np.isfinite(got).all(), f"{what}: non-finite values in the output"
    if ref.size == 0:
        return {"max_abs": 0.0, "max_over_bound": 0.0, "rms_ref": 0.0}
    diff = np.abs(got - ref)
    rms = np.sqrt(np.mean(ref * ref, axis=1, keepdims=True))
    bound = RTOL * np.abs(ref) + RTOL * rms
    ratio = diff / np.maximum(bound, 1e-30)
    ratio[(diff == 0)] = 0.0
    worst = np.unravel_index(int(np.argmax(ratio)), ratio.shape)
    stats = {"max_abs": float(diff.max()), "rms_ref": float(np.sqrt(np.mean(ref * ref))),
             "max_over_bound": float(ratio.max()), "worst_row": int(worst[0])}
    assert stats["max_abs"] <= ATOL, f"{what}: max abs error {stats['max_abs']:.3e} > {ATOL}"
    assert stats["max_over_bound"] <= 1.0, (
        f"{what}: row {worst[0]} dim {worst[1]}: got {got[worst]:.6f} ref {ref[worst]:.6f} "
        f"|diff| {diff[worst]:.3e} > bound {bound[worst]:.3e} (row rms {rms[worst[0], 0]:.3e})")
    return stats


# ---- the five benchmark configurations (lengths only; seeded) ---------------------------
from paged_attn_b200.workloads import config_lengths  # noqa: E402,F401  (tests use it from here)
