"""Head sizes other than 128 (crates/mlx-paged-attn/src/config.rs:47-50 accepts 32, 64, 80, 96,
112, 120, 128, 192, 256; all are built): KV write bit-exact, decode and multi-token attention
against the oracle.

What the library does with them: the write kernel and the split-KV kernel are compiled per
head size (16-bit pools; 16-token blocks, and 32-token blocks up to head size 128); the tcgen05
tile kernel, the FP8 cache, the fused norm + rotary + write launch and 8-token blocks are
head-size-128 code and are refused for the other sizes with PA_ERR_UNSUPPORTED.  Chunks too wide for the split-KV kernel (more
than 24 columns; 16 with head size 192, 8 with 256) are served as consecutive pieces, as with
8-token blocks."""
import numpy as np
import pytest
import torch

import paged_attn_b200 as pa
from gpu_util import DeviceCase, to_bits, to_dev
from pa_testlib import BS, Case, attention_oracle, check_attention, elems_to_f32

pytestmark = pytest.mark.gpu

INVALID_ARG, UNSUPPORTED = 1, 2   # pa_status values (include/paged_attn_b200.h)


def run_case(case, varlen=True, softcap=1.0):
    dc = DeviceCase(case)
    dc.write()
    torch.cuda.synchronize()
    k_ref, v_ref = case.pools_after_write()
    assert (to_bits(dc.k_pool) == k_ref).all(), "K pool differs from the oracle"
    assert (to_bits(dc.v_pool) == v_ref).all(), "V pool differs from the oracle"
    got = dc.attend(varlen=varlen, softcap=softcap)
    ref = attention_oracle(case, k_ref, v_ref, softcap=softcap, varlen=varlen)
    assert got.shape[-1] == case.D
    return got, ref


OTHER_SIZES = [32, 64, 80, 96, 112, 120, 192, 256]


@pytest.mark.parametrize("hd", OTHER_SIZES)
@pytest.mark.parametrize("f16", [False, True])
@pytest.mark.parametrize("G,Hkv", [(1, 2), (4, 8), (8, 4)])
def test_decode(cuda_device, hd, f16, G, Hkv):
    # context 1, one block exactly, k*BS +- 1, an empty sequence, and contexts long enough
    # to be split over many CTAs (the merge inside the launch)
    kv = [1, 16, 17, 31, 32, 33, 0, 700, 12000, 5000, 255]
    ql = [1 if n else 0 for n in kv]
    case = Case(kv, ql, G * Hkv, Hkv, 1400, seed=60 + hd + G, f16=f16, head_size=hd)
    # decode entry: one query row per sequence, empty ones included
    full_q = np.zeros((len(kv), G * Hkv, hd), dtype=np.uint16)
    full_q[np.asarray(ql) > 0] = case.q
    case.q, case.total_q = full_q, len(kv)
    case.cu_q = np.arange(len(kv) + 1, dtype=np.int32)
    got, ref = run_case(case, varlen=False)
    assert (got[np.asarray(kv) == 0] == 0).all()
    print(hd, f16, G, check_attention(got, ref, f"decode, head size {hd}"))
    got_cap, ref_cap = run_case(case, varlen=False, softcap=30.0)
    check_attention(got_cap, ref_cap, f"decode with soft cap, head size {hd}")


@pytest.mark.parametrize("hd", OTHER_SIZES)
def test_verify_and_chunks_in_one_call(cuda_device, hd):
    # decode + 5-token verify (20 columns) + prefill chunks: head sizes up to 112 take the
    # verify sequences in the wide split-KV variant, 192 and 256 cut them into pieces of 4 and
    # 2 tokens; the chunks go through the split-KV kernel in pieces for all of them
    kv = [1500, 3333, 16, 2053, 4101, 700, 300 + 77, 512 + 300]
    ql = [1, 1, 1, 5, 5, 5, 77, 300]
    case = Case(kv, ql, 32, 8, 1024, seed=70 + hd, head_size=hd)
    got, ref = run_case(case)
    print(hd, check_attention(got, ref, f"mixed batch, head size {hd}"))
    # run to run the same bits
    dc = DeviceCase(case)
    dc.write()
    assert (dc.attend() == got).all()


@pytest.mark.parametrize("hd", OTHER_SIZES)
def test_config2_shape_reduced(cuda_device, hd):
    # configuration-2-shaped decode (32 query / 8 kv heads), 12 sequences, whole output
    rng = np.random.Generator(np.random.PCG64(hd))
    kv = rng.integers(1024, 8193, 12)
    case = Case(kv, np.ones(12, int), 32, 8, 6200, seed=80 + hd, head_size=hd)
    got, ref = run_case(case, varlen=False)
    print(hd, check_attention(got, ref, f"configuration 2 reduced, head size {hd}"))


@pytest.mark.parametrize("hd", OTHER_SIZES)
def test_decode_step_runs_write_then_attention(cuda_device, hd):
    # the one-call decode step exists for every head size; the in-kernel write is
    # head-size-128 code, so here it is the write kernel followed by the attention kernel
    kv = [900, 17, 4000, 1, 16]
    case = Case(kv, [1] * 5, 16, 4, 512, seed=90 + hd, head_size=hd)
    dc = DeviceCase(case)
    out = torch.full((5, 16, hd), float("nan"), dtype=torch.bfloat16, device="cuda")
    dc.cache.decode_step(out, dc.q, dc.k_new, dc.v_new, dc.slots, dc.tables, dc.lens, 5, 16, case.MB,
                         case.scale, dc.ws, dc.ws_bytes)
    torch.cuda.synchronize()
    dc.cache.check_errors()
    k_ref, v_ref = case.pools_after_write()
    assert (to_bits(dc.k_pool) == k_ref).all() and (to_bits(dc.v_pool) == v_ref).all()
    check_attention(elems_to_f32(to_bits(out), False), attention_oracle(case, k_ref, v_ref, varlen=False),
                    f"decode step, head size {hd}")


@pytest.mark.parametrize("hd", [h for h in OTHER_SIZES if h <= 128])
def test_32_token_blocks(cuda_device, hd):
    """The reference's default block size (crates/mlx-paged-attn/src/config.rs:128) with the
    head sizes up to 128: a warp takes a whole 32-token block from one stage."""
    kv = [1, 15, 16, 17, 31, 32, 33, 47, 48, 49, 64, 255, 256, 257, 1000, 4097, 9000]
    case = Case(kv, [1] * len(kv), 32, 8, 600, seed=95 + hd, head_size=hd, bs=32)
    got, ref = run_case(case, varlen=False)
    print(hd, check_attention(got, ref, f"decode, 32-token blocks, head size {hd}"))
    # verify widths and a chunk (served in pieces) in one call
    kv2, ql2 = [700, 64, 1029, 300, 2500, 17, 300 + 40], [1, 2, 3, 6, 5, 1, 40]
    case2 = Case(kv2, ql2, 8, 2, 200, seed=96 + hd, head_size=hd, bs=32)
    got2, ref2 = run_case(case2)
    check_attention(got2, ref2, f"verify widths and a chunk, 32-token blocks, head size {hd}")


def test_what_is_refused(cuda_device):
    with pytest.raises(pa.PagedAttnError) as e:   # not one of the reference's either
        pa.PagedCache(BS, 8, 100, 2)
    assert e.value.status == INVALID_ARG
    for hd in OTHER_SIZES:
        for bs in (8, 32):
            if bs == 32 and hd <= 128:
                continue   # built: test_32_token_blocks
            with pytest.raises(pa.PagedAttnError) as e:
                pa.PagedCache(bs, 8, hd, 2)
            assert e.value.status == UNSUPPORTED
        with pytest.raises(pa.PagedAttnError) as e:
            pa.PagedCache(BS, 8, hd, 2, fp8=True)
        assert e.value.status == UNSUPPORTED
        # a chunk too wide for the split-KV kernel needs host context lengths to be cut up
        case = Case([400], [300], 8, 2, 64, seed=3, head_size=hd)
        dc = DeviceCase(case)
        dc.write()
        with pytest.raises(pa.PagedAttnError) as e:
            dc.attend(host_lens=False)
        assert e.value.status == INVALID_ARG
