"""The decode entry for callers that cannot allocate device memory
(pa_paged_attention_decode_static) must give what the ordinary entry gives.

It keeps its split-KV partial results in an array inside the library image
rather than in a workspace the caller allocates, and every call shares that
array, so the check is made on two different batches back to back: if the
second call picked up anything the first one left behind, it would show.
This file sorts last on purpose, so a failure here cannot hide another test's.
"""
import numpy as np
import pytest
import torch

from gpu_util import DeviceCase, to_bits
from pa_testlib import Case, D, bf16_to_f32

pytestmark = pytest.mark.gpu


def both_entries(case):
    dc = DeviceCase(case)
    dc.write()
    want = torch.full((case.S, case.Hq, D), float("nan"), dtype=torch.bfloat16, device="cuda")
    got = torch.full_like(want, float("nan"))
    dc.cache.decode(want, dc.q, dc.tables, dc.lens, case.S, case.Hq, case.MB, case.scale, dc.ws,
                    dc.ws_bytes)
    dc.cache.decode_static(got, dc.q, dc.tables, dc.lens, case.S, case.Hq, case.MB, case.scale)
    torch.cuda.synchronize()
    dc.cache.check_errors()
    return bf16_to_f32(to_bits(got)), bf16_to_f32(to_bits(want))


def test_static_scratch_entry_matches_workspace_entry(cuda_device):
    # first batch: long contexts, so that items are split across CTAs and the
    # partial slots are really used
    first = Case([9000, 300, 4100, 17, 2500, 12000], [1] * 6, 32, 8, 2048, seed=101)
    got, want = both_entries(first)
    assert np.isfinite(want).all()
    # same kernel, same partition, same merge order: the results are identical,
    # which is well inside the 2e-2 / 1e-2 tolerance the parity tests use
    assert np.array_equal(got, want)
    # second batch right after, different shapes and lengths, same shared scratch
    second = Case([700, 16000, 33, 5000], [1] * 4, 64, 8, 2048, seed=102)
    got2, want2 = both_entries(second)
    assert np.isfinite(want2).all()
    assert np.array_equal(got2, want2)
    assert np.abs(want2).max() > 0
