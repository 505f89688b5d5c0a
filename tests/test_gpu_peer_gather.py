"""Head gather over peer memory.  The data path and the flag protocol are checked on one
GPU with the ranks' buffers side by side in its memory: every rank publishes first, the
waits come after, so no launch ever waits for one that has not been issued.  The run on
several GPUs (symmetric-memory buffers, checked against an NCCL all-gather) is in
bench.py --gather peer."""
import numpy as np
import pytest
import torch

import paged_attn_b200 as pa
from pa_testlib import BS, D

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world,hl,T", [(2, 4, 64), (4, 2, 33), (8, 1, 5), (1, 8, 7), (2, 4, 0)])
def test_publish_then_wait_fills_every_buffer(cuda_device, world, hl, T):
    cache = pa.PagedCache(BS, 8, D, 1)
    gen = torch.Generator(device="cuda").manual_seed(5)
    locals_ = [torch.randn(T, hl, D, generator=gen, device="cuda").to(torch.bfloat16)
               for _ in range(world)]
    # (T = 0: an empty step moves nothing but still publishes every writer's flag, so the
    # waits return at once instead of running into their time-out)
    fulls = [torch.full((max(T, 1), world * hl, D), float("nan"), dtype=torch.bfloat16, device="cuda")[:T]
             for _ in range(world)]
    flags = [torch.zeros(world, dtype=torch.int32, device="cuda") for _ in range(world)]
    for epoch in (1, 2):
        for r in range(world):
            cache.gather_heads_peer_store(locals_[r], T, hl, world, r,
                                          [f.data_ptr() for f in fulls],
                                          [f.data_ptr() for f in flags], epoch, wait=False)
        for r in range(world):
            cache.gather_heads_wait(flags[r], world, epoch)
        torch.cuda.synchronize()
        cache.check_errors()
        want = torch.cat(locals_, dim=1)
        for r in range(world):
            assert torch.equal(fulls[r].view(torch.int16), want.view(torch.int16)), (epoch, r)
            assert (flags[r] == epoch).all()
        locals_ = [x * 0.5 for x in locals_]   # new values for the second epoch


def test_a_missing_writer_is_reported_not_waited_for_forever(cuda_device):
    """A flag that nothing sets: the wait gives up after about a second and the time-out
    comes back through the error word; the handle stays usable."""
    cache = pa.PagedCache(BS, 8, D, 1)
    flags = torch.zeros(2, dtype=torch.int32, device="cuda")
    flags[0] = 1
    cache.gather_heads_wait(flags, 2, 1)
    torch.cuda.synchronize()
    with pytest.raises(pa.PagedAttnError) as e:
        cache.check_errors()
    assert e.value.status == 5
    flags[1] = 1
    cache.gather_heads_wait(flags, 2, 1)
    torch.cuda.synchronize()
    cache.check_errors()


def test_peer_gather_rejects_bad_arguments(cuda_device):
    cache = pa.PagedCache(BS, 8, D, 1)
    x = torch.zeros(4, 2, D, dtype=torch.bfloat16, device="cuda")
    full = torch.zeros(4, 4, D, dtype=torch.bfloat16, device="cuda")
    fl = torch.zeros(2, dtype=torch.int32, device="cuda")
    for kw in (dict(world=9, rank=0), dict(world=2, rank=2), dict(world=2, rank=-1)):
        with pytest.raises(pa.PagedAttnError):
            cache.gather_heads_peer_store(x, 4, 2, kw["world"], kw["rank"],
                                          [full.data_ptr()] * max(kw["world"], 1),
                                          [fl.data_ptr()] * max(kw["world"], 1), 1, wait=False)
