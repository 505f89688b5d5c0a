"""World-size-2 CPU test (gloo) of the KV-head sharding: each rank attends over
its own heads' pools with the shared block tables, the gathered result must equal
the unsharded oracle bit for bit.  Exercises the same shard arithmetic and gather
bench.py uses with NCCL."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from paged_attn_b200 import sharding
from pa_testlib import BS, D, Case, oracle, p


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, result_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        case = Case([70, 33, 300, 16, 5], [3, 1, 1, 16, 5], 16, 4, 64, seed=77)
        k_pool, v_pool = case.pools_after_write()
        ka, kb = sharding.kv_head_range(rank, world, case.Hkv)
        qa, qb = sharding.q_head_range(rank, world, case.Hq, case.Hkv)
        k_l = np.ascontiguousarray(k_pool[:, ka:kb])
        v_l = np.ascontiguousarray(v_pool[:, ka:kb])
        q_l = np.ascontiguousarray(case.q[:, qa:qb])
        out_l = np.zeros((case.total_q, qb - qa, D), dtype=np.float32)
        oracle().oracle_paged_attention_varlen(
            p(out_l), p(q_l), p(k_l), p(v_l), p(case.block_tables), p(case.kv_lens), p(case.cu_q),
            case.S, qb - qa, kb - ka, D, BS, case.MB, (qb - qa) * D, case.scale, 1.0)
        full = sharding.gather_heads(torch.from_numpy(out_l), world).numpy()
        if rank == 0:
            ref = np.zeros((case.total_q, case.Hq, D), dtype=np.float32)
            oracle().oracle_paged_attention_varlen(
                p(ref), p(case.q), p(k_pool), p(v_pool), p(case.block_tables), p(case.kv_lens),
                p(case.cu_q), case.S, case.Hq, case.Hkv, D, BS, case.MB, case.Hq * D, case.scale, 1.0)
            np.save(result_path, np.array([float(np.array_equal(full, ref)), float(np.abs(ref).max())]))
    finally:
        dist.destroy_process_group()


def test_kv_head_sharding_two_ranks(tmp_path):
    result = str(tmp_path / "result.npy")
    mp.spawn(_rank_main, args=(2, _free_port(), result), nprocs=2, join=True)
    equal, mag = np.load(result)
    assert equal == 1.0 and mag > 0


def test_shard_ranges():
    assert sharding.kv_head_range(3, 8, 8) == (3, 4)
    assert sharding.q_head_range(1, 2, 64, 8) == (32, 64)
    assert [sharding.kv_head_range(r, 4, 8) for r in range(4)] == [(0, 2), (2, 4), (4, 6), (6, 8)]
    with pytest.raises(ValueError):
        sharding.kv_head_range(0, 3, 8)
    with pytest.raises(ValueError):
        sharding.kv_head_range(2, 2, 8)


def test_shard_head_ranges_c_abi_matches_python():
    """The C ABI helper and the Python mirror give the same head ranges, and refuse the
    same splits."""
    import ctypes as C

    from paged_attn_b200 import PagedAttnError, sharding
    from paged_attn_b200.host import lib
    l = lib()
    for world in (1, 2, 4, 8):
        for hq, hkv in ((32, 8), (64, 8), (16, 8), (8, 8)):
            for rank in range(world):
                out = [C.c_int32() for _ in range(4)]
                rc = l.pa_shard_head_ranges(rank, world, hq, hkv, *[C.byref(o) for o in out])
                assert rc == 0
                assert (out[0].value, out[1].value) == sharding.kv_head_range(rank, world, hkv)
                assert (out[2].value, out[3].value) == sharding.q_head_range(rank, world, hq, hkv)
    out = [C.c_int32() for _ in range(4)]
    refs = [C.byref(o) for o in out]
    assert l.pa_shard_head_ranges(0, 3, 32, 8, *refs) == 1      # 8 heads do not split 3 ways
    assert l.pa_shard_head_ranges(2, 2, 32, 8, *refs) == 1      # rank out of range
    assert l.pa_shard_head_ranges(0, 2, 30, 8, *refs) == 1      # 30 is not a multiple of 8
