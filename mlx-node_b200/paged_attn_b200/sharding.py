"""KV-head sharding of the paged-attention path across the GPUs of one box.

A (sequence, kv head) pair touches only that head's K and V chunks and that
head's query heads (kv_head = q_head // G,
crates/mlx-paged-attn/metal/attention/paged_attention.metal:837-840; the pools
are [num_blocks, num_kv_heads, ...]), so rank r owns kv heads
[r*Hkv/world, (r+1)*Hkv/world) with pools [num_blocks, Hkv/world, ...] and the
SAME block ids, block tables, context lengths and slot mapping as every other
rank (one host allocator).  No collective sits on the data path; the optional
all-gather below rebuilds [tokens, Hq, D] for a consumer that needs every head.
"""
from __future__ import annotations


def kv_head_range(rank: int, world: int, num_kv_heads: int) -> tuple[int, int]:
    if world < 1 or not 0 <= rank < world:
        raise ValueError("bad rank/world")
    if num_kv_heads % world:
        raise ValueError(f"{num_kv_heads} kv heads do not split {world} ways")
    n = num_kv_heads // world
    return rank * n, (rank + 1) * n


def q_head_range(rank: int, world: int, num_q_heads: int, num_kv_heads: int) -> tuple[int, int]:
    if num_q_heads % num_kv_heads:
        raise ValueError("query heads must be a multiple of kv heads")
    g = num_q_heads // num_kv_heads
    a, b = kv_head_range(rank, world, num_kv_heads)
    return a * g, b * g


def gather_heads(out_local, world: int, group=None):
    """[T, Hq/world, D] on every rank -> [T, Hq, D] on every rank (NCCL or gloo)."""
    import torch
    import torch.distributed as dist
    if world == 1:
        return out_local
    t, hl, d = out_local.shape
    parts = torch.empty((world * t, hl, d), dtype=out_local.dtype, device=out_local.device)
    dist.all_gather_into_tensor(parts, out_local.contiguous(), group=group)
    return parts.view(world, t, hl, d).permute(1, 0, 2, 3).reshape(t, world * hl, d)
