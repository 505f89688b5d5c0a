"""The five benchmark configurations of the paged-attention path, as lengths only
(seeded); tensors are drawn by whoever runs them.  Shared by bench.py and the tests.

Context lengths stand in for a serving trace: uniform or lognormal draws with the
ranges each configuration names.  Configuration 3's lognormal uses sigma = 1.0 (only
the median is given) and a 65536-block pool."""
from __future__ import annotations

import math

import numpy as np

DESCRIPTIONS = {
    "c1": "Qwen3-0.6B-shaped decode",
    "c2": "Qwen3-8B-shaped decode",
    "c3": "Qwen3-32B-shaped decode, lognormal contexts (median 4096, sigma 1, clipped to [256, 32768])",
    "c4": "chunked prefill: 8192 cached + 2048 new tokens per sequence, causal",
    "c5": "mixed batch: 48 decode + 8 verify (5 queries) + 2 prefill chunks of 1024 over 4096",
}


def config_lengths(name: str, seed: int = 0):
    """(kv_lens, q_lens, Hq, Hkv, NB) of the named configuration.  kv_lens count the
    tokens written this step."""
    rng = np.random.Generator(np.random.PCG64(seed + 1000))
    if name == "c1":
        return rng.integers(512, 2049, 8), np.ones(8, int), 16, 8, 1024
    if name == "c2":
        return rng.integers(1024, 8193, 64), np.ones(64, int), 32, 8, 40000
    if name == "c3":
        z = rng.standard_normal(128)
        kv = np.clip(np.rint(np.exp(math.log(4096.0) + z)), 256, 32768).astype(int)
        return kv, np.ones(128, int), 64, 8, 65536
    if name == "c4":
        return np.full(8, 8192 + 2048), np.full(8, 2048), 32, 8, 8192
    if name == "c5":
        dec = rng.integers(1024, 16385, 48)
        ver = rng.integers(2048, 8193, 8) + 5
        pre = np.full(2, 4096 + 1024)
        kv = np.concatenate([dec, ver, pre])
        ql = np.concatenate([np.ones(48, int), np.full(8, 5), np.full(2, 1024)])
        return kv, ql, 32, 8, 60000
    raise KeyError(name)
