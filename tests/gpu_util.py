"""Device-side helpers for the GPU tests: numpy bf16 bit patterns <-> torch
tensors, and a runner that pushes a Case through the C ABI."""
import numpy as np
import torch

import paged_attn_b200 as pa
from pa_testlib import BS, CANARY, D, X, bf16_to_f32, elems_to_f32


def to_dev(bits: np.ndarray, f16: bool = False) -> torch.Tensor:
    """uint16 bit patterns -> bf16 (or f16) tensor on the device."""
    return torch.from_numpy(bits.view(np.int16)).cuda().view(torch.float16 if f16 else torch.bfloat16)


def to_bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


class _Raw:
    def __init__(self, ptr, shape):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": "<i2",
                                         "data": (int(ptr), False), "version": 2}


def device_view(ptr: int, shape) -> torch.Tensor:
    """bf16 tensor over device memory the library owns (no copy)."""
    return torch.as_tensor(_Raw(ptr, shape), device="cuda").view(torch.bfloat16)


class DeviceCase:
    """Uploads a Case and owns the pool tensors the cache handle wraps."""

    def __init__(self, case, k_pool=None, v_pool=None):
        self.case = case
        f16 = getattr(case, "f16", False)
        self.k_pool = to_dev(case.k_pool if k_pool is None else k_pool, f16)
        self.v_pool = to_dev(case.v_pool if v_pool is None else v_pool, f16)
        self.D = getattr(case, "D", D)
        self.cache = pa.PagedCache(getattr(case, "bs", BS), case.NB, self.D, case.Hkv, dtype=0 if f16 else 1,
                                   key_pools=[self.k_pool], value_pools=[self.v_pool])
        self.q = to_dev(case.q, f16)
        self.k_new = to_dev(case.k_new, f16)
        self.v_new = to_dev(case.v_new, f16)
        self.slots = torch.from_numpy(case.slot_mapping).cuda()
        self.tables = torch.from_numpy(case.block_tables).cuda()
        self.lens = torch.from_numpy(case.kv_lens).cuda()
        self.ws_bytes = self.cache.workspace_bytes()
        self.ws = torch.empty(self.ws_bytes, dtype=torch.uint8, device="cuda")
        # fill the scratch with NaN patterns so stale partials cannot pass for results
        self.ws.view(torch.int16).fill_(0x7FFF)

    def write(self):
        c = self.case
        self.cache.reshape_and_cache(self.k_new, self.v_new, self.slots, len(c.slot_mapping),
                                     c.Hkv * self.D, c.Hkv * self.D)

    def attend(self, varlen=True, softcap=1.0, host_lens=True):
        c = self.case
        f16 = getattr(c, "f16", False)
        out = torch.full((max(c.total_q, 1), c.Hq, self.D), float("nan"),
                         dtype=torch.float16 if f16 else torch.bfloat16, device="cuda")
        if varlen:
            self.cache.varlen(out, self.q, self.tables, self.lens, c.cu_q, c.S, c.Hq, c.MB,
                              c.scale, self.ws, self.ws_bytes, softcap=softcap,
                              context_lens_host=c.kv_lens if host_lens else None)
        else:
            self.cache.decode(out, self.q, self.tables, self.lens, c.S, c.Hq, c.MB, c.scale,
                              self.ws, self.ws_bytes, softcap=softcap)
        torch.cuda.synchronize()
        self.cache.check_errors()
        return elems_to_f32(to_bits(out), f16)[:c.total_q]
