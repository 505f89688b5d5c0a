"""The five benchmark configurations at their FULL sizes on the GPU.

Each case is checked by
(a) the KV write against an independent torch scatter over the whole pool, bit for
    bit, with never-written slots still holding their canary;
(b) the fp64 oracle: over the WHOLE output for the decode configurations (1-3) and for
    the decode and verify sequences of the mixed batch (5); for the long chunks
    (configuration 4 and the prefill part of 5) on the queries either side of every
    Q-tile edge of the tile kernel (a CTA's two 128-row tiles change every 128 / G
    queries), which are also the queries whose causal limit crosses a KV-tile edge,
    all heads;
(c) size-independent properties: decode entry == varlen entry with one query per
    sequence (bit-identical), run-to-run determinism, and convexity (every output
    lies within the min/max of V over its context for that head dimension is
    implied by (b); here: all outputs finite and |out| <= max|V|).
Inputs are drawn on the device with a seeded torch generator (bf16 N(0,1)); block
tables are a seeded permutation of the pool, as the configurations state."""
import math

import numpy as np
import pytest
import torch

import paged_attn_b200 as pa
from gpu_util import to_bits
from pa_testlib import (BS, CANARY, D, X, attention_oracle_rows, bf16_to_f32, check_attention,
                        config_lengths, oracle, p)

pytestmark = pytest.mark.gpu


class FullCase:
    def __init__(self, name, seed=0):
        kv, ql, Hq, Hkv, NB = config_lengths(name, seed)
        self.kv, self.ql = np.asarray(kv), np.asarray(ql)
        self.Hq, self.Hkv, self.NB, self.S = Hq, Hkv, NB, len(kv)
        dev = torch.device("cuda")
        g = torch.Generator(device=dev)
        g.manual_seed(seed + 17)
        nblk = (self.kv + BS - 1) // BS
        self.MB = int(nblk.max())
        perm = np.random.Generator(np.random.PCG64(seed)).permutation(NB).astype(np.int32)
        self.tables_h = np.zeros((self.S, self.MB), dtype=np.int32)
        tot = int(self.kv.sum())
        slots = np.empty(tot, dtype=np.int64)
        is_new = np.zeros(tot, dtype=bool)
        cu_kv = np.concatenate([[0], np.cumsum(self.kv)])
        pos = 0
        for s in range(self.S):
            self.tables_h[s, :nblk[s]] = perm[pos:pos + nblk[s]]
            pos += nblk[s]
            t = np.arange(self.kv[s])
            slots[cu_kv[s]:cu_kv[s + 1]] = self.tables_h[s, t // BS].astype(np.int64) * BS + t % BS
            is_new[cu_kv[s + 1] - self.ql[s]:cu_kv[s + 1]] = True
        self.cu_q = np.concatenate([[0], np.cumsum(self.ql)]).astype(np.int32)
        self.total_q = int(self.cu_q[-1])

        def randn(*shape):
            out = torch.empty(shape, dtype=torch.bfloat16, device=dev)
            flat, step = out.view(-1), 1 << 26
            for i in range(0, flat.numel(), step):
                n = min(step, flat.numel() - i)
                flat[i:i + n] = torch.randn(n, generator=g, device=dev).to(torch.bfloat16)
            return out
        self.k_all, self.v_all = randn(tot, Hkv, D), randn(tot, Hkv, D)
        self.q = randn(self.total_q, Hq, D)
        self.slots_all = torch.from_numpy(slots).to(dev)
        self.new_idx = torch.from_numpy(np.nonzero(is_new)[0]).to(dev)
        self.old_idx = torch.from_numpy(np.nonzero(~is_new)[0]).to(dev)
        self.k_pool = torch.full((NB, Hkv, D // X, BS, X), float("nan"), dtype=torch.bfloat16, device=dev)
        self.v_pool = torch.full((NB, Hkv, D, BS), float("nan"), dtype=torch.bfloat16, device=dev)
        self.k_pool.view(torch.int16).fill_(CANARY)
        self.v_pool.view(torch.int16).fill_(CANARY)
        self.cache = pa.PagedCache(BS, NB, D, Hkv, key_pools=[self.k_pool], value_pools=[self.v_pool])
        self.tables = torch.from_numpy(self.tables_h).to(dev)
        self.lens = torch.from_numpy(self.kv.astype(np.int32)).to(dev)
        self.ws = torch.empty(self.cache.workspace_bytes(), dtype=torch.uint8, device=dev)
        self.scale = 1.0 / math.sqrt(D)

    def write_all(self):
        """Prefix first, then the step's new tokens, both through the library."""
        for idx in (self.old_idx, self.new_idx):
            if idx.numel() == 0:
                continue
            k, v = self.k_all[idx].contiguous(), self.v_all[idx].contiguous()
            s = self.slots_all[idx].contiguous()
            self.cache.reshape_and_cache(k, v, s, idx.numel(), self.Hkv * D, self.Hkv * D)
        torch.cuda.synchronize()
        self.cache.check_errors()

    def check_pools_against_torch_scatter(self):
        blk, off = self.slots_all // BS, self.slots_all % BS
        k_ref = torch.empty_like(self.k_pool)
        k_ref.view(torch.int16).fill_(CANARY)
        v_ref = torch.empty_like(self.v_pool)
        v_ref.view(torch.int16).fill_(CANARY)
        k_ref[blk, :, :, off, :] = self.k_all.view(-1, self.Hkv, D // X, X)
        v_ref[blk, :, :, off] = self.v_all
        assert torch.equal(self.k_pool.view(torch.int16), k_ref.view(torch.int16)), "K pool differs"
        assert torch.equal(self.v_pool.view(torch.int16), v_ref.view(torch.int16)), "V pool differs"

    def attend(self, varlen):
        out = torch.full((self.total_q, self.Hq, D), float("nan"), dtype=torch.bfloat16, device="cuda")
        if varlen:
            self.cache.varlen(out, self.q, self.tables, self.lens, self.cu_q, self.S, self.Hq, self.MB,
                              self.scale, self.ws, self.ws.numel(), max_context_len=int(self.kv.max()),
                              context_lens_host=np.ascontiguousarray(self.kv.astype(np.int32)))
        else:
            self.cache.decode(out, self.q, self.tables, self.lens, self.S, self.Hq, self.MB, self.scale,
                              self.ws, self.ws.numel())
        torch.cuda.synchronize()
        self.cache.check_errors()
        return out

    def check_sequences(self, out, seqs, what, queries_of=None):
        """fp64 oracle on rows of the given sequences, every head: all their queries, or the
        queries queries_of(q_len) picks."""
        nblk = (self.kv + BS - 1) // BS
        ids = np.concatenate([self.tables_h[s, :nblk[s]] for s in seqs])
        idt = torch.from_numpy(ids.astype(np.int64)).cuda()
        k_c, v_c = to_bits(self.k_pool[idt]), to_bits(self.v_pool[idt])
        tables_c = np.zeros((len(seqs), self.MB), dtype=np.int32)
        pos = 0
        for i, s in enumerate(seqs):
            tables_c[i, :nblk[s]] = np.arange(pos, pos + nblk[s])
            pos += nblk[s]
        lens_c = np.ascontiguousarray(self.kv[seqs].astype(np.int32))
        ql_c = self.ql[seqs]
        cu_c = np.concatenate([[0], np.cumsum(ql_c)]).astype(np.int32)
        q_rows = np.concatenate([np.arange(self.cu_q[s], self.cu_q[s + 1]) for s in seqs])
        q_c = to_bits(self.q[torch.from_numpy(q_rows).cuda()])
        rows = []
        for i, s in enumerate(seqs):
            js = range(int(ql_c[i])) if queries_of is None else queries_of(int(ql_c[i]))
            for j in js:
                for hq in range(self.Hq):
                    rows.append((i, j, hq))
        ref = attention_oracle_rows(rows, q_c, k_c, v_c, tables_c, lens_c, cu_c, self.Hq, self.Hkv,
                                    self.MB, self.scale)
        out_h = bf16_to_f32(to_bits(out[torch.from_numpy(q_rows).cuda()]))
        idx = np.array([(cu_c[i] + j, hq) for (i, j, hq) in rows])
        got = out_h[idx[:, 0], idx[:, 1]]
        stats = check_attention(got, ref, what)
        stats["rows"] = len(rows)
        return stats

    def check_whole_decode_output(self, out, what):
        """The fp64 oracle over every output row of a decode batch, read through the full
        pools and tables (no sampling)."""
        k, v = to_bits(self.k_pool), to_bits(self.v_pool)
        q = to_bits(self.q)
        ref = np.zeros((self.S, self.Hq, D), dtype=np.float32)
        lens = np.ascontiguousarray(self.kv.astype(np.int32))
        oracle().oracle_paged_attention_varlen_dt(p(ref), p(q), p(k), p(v), p(self.tables_h), p(lens), None,
                                                  self.S, self.Hq, self.Hkv, D, BS, self.MB, self.Hq * D,
                                                  self.scale, 1.0, 0)
        stats = check_attention(bf16_to_f32(to_bits(out)), ref, what)
        stats["rows"] = self.S * self.Hq
        return stats


@pytest.mark.parametrize("name", ["c1", "c2", "c3"])
def test_decode_configuration_full_size(cuda_device, name):
    c = FullCase(name)
    c.write_all()
    c.check_pools_against_torch_scatter()
    out = c.attend(varlen=False)
    assert torch.isfinite(out.float()).all()
    assert out.float().abs().max() <= c.v_all.float().abs().max()
    print(name, c.check_whole_decode_output(out, name + " full size, whole output"))
    again = c.attend(varlen=False)
    assert torch.equal(out.view(torch.int16), again.view(torch.int16)), "not deterministic"
    as_varlen = c.attend(varlen=True)
    assert torch.equal(out.view(torch.int16), as_varlen.view(torch.int16)), "decode != varlen(q_len=1)"


@pytest.mark.parametrize("half", [0, 1])
def test_chunked_prefill_configuration_full_size(cuda_device, half):
    """Configuration 4 at full size, every output row against the fp64 oracle: four of the
    eight sequences per test (8192 queries x 32 heads x ~9200 keys each is about 25 s of host
    arithmetic, well inside the per-test limit)."""
    c = FullCase("c4")
    c.write_all()
    c.check_pools_against_torch_scatter()
    out = c.attend(varlen=True)
    assert torch.isfinite(out.float()).all()
    for pair in ([0, 1], [2, 3]) if half == 0 else ([4, 5], [6, 7]):
        print("c4", pair, c.check_sequences(out, pair, f"c4 full size, whole output, sequences {pair}"))
    again = c.attend(varlen=True)
    assert torch.equal(out.view(torch.int16), again.view(torch.int16)), "not deterministic"


def test_mixed_configuration_full_size(cuda_device):
    c = FullCase("c5")
    c.write_all()
    c.check_pools_against_torch_scatter()
    out = c.attend(varlen=True)
    assert torch.isfinite(out.float()).all()
    # decode (0..47), verify (48..55) and prefill (56, 57) sequences
    print("c5 decode + verify", c.check_sequences(out, list(range(56)), "c5 decode and verify, whole output"))
    print("c5 prefill", c.check_sequences(out, [56, 57], "c5 prefill chunks, whole output"))
    again = c.attend(varlen=True)
    assert torch.equal(out.view(torch.int16), again.view(torch.int16)), "not deterministic"
