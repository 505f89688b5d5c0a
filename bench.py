#!/usr/bin/env python
"""Benchmark of the paged-attention hot path on B200.

A step is one pass of the path over one synthetic batch: the KV block write of
the step's new tokens (reshape_and_cache) followed by paged attention over the
block-table cache, the order one transformer layer runs them.  Decode batches
go through one call (pa_decode_step): one launch while a rank holds at most
2 x SMs (sequence, kv head) pairs - the attention kernel writes the tokens
itself - and the write kernel chained to the attention kernel otherwise.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c3]
  python bench.py --impl reference ...      # the CPU path, timed on the host cores

Headline workload ("c3", for every N): Qwen3-32B-shaped decode, 64 query / 8 KV
heads, head 128, block 16, one batch of 128 sequences with lognormal contexts
(median 4096, clipped to [256, 32768]), bf16 N(0,1), block tables a random
permutation of a 65536-block pool.  With N GPUs the KV heads (and their query
heads and pools) are split N ways: every rank runs the same 128 sequences on
8/N KV heads, no data-path collective, total work fixed (strong scaling).

On one GPU the line also carries `also`: configuration 2 (decode), 4 (chunked
prefill, tensor bound) and 5 (mixed batch) timed the same way in the same process.

Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, "mlx-node_b200")
if PKG not in sys.path:
    sys.path.insert(0, PKG)

D = 128
L2_BYTES = 126 << 20


def _oracle_tools():
    """The CPU oracle (checker and CPU baseline only; never on the timed GPU path)."""
    tests = os.path.join(ROOT, "tests")
    if tests not in sys.path:
        sys.path.insert(0, tests)
    import pa_testlib
    return pa_testlib


# ---------------------------------------------------------------------------------------
def algorithmic_bytes(kv_lens, q_lens, Hq, Hkv, bs, kv_elem_bytes=2) -> int:
    """One pass over the live KV bytes (once per KV head, whatever the group size or the
    number of splits), the block-table entries and lengths, Q read and O written."""
    kv = int(np.sum(kv_lens))
    blocks = int(np.sum((np.asarray(kv_lens) + bs - 1) // bs))
    tq = int(np.sum(q_lens))
    return kv * 2 * Hkv * D * kv_elem_bytes + blocks * 4 + len(kv_lens) * 4 + 2 * tq * Hq * D * 2


def write_bytes(q_lens, Hkv, kv_elem_bytes=2) -> int:
    t = int(np.sum(q_lens))
    return t * (2 * Hkv * D) * (2 + kv_elem_bytes) + t * 8


def attention_flops(kv_lens, q_lens, Hq) -> int:
    f = 0
    for kv, ql in zip(kv_lens, q_lens):
        f += int(ql) * int(kv - ql) + int(ql) * (int(ql) + 1) // 2
    return 4 * D * Hq * f


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            m = json.load(f)
        return {"hbm": float(m["hbm_gbs"]), "tf": float(m["bf16_tflops"]),
                "tf_sustained": float(m.get("bf16_tflops_sustained", 0.0)) or None,
                "kind": "measured (MEASURED_PEAKS.json)"}
    return {"hbm": 6650.0, "tf": 1590.0, "tf_sustained": 1400.0, "kind": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while a leg runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def stop(self, t_load0=None, t_load1=None) -> dict:
        """Summary of the samples taken between the two host times (all, if none given)."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.08)
        self.proc.terminate()
        sm, mx, power, reasons = [], None, [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for t, line in self.lines:
            if t_load0 is not None and not (t_load0 <= t <= t_load1):
                continue
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx = float(parts[1])
                power.append(float(parts[2]))
            except ValueError:
                continue
            for n, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx,
                "reasons": sorted(reasons), "samples": len(sm),
                "power_w": statistics.median(power) if power else None,
                "covers": "soak of the same step (>= 0.6 s), the timed steps and the kernel-only loop"}


def l2_statement(kv, hkv_local, kv_elem_bytes=2):
    """Whether one step's KV bytes per GPU exceed the L2 (no flush is done between steps)."""
    step = int(np.sum(kv)) * 2 * hkv_local * D * kv_elem_bytes
    if step > L2_BYTES:
        return f"inputs larger than L2 ({step / 1e6:.0f} MB of KV per step and GPU, L2 126 MB)"
    return (f"working set {step / 1e6:.0f} MB fits in the 126 MB L2 and nothing flushes it: "
            "L2-resident timing, reported for latency only")


def workload_config(name, world, kv, ql, Hq, Hkv, bs):
    from paged_attn_b200.workloads import DESCRIPTIONS
    return {"workload": f"{name}: {DESCRIPTIONS[name]}; {len(kv)} sequences, {Hq} query / {Hkv} kv "
                        f"heads, head {D}, block {bs}, {int(np.sum(ql))} query tokens over "
                        f"{int(np.sum(kv))} cached tokens; step = KV write + paged attention",
            "sharding": (f"kv heads split {world} ways: every rank runs all {len(kv)} sequences on "
                         f"{Hkv // world} kv / {Hq // world} query heads, own pool, no collective")
            if world > 1 else "single GPU",
            "l2": l2_statement(kv, Hkv // max(world, 1))}


# ---------------------------------------------------------------------------------------
class CpuSample:
    """A bounded sample of a decode workload for the CPU path: the first n sequences, their
    blocks compacted into a small pool.  A step = scatter write of the n new tokens + the
    reference's software attention (crates/mlx-sys/src/mlx.cpp:4080-4159, restated in
    oracle/paged_oracle.c), on every host core."""

    def __init__(self, name, kv, ql, Hq, Hkv, bs, n_s):
        T = _oracle_tools()
        self.T, self.n_s, self.Hq, self.Hkv, self.bs, self.name, self.total = T, n_s, Hq, Hkv, bs, name, len(kv)
        self.lib = T.oracle()
        self.lib.oracle_set_num_threads(len(os.sched_getaffinity(0)))
        self.cores = int(self.lib.oracle_num_threads())
        kv_s, ql_s = kv[:n_s], ql[:n_s]
        nb = int(((kv_s + bs - 1) // bs).sum())
        self.case = T.Case(kv_s, ql_s, Hq, Hkv, nb + 8, seed=0, bs=bs)
        c = self.case
        c.k_pool[c.k_pool == T.CANARY] = 0
        c.v_pool[c.v_pool == T.CANARY] = 0
        self.out = np.zeros((c.S, Hq, D), dtype=np.uint16)

    def step(self):
        T, c = self.T, self.case
        T.write_oracle(c.k_pool, c.v_pool, c.k_new, c.v_new, c.slot_mapping, self.Hkv)
        rc = self.lib.baseline_mlx_paged_forward(T.p(self.out), T.p(c.q), T.p(c.k_pool), T.p(c.v_pool),
                                                 T.p(c.block_tables), T.p(c.kv_lens), c.S, self.Hq,
                                                 self.Hkv, D, self.bs, c.MB, c.scale)
        assert rc == 0

    def describe(self, steps):
        return (f"first {self.n_s} of {self.total} sequences of workload {self.name} "
                f"({int(self.case.kv_lens.sum())} cached tokens), KV write + attention, {steps} step(s)")


def cpu_sample_size(kv):
    return min(len(kv), max(len(os.sched_getaffinity(0)), 8))


def run_reference(args, rank: int, world: int) -> None:
    """The reference's CPU implementation of the path on the host cores.  The reference
    itself cannot be built here (Metal kernels; MLX sources absent; no Rust toolchain), so
    this times the oracle port of its software path plus the scatter form of its block
    write, with every host thread, on a bounded sample of the same workload; rank 0 only."""
    if rank != 0:
        return
    from paged_attn_b200.workloads import config_lengths
    kv, ql, Hq, Hkv, _ = config_lengths(args.workload)
    if args.workload in ("c4", "c5"):
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference has no paged multi-token attention "
                          "(crates/mlx-paged-attn/src/scheduler.rs:237-242); only decode workloads "
                          "have a CPU path"}))
        return
    n_s = cpu_sample_size(kv)
    sample = CpuSample(args.workload, kv, ql, Hq, Hkv, args.block_size, n_s)
    t0 = time.perf_counter()
    sample.step()  # first warm-up step, also the estimate that bounds the run
    t_one = time.perf_counter() - t0
    budget = 150.0
    if (args.steps + args.warmup) * t_one > budget and n_s > 2:
        n_s = max(2, int(n_s * budget / ((args.steps + args.warmup) * t_one)))
        sample = CpuSample(args.workload, kv, ql, Hq, Hkv, args.block_size, n_s)
        sample.step()
    for _ in range(max(args.warmup - 1, 0)):
        sample.step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        sample.step()
    dt = (time.perf_counter() - t0) / args.steps
    value = n_s / dt
    line = {
        "impl": "reference", "metric": "paged_decode_attn_tokens_per_s", "value": value,
        "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args.workload, max(world, 1), kv, ql, Hq, Hkv, args.block_size),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": sample.cores, "kind": "port",
                         "sample": sample.describe(args.steps)},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------
class Workload:
    """One configuration resident on this rank's GPU: pools pre-filled through the
    library's own write, the step's new tokens, queries, tables, lengths, workspace."""

    def __init__(self, name, rank, world, local_rank, args, seqs=0):
        import torch
        import paged_attn_b200 as pa
        from paged_attn_b200 import sharding
        from paged_attn_b200.workloads import config_lengths
        self.torch, self.pa, self.name, self.args = torch, pa, name, args
        self.rank, self.world = rank, world
        bs = self.bs = args.block_size
        kv, ql, Hq, Hkv, NB = config_lengths(name)
        if seqs:
            kv, ql = kv[:seqs], ql[:seqs]
        if bs != 16:  # the same pool bytes in other block sizes
            NB = max(NB * 16 // bs, int(((kv + bs - 1) // bs).sum()))
        if args.pool_blocks:
            NB = args.pool_blocks
        assert int(((kv + bs - 1) // bs).sum()) <= NB
        self.kv, self.ql, self.Hq, self.Hkv, self.NB = kv, ql, Hq, Hkv, NB
        ka, kb = sharding.kv_head_range(rank, world, Hkv)
        qa, qb = sharding.q_head_range(rank, world, Hq, Hkv)
        hkv_l, hq_l = self.hkv_l, self.hq_l = kb - ka, qb - qa
        S, total_q = self.S, self.total_q = len(kv), int(np.sum(ql))
        nblk = (kv + bs - 1) // bs
        MB = self.MB = int(nblk.max())
        rng = np.random.Generator(np.random.PCG64(0))  # same tables on every rank (one host allocator)
        perm = rng.permutation(NB).astype(np.int32)
        tables_h = self.tables_h = np.zeros((S, MB), dtype=np.int32)
        slots_all = np.empty(int(kv.sum()), dtype=np.int64)
        is_new = np.zeros(int(kv.sum()), dtype=bool)
        cu_kv = np.concatenate([[0], np.cumsum(kv)])
        self.cu_q = np.concatenate([[0], np.cumsum(ql)]).astype(np.int32)
        pos = 0
        for s in range(S):
            tables_h[s, :nblk[s]] = perm[pos:pos + nblk[s]]
            pos += nblk[s]
            t = np.arange(kv[s])
            slots_all[cu_kv[s]:cu_kv[s + 1]] = tables_h[s, t // bs].astype(np.int64) * bs + t % bs
            is_new[cu_kv[s + 1] - ql[s]:cu_kv[s + 1]] = True
        dev = self.dev = torch.device("cuda", local_rank)
        gen = torch.Generator(device=dev)
        gen.manual_seed(1234 + rank)

        def randn_bf16(*shape):
            out = torch.empty(shape, dtype=torch.bfloat16, device=dev)
            flat = out.view(-1)
            step = 1 << 26
            for i in range(0, flat.numel(), step):
                n = min(step, flat.numel() - i)
                flat[i:i + n] = torch.randn(n, generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
            return out

        if args.fp8:
            self.k_pool = torch.zeros(NB, hkv_l, D // 16, bs, 16, dtype=torch.uint8, device=dev)
            self.v_pool = torch.zeros(NB, hkv_l, D, bs, dtype=torch.uint8, device=dev)
        else:
            self.k_pool = torch.zeros(NB, hkv_l, D // 8, bs, 8, dtype=torch.bfloat16, device=dev)
            self.v_pool = torch.zeros(NB, hkv_l, D, bs, dtype=torch.bfloat16, device=dev)
        cache = self.cache = pa.PagedCache(bs, NB, D, hkv_l, device=local_rank, key_pools=[self.k_pool],
                                           value_pools=[self.v_pool], fp8=args.fp8)
        if args.fp8:
            cache.set_kv_scales(1.0 / 32, 1.0 / 32)  # N(0,1) values sit well inside +-240 * scale
            # the wrapped pools were zero-filled above; the library's own writes switch the
            # kernels back to exact decoding should a value ever overflow
            cache.fp8_set_exact_decode(False)
        k_all = randn_bf16(int(kv.sum()), hkv_l, D)
        v_all = randn_bf16(int(kv.sum()), hkv_l, D)
        slots_all_d = torch.from_numpy(slots_all).to(dev)
        new_idx = torch.from_numpy(np.nonzero(is_new)[0]).to(dev)
        # prefix through the library's own write (its bit-exactness is what the tests pin)
        old_slots = slots_all_d.clone()
        old_slots[new_idx] = -1
        cache.reshape_and_cache(k_all, v_all, old_slots, int(kv.sum()), hkv_l * D, hkv_l * D)
        self.k_new, self.v_new = k_all[new_idx].contiguous(), v_all[new_idx].contiguous()
        self.slots = slots_all_d[new_idx].contiguous()
        del k_all, v_all, old_slots
        self.q = randn_bf16(total_q, hq_l, D)
        self.out = torch.zeros(total_q, hq_l, D, dtype=torch.bfloat16, device=dev)
        self.tables = torch.from_numpy(tables_h).to(dev)
        self.lens = torch.from_numpy(kv.astype(np.int32)).to(dev)
        self.ws_bytes = cache.workspace_bytes()
        self.ws = torch.empty(self.ws_bytes, dtype=torch.uint8, device=dev)
        self.scale = 1.0 / math.sqrt(D)
        self.decode_only = bool((ql == 1).all())
        self.kv_i32 = np.ascontiguousarray(kv.astype(np.int32))
        self.stream = torch.cuda.current_stream().cuda_stream
        self.eb = 1 if args.fp8 else 2
        if args.producer:
            # projections in, rotated queries out (separate buffer so every step does the same work)
            self.q_raw = self.q
            self.q = torch.empty_like(self.q_raw)
            self.norm_w = torch.ones(D, dtype=torch.bfloat16, device=dev)
            pos_h = np.concatenate([kv[s] - ql[s] + np.arange(ql[s]) for s in range(S)]).astype(np.int32)
            self.positions = torch.from_numpy(pos_h).to(dev)
        torch.cuda.synchronize()
        cache.check_errors(self.stream)

    # -- device-resident legs ------------------------------------------------------------
    def attn_only(self):
        c = self.cache
        if self.decode_only:
            c.decode(self.out, self.q, self.tables, self.lens, self.S, self.hq_l, self.MB, self.scale,
                     self.ws, self.ws_bytes, stream=self.stream)
        else:
            c.varlen(self.out, self.q, self.tables, self.lens, self.cu_q, self.S, self.hq_l, self.MB,
                     self.scale, self.ws, self.ws_bytes, max_context_len=int(self.kv.max()),
                     stream=self.stream, context_lens_host=self.kv_i32)

    def step(self):
        c, a = self.cache, self.args
        if a.producer:
            c.qk_norm_rope_and_cache(self.q, self.q_raw, self.k_new, self.v_new, self.norm_w, self.norm_w,
                                     1e-6, self.positions, 1.0e6, D, self.slots, self.total_q, self.hq_l,
                                     self.hq_l * D, self.hq_l * D, self.hkv_l * D, self.hkv_l * D,
                                     stream=self.stream)
            self.attn_only()
        elif self.decode_only and not a.two_launches:
            c.decode_step(self.out, self.q, self.k_new, self.v_new, self.slots, self.tables, self.lens,
                          self.S, self.hq_l, self.MB, self.scale, self.ws, self.ws_bytes, stream=self.stream)
        else:
            c.reshape_and_cache(self.k_new, self.v_new, self.slots, self.total_q, self.hkv_l * D,
                                self.hkv_l * D, stream=self.stream)
            self.attn_only()

    # -- host-buffer leg -----------------------------------------------------------------
    def host_step_fn(self):
        """(callable, h2d-bytes function, d2h bytes): one step from pinned HOST buffers; the
        call brings the inputs in, runs the kernels, copies the result out, synchronises.

        Decode workloads run a real decode loop through the bound host cache
        (pa_kv_extend_sequences + pa_kv_decode_step_host): every step the sequences grow by
        one token, the host cache hands out the slot (and now and then a new block), the
        block tables stay resident on the device and only new entries travel.  Mixed
        workloads go through pa_varlen_step_host with the step's tables sent whole."""
        torch = self.torch
        pin = lambda t: t.cpu().pin_memory()
        q_h, k_h, v_h = pin(self.q), pin(self.k_new), pin(self.v_new)
        out_h = torch.empty_like(self.q, device="cpu").pin_memory()
        d2h = int(out_h.numel() * 2)
        c = self.cache
        self._keep_host = [q_h, k_h, v_h, out_h]
        bound = self._bound_decode_cache() if self.decode_only else None
        if bound is not None:
            host, b, ids = bound
            sent0 = [b.stats()["table_entries_sent"], 0]

            def fn():
                host.extend_sequences(ids, 1)
                b.decode_step_host(out_h, q_h, k_h, v_h, ids, self.hq_l, self.scale)
                sent0[1] += 1

            def h2d():
                per_step = (b.stats()["table_entries_sent"] - sent0[0]) / max(sent0[1], 1)
                return int(q_h.numel() * 2 + k_h.numel() * 2 + v_h.numel() * 2 + 256 + 16 * self.S + 12 * per_step)
            return fn, h2d, d2h, ("pa_kv_extend_sequences + pa_kv_decode_step_host: decode loop through the "
                                  "bound host cache, block tables resident on the device")
        slots_h, tables_p, lens_h = pin(self.slots), pin(self.tables), pin(self.lens)
        self._keep_host += [slots_h, tables_p, lens_h]
        n_h2d = sum(t.numel() * t.element_size() for t in (q_h, k_h, v_h, slots_h, tables_p, lens_h))
        if self.decode_only:
            def fn():
                c.decode_step_host(out_h, q_h, k_h, v_h, slots_h, tables_p, lens_h, self.S, self.hq_l,
                                   self.MB, self.scale)
            return fn, (lambda: int(n_h2d)), d2h, "pa_decode_step_host"
        n_h2d += self.cu_q.nbytes

        def fn():
            c.varlen_step_host(out_h, q_h, k_h, v_h, slots_h, tables_p, lens_h, self.cu_q, self.S,
                               self.hq_l, self.MB, self.scale)
        return fn, (lambda: int(n_h2d)), d2h, "pa_varlen_step_host"

    def _bound_decode_cache(self):
        """Host cache over this rank's pool with every sequence one token short of the
        workload's context, the pool refilled at the host allocator's slots."""
        torch = self.torch
        from paged_attn_b200.host import BoundCache, PagedKVCacheHost, host_config, seq_id_array
        block_bytes = 2 * self.hkv_l * D * self.bs * self.eb
        mb = (self.NB * block_bytes) >> 20
        if mb < 256:
            return None  # PagedAttentionConfig::validate wants at least 256 MB
        max_seq = ((int(self.kv.max()) + 1024 + self.bs - 1) // self.bs) * self.bs
        cfg = host_config(block_size=self.bs, gpu_memory_mb=mb, head_size=D, num_kv_heads=self.hkv_l,
                          num_layers=1, use_fp8_cache=int(self.args.fp8), max_seq_len=max_seq)
        host = PagedKVCacheHost(cfg)
        assert host.total_blocks() <= self.NB
        ids = [host.add_sequence(int(n) - 1) for n in self.kv]
        slots = np.concatenate([np.asarray(host.get_slot_mapping(sid, 0, int(n) - 1), dtype=np.int64)
                                for sid, n in zip(ids, self.kv)])
        slots_d = torch.from_numpy(slots).to(self.dev)
        gen = torch.Generator(device=self.dev)
        gen.manual_seed(99 + self.rank)
        step = 1 << 17
        for i in range(0, len(slots), step):  # refill in pieces to bound the temporaries
            n = min(step, len(slots) - i)
            k = torch.randn(n, self.hkv_l, D, generator=gen, device=self.dev).to(torch.bfloat16)
            v = torch.randn(n, self.hkv_l, D, generator=gen, device=self.dev).to(torch.bfloat16)
            self.cache.reshape_and_cache(k, v, slots_d[i:i + n], n, self.hkv_l * D, self.hkv_l * D)
        torch.cuda.synchronize()
        b = BoundCache(host, self.cache)
        if self.args.fp8:
            b.set_layer_scales(0, 1.0 / 32, 1.0 / 32)
        self._keep_bound = (host, b)
        return host, b, seq_id_array(ids)

    # -- algorithmic work of this rank ---------------------------------------------------
    def attn_bytes(self):
        return algorithmic_bytes(self.kv, self.ql, self.hq_l, self.hkv_l, self.bs, self.eb)

    def step_bytes(self):
        return self.attn_bytes() + write_bytes(self.ql, self.hkv_l, self.eb)

    def flops(self):
        return attention_flops(self.kv, self.ql, self.hq_l)


def time_workload(w, steps, warmup, dist, sample_clocks, e2e=True, extra_step=None):
    """Soak, W warm-up steps, K timed steps between two events on the launching stream
    (max over ranks), then the attention call alone (same inputs) and the host-buffer leg."""
    torch, pa = w.torch, w.pa
    step = extra_step or w.step

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=w.dev)
        if dist is not None:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    for _ in range(3):
        step()
    w.cache.check_errors(w.stream)
    t_one = timed(step, 5) / 5.0  # ms
    sampler = ClockSampler(w.dev.index).start() if sample_clocks else None
    t_load0 = time.perf_counter()
    soak = max(warmup, int(600.0 / max(t_one, 1e-3)))  # >= 0.6 s of the same step under the sampler
    soak = min(soak, 20000)
    if w.args.no_soak:
        soak = warmup
    for _ in range(soak - warmup):
        step()
    for _ in range(warmup):
        step()
    launches0 = pa.kernel_launch_count()
    total_ms = timed(step, steps)
    launches = pa.kernel_launch_count() - launches0
    n_attn = max(steps, min(2000, int(300.0 / max(t_one, 1e-3))))
    attn_ms = timed(w.attn_only, n_attn) / n_attn
    t_load1 = time.perf_counter()
    clocks = sampler.stop(t_load0, t_load1) if sampler else None
    w.cache.check_errors(w.stream)
    # The attention call timed ALONE, the way the peaks it is held against were measured
    # (best of 10 single launches, CUDA events): after a pause, so that the clocks are those
    # of a burst and not those the power cap settles at under the long loops above.
    if not w.args.no_soak:
        time.sleep(1.5)
    for _ in range(5):
        w.attn_only()
    burst = min(timed(w.attn_only, 1) for _ in range(10))
    res = {"ms_per_step": total_ms / steps, "attn_ms": burst, "attn_ms_sustained": attn_ms,
           "launches": int(launches), "launches_per_step": launches / steps, "clocks": clocks,
           "soak_steps": soak}
    if e2e:
        res["e2e"] = e2e_leg(w, steps, dist)
    return res


def e2e_leg(w, steps, dist):
    """The step from pinned host buffers through the host-buffer entry, host wall clock
    around synchronous calls, max over ranks.  Refills the pools (decode workloads), so it
    runs after everything that checks the device legs' results."""
    torch = w.torch

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    fn, h2d, d2h, entry = w.host_step_fn()
    for _ in range(5):
        fn()
    barrier()
    n_e2e = max(50 if w.decode_only else 10, min(steps, 100))  # enough calls for a steady figure
    t0 = time.perf_counter()
    for _ in range(n_e2e):
        fn()
    barrier()
    dt = torch.tensor([(time.perf_counter() - t0) / n_e2e], device=w.dev)
    if dist is not None:
        dist.all_reduce(dt, op=dist.ReduceOp.MAX)
    w.cache.check_errors(w.stream)
    return {"value": w.total_q / float(dt.item()), "unit": "tokens/s",
            "h2d_bytes_per_step": h2d(), "d2h_bytes_per_step": d2h,
            "ms_per_step": float(dt.item()) * 1e3, "steps": n_e2e, "entry": entry,
            "timed": "host wall clock around synchronous calls with pinned host buffers, max over ranks"}


# DRAM traffic per algorithmic byte of the attention call, from one profiler capture each on a
# small case of the same kernel (inputs larger than L2; traffic grows in proportion to the cached
# tokens, so it is scaled to the full launch by the algorithmic bytes).  The captures are
# summarised under profiles/.
TRAFFIC = {
    "splitkv": (1.007, "dram__bytes_read.sum + dram__bytes_write.sum of splitkv_kernel on the first 24 sequences "
                       "of configuration 3 (648.1 MB moved for 643.8 MB algorithmic), scaled by algorithmic bytes"),
    "tile64": (0.808, "dram__bytes_read.sum + dram__bytes_write.sum of tile_attention_tc64_kernel on one sequence "
                      "of configuration 4 (61.0 MB moved for 75.5 MB algorithmic: the 32 CTAs that share a kv "
                      "head are served from L2), scaled by the number of sequences"),
}


def roofline_of(w, res, peaks):
    """achieved = algorithmic bytes (or flops) of one attention call / its average duration
    in a back-to-back loop of the timed region (CUDA events), against the measured HBM peak
    or, for the tensor-bound workload, the measured sustained bf16 peak (the loop runs under
    the power cap like the seconds-long GEMM loop that peak comes from).  `burst` gives the
    same call timed alone (best of 10 single launches after a pause) against the burst peak."""
    tensor_bound = w.name == "c4"
    burst_ms, loop_ms = res["attn_ms"], res["attn_ms_sustained"]
    if tensor_bound:
        work, unit, scale = w.flops(), "TFLOP/s", 1e12
        peak, peak_burst = peaks["tf_sustained"] or peaks["tf"], peaks["tf"]
        kernel = "tile_attention_tc64_kernel" if w.bs == 16 and not w.args.fp8 else "tile_attention_tc_kernel"
    else:
        work, unit, scale = w.attn_bytes(), "GB/s", 1e9
        peak = peak_burst = peaks["hbm"]
        kernel = "splitkv_kernel" if w.decode_only else "splitkv_kernel + tile attention kernel"
    achieved = work / (loop_ms * 1e-3) / scale
    burst = work / (burst_ms * 1e-3) / scale
    traffic, traffic_note = None, "not captured for this combination of kernels"
    if w.bs == 16 and not w.args.fp8 and (w.decode_only or tensor_bound):
        ratio, traffic_note = TRAFFIC["splitkv" if w.decode_only else "tile64"]
        traffic = int(ratio * w.attn_bytes())
    return {"bound": "tensor" if tensor_bound else "hbm", "achieved": achieved, "peak": peak, "unit": unit,
            "frac": achieved / peak, "traffic": traffic, "traffic_source": traffic_note,
            "peak_source": peaks["kind"] + (", sustained bf16 figure" if tensor_bound and peaks["tf_sustained"] else ""),
            "kernel": kernel, "kernel_ms": loop_ms,
            "burst": {"kernel_ms": burst_ms, "achieved": burst, "peak": peak_burst, "frac": burst / peak_burst},
            "timing": "average of a back-to-back loop of the attention call inside the timed region (CUDA "
                      "events); `burst` = best of 10 single calls after a 1.5 s pause, as the burst peak was measured",
            "algorithmic_bytes": w.attn_bytes(), "algorithmic_flops": w.flops(), "per": "rank"}


# ---------------------------------------------------------------------------------------
def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c3", choices=["c1", "c2", "c3", "c4", "c5"])
    ap.add_argument("--gather", nargs="?", const="nccl", default=None, choices=["nccl", "peer"],
                    help="all-gather the head outputs inside the step (N > 1): over NCCL, or "
                         "'peer' = the library's stores into the other ranks' buffers "
                         "(symmetric memory), checked once against NCCL")
    ap.add_argument("--fp8", action="store_true",
                    help="E4M3 KV cache (one byte per element)")
    ap.add_argument("--producer", action="store_true",
                    help="the step's write becomes the fused QK-norm + rotary + KV-write launch")
    ap.add_argument("--two-launches", action="store_true",
                    help="decode step as write kernel + attention kernel instead of one launch")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--no-also", action="store_true", help="headline workload only")
    ap.add_argument("--no-soak", action="store_true",
                    help="skip the 0.6 s soak and the pause before the burst timing (profiler captures: few "
                         "launches before the captured ones)")
    ap.add_argument("--seqs", type=int, default=0, help="use only the first N sequences (small captures)")
    ap.add_argument("--pool-blocks", type=int, default=0, help="override the pool size in blocks")
    ap.add_argument("--block-size", type=int, default=16, choices=[8, 16, 32],
                    help="tokens per pool block (the configurations are quoted on 16)")
    ap.add_argument("--head-size", type=int, default=128, choices=[32, 64, 80, 96, 112, 120, 128, 192, 256],
                    help="head size of the decode workloads (other than 128: 16-bit pools, 16-token blocks)")
    ap.add_argument("--as-rank-of", type=int, default=0, metavar="N",
                    help="on one GPU, run the share of rank 0 of an N-way kv-head split "
                         "(to study a rank's step without N GPUs)")
    args = ap.parse_args()
    global D
    D = args.head_size
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    args.warmup = max(args.warmup, 3)

    import torch
    import paged_attn_b200 as pa
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback "
                         "(use --impl reference for the CPU path)")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    shard_world = args.as_rank_of if (args.as_rank_of and world == 1) else world
    peaks = measured_peaks()

    w = Workload(args.workload, rank if world > 1 else 0, shard_world, local_rank, args, seqs=args.seqs)
    from paged_attn_b200 import sharding
    do_gather = args.gather is not None and world > 1
    peer = None
    step_fn = None
    if do_gather:
        if args.gather == "peer":
            import torch.distributed._symmetric_memory as symm_mem
            # two full-width output buffers (alternating, so that a rank never overwrites what a
            # slower rank is still reading) and the flag words, all in symmetric memory
            fulls = [symm_mem.empty((w.total_q, w.Hq, D), dtype=torch.bfloat16, device=w.dev) for _ in range(2)]
            flag_t = symm_mem.empty((64,), dtype=torch.int32, device=w.dev)
            flag_t.zero_()
            hd = [symm_mem.rendezvous(t, dist.group.WORLD) for t in fulls]
            hf = symm_mem.rendezvous(flag_t, dist.group.WORLD)
            dist.barrier()
            peer = {"fulls": fulls, "out_ptrs": [[int(p) for p in h.buffer_ptrs] for h in hd],
                    "flag_ptrs": [int(p) for p in hf.buffer_ptrs], "epoch": 0}

        def step_fn():
            w.step()
            if peer is not None:
                peer["epoch"] += 1
                k = peer["epoch"] & 1
                w.cache.gather_heads_peer_store(w.out, w.total_q, w.hq_l, world, rank, peer["out_ptrs"][k],
                                                peer["flag_ptrs"], peer["epoch"], stream=w.stream)
            else:
                sharding.gather_heads(w.out, world)
        if peer is not None:
            for _ in range(3):
                step_fn()
            torch.cuda.synchronize()
            ref_full = sharding.gather_heads(w.out, world)
            got_full = peer["fulls"][peer["epoch"] & 1]
            same = torch.equal(ref_full.view(torch.int16), got_full.view(torch.int16))
            flag = torch.tensor([1 if same else 0], device=w.dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            peer["checked"] = bool(flag.item())
            dist.barrier()

    res = time_workload(w, args.steps, args.warmup, dist, sample_clocks=(rank == 0), e2e=False,
                        extra_step=step_fn)
    roof = roofline_of(w, res, peaks)

    cpu_base = None
    if (rank == 0 and world == 1 and not args.as_rank_of and w.decode_only and not args.no_cpu_baseline
            and not args.fp8 and not args.seqs):
        cpu_base = cpu_baseline_and_spot_check(w)
    if not args.no_e2e:
        res["e2e"] = e2e_leg(w, args.steps, dist)

    also = None
    if world == 1 and not args.no_also and not args.as_rank_of and args.workload == "c3" and not args.seqs:
        kv_h, ql_h, Hq_h, Hkv_h = w.kv, w.ql, w.Hq, w.Hkv
        step_b = w.step_bytes()
        del w
        torch.cuda.empty_cache()
        also = {}
        for name in ("c2", "c5", "c4"):  # the tensor-bound leg last: it heats the GPU most
            time.sleep(1.0)
            wl = Workload(name, 0, 1, local_rank, args)
            r = time_workload(wl, args.steps, args.warmup, None, sample_clocks=True, e2e=not args.no_e2e)
            rf = roofline_of(wl, r, peaks)
            also[name] = {
                "workload": workload_config(name, 1, wl.kv, wl.ql, wl.Hq, wl.Hkv, wl.bs)["workload"],
                "value": wl.total_q / (r["ms_per_step"] * 1e-3), "unit": "tokens/s",
                "ms_per_step": r["ms_per_step"], "kernel_ms": rf["kernel_ms"],
                "gpu_launches_per_step": r["launches_per_step"], "roofline": rf,
                "e2e": r.get("e2e"), "clocks": r["clocks"],
            }
            del wl
            torch.cuda.empty_cache()
        w_meta = (kv_h, ql_h, Hq_h, Hkv_h, step_b)
    else:
        w_meta = (w.kv, w.ql, w.Hq, w.Hkv, w.step_bytes())

    if rank == 0:
        kv, ql, Hq, Hkv, step_b = w_meta
        ms_per_step = res["ms_per_step"]
        total_q = int(np.sum(ql))
        line = {
            "metric": "paged_decode_attn_tokens_per_s", "value": total_q / (ms_per_step * 1e-3),
            "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(args.workload, shard_world, kv, ql, Hq, Hkv, args.block_size),
            "roofline": roof, "cpu_baseline": cpu_base, "e2e": res.get("e2e"),
            "gpu_launches": res["launches"], "clocks": res["clocks"],
            "step_bytes": step_b, "step_gbs": step_b / (ms_per_step * 1e-3) / 1e9,
            "soak_steps_before_warmup": res["soak_steps"],
        }
        if also:
            line["also"] = also
        if args.as_rank_of and world == 1:
            line["config"]["sharding"] = (f"ONE GPU running rank 0's share of a {args.as_rank_of}-way "
                                          "kv-head split (study run, not a multi-GPU number)")
        if args.fp8:
            line["config"]["kv_cache"] = "E4M3 bytes, scales 1/32; q, out and the written k, v bf16"
            line["config"]["l2"] = l2_statement(kv, Hkv // shard_world, 1)
            line["dtype"] = "e4m3 cache, bf16 queries and output, fp32 accumulation"
        if args.producer:
            line["config"]["producer"] = "QK norm + rotary embedding fused into the KV write launch"
        if args.two_launches:
            line["config"]["step"] = "write kernel, then attention kernel (two launches)"
        if do_gather:
            line["config"]["gather"] = (
                "stores into every rank's buffer over NVLink + one flag per rank pair, inside the "
                "step; equal to an NCCL all_gather of the same outputs: " + str(peer["checked"])
                if peer is not None else "NCCL all_gather of head outputs inside the step")
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


def cpu_baseline_and_spot_check(w):
    """Times the CPU path on a bounded sample of the same workload (the sample the
    reference arm uses) and, on the same sequences, spot-checks the GPU result of this
    very run against the fp64 oracle."""
    import torch
    T = _oracle_tools()
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from gpu_util import to_bits
    n_s = cpu_sample_size(w.kv)
    sample = CpuSample(w.name, w.kv, w.ql, w.Hq, w.Hkv, w.bs, n_s)
    sample.step()
    t0 = time.perf_counter()
    reps = 0
    while reps < 3 or (time.perf_counter() - t0 < 10.0 and reps < 50):
        sample.step()
        reps += 1
    dt = (time.perf_counter() - t0) / reps
    # spot check of the GPU output of this run: 4 rows per sampled sequence, against the
    # oracle reading the GPU's own pool contents (blocks of the sample compacted)
    bs = w.bs
    nblk = (w.kv[:n_s] + bs - 1) // bs
    ids = np.concatenate([w.tables_h[s, :nblk[s]] for s in range(n_s)])
    idt = torch.from_numpy(ids.astype(np.int64)).to(w.k_pool.device)
    k_c, v_c = to_bits(w.k_pool[idt]), to_bits(w.v_pool[idt])
    tables_c = np.zeros((n_s, w.tables_h.shape[1]), dtype=np.int32)
    pos = 0
    for s in range(n_s):
        tables_c[s, :nblk[s]] = np.arange(pos, pos + nblk[s])
        pos += nblk[s]
    q_c = to_bits(w.q[:n_s])
    lens_c = np.ascontiguousarray(w.kv[:n_s].astype(np.int32))
    rows = [(s, 0, (7 * s + 3 * i) % w.Hq) for s in range(n_s) for i in range(4)]
    ref = T.attention_oracle_rows(rows, q_c, k_c, v_c, tables_c, lens_c, None, w.Hq, w.Hkv,
                                  tables_c.shape[1], w.scale)
    got_all = T.bf16_to_f32(to_bits(w.out[:n_s]))
    got = np.stack([got_all[s, hq] for (s, _, hq) in rows])
    stats = T.check_attention(got, ref, "bench spot check")
    return {"value": n_s / dt, "unit": "tokens/s", "cores": sample.cores, "kind": "port",
            "sample": sample.describe(reps), "ms_per_step": dt * 1e3,
            "gpu_spot_check": {"rows": len(rows), "max_abs": stats["max_abs"],
                               "max_over_bound": stats["max_over_bound"]}}


if __name__ == "__main__":
    main()
