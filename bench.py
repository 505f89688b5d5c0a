#!/usr/bin/env python
"""Benchmark of the paged-attention hot path on B200.

A step is one pass of the path over one synthetic batch: the KV block write of
the step's new tokens (reshape_and_cache) followed by paged attention over the
block-table cache, exactly the order one transformer layer runs them.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2]
  python bench.py --impl reference ...      # the CPU path, timed on the host cores

Default workload ("c2"): Qwen3-8B-shaped decode, 32 query / 8 KV heads, head
128, block 16, 64 sequences with contexts uniform in [1024, 8192], bf16 N(0,1),
block tables a random permutation of a 40000-block pool.  With N GPUs the KV
heads are sharded N ways (each rank owns its heads' pool, no data-path
collective) and the batch grows to 64*N sequences, so per-GPU bytes stay fixed
(weak scaling).  Other workloads (c1, c3, c4, c5) are for study, not the headline.

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
for _p in (os.path.join(ROOT, "mlx-node_b200"), os.path.join(ROOT, "tests")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

D, BS = 128, 16
L2_BYTES = 126 << 20


# ---------------------------------------------------------------------------------------
def workload_lengths(name: str, world: int):
    """(kv_lens, q_lens, Hq, Hkv, NB).  kv_lens count the tokens written this step."""
    from pa_testlib import config_lengths
    if name == "c2" and world > 1:
        parts = [config_lengths("c2", seed=r) for r in range(world)]
        kv = np.concatenate([x[0] for x in parts])
        ql = np.concatenate([x[1] for x in parts])
        return kv, ql, 32, 8, 40000 * world
    return config_lengths(name)


def algorithmic_bytes(kv_lens, q_lens, Hq, Hkv, kv_elem_bytes=2) -> int:
    """One pass over the live KV bytes (once per KV head, whatever the group size or the
    number of splits), the block-table entries and lengths, Q read and O written."""
    kv = int(np.sum(kv_lens))
    blocks = int(np.sum((np.asarray(kv_lens) + BS - 1) // BS))
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
        return float(m["hbm_gbs"]), float(m["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
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
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx = float(parts[1])
            except ValueError:
                continue
            for n, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx,
                "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------------------
def run_reference(args, rank: int, world: int) -> None:
    """The reference's CPU implementation of the path on the host cores.  The
    reference itself cannot be built here (Metal kernels; MLX sources absent; no Rust
    toolchain), so this times the oracle port of its software path
    (crates/mlx-sys/src/mlx.cpp:4080-4159) plus the scatter form of its block write,
    with every host thread, on a bounded sample of the same workload."""
    if rank != 0:
        return
    from pa_testlib import Case, oracle, p, write_oracle
    kv, ql, Hq, Hkv, _ = workload_lengths(args.workload, max(world, 1))
    if args.workload in ("c4", "c5"):
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference has no paged multi-token attention "
                          "(crates/mlx-paged-attn/src/scheduler.rs:237-242); only decode workloads "
                          "have a CPU path"}))
        return
    lib = oracle()
    lib.oracle_set_num_threads(len(os.sched_getaffinity(0)))
    cores = int(lib.oracle_num_threads())
    n_s = min(len(kv), max(cores, 8))
    kv_s, ql_s = kv[:n_s], ql[:n_s]
    nb = int(((kv_s + BS - 1) // BS).sum())
    case = Case(kv_s, ql_s, Hq, Hkv, nb + 8, seed=0, bs=BS)
    k_pool, v_pool = case.k_pool, case.v_pool
    k_pool[k_pool == 0x7FFF] = 0
    v_pool[v_pool == 0x7FFF] = 0
    out = np.zeros((case.S, Hq, D), dtype=np.uint16)

    def step():
        write_oracle(k_pool, v_pool, case.k_new, case.v_new, case.slot_mapping, Hkv)
        rc = lib.baseline_mlx_paged_forward(p(out), p(case.q), p(k_pool), p(v_pool),
                                            p(case.block_tables), p(case.kv_lens), case.S, Hq,
                                            Hkv, D, BS, case.MB, case.scale)
        assert rc == 0
    for _ in range(min(args.warmup, 1)):
        step()
    t0 = time.perf_counter()
    steps = max(1, min(args.steps, 5))
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    value = n_s / dt
    sample = f"first {n_s} of {len(kv)} sequences of workload {args.workload}, {steps} step(s)"
    line = {
        "impl": "reference", "metric": "paged_decode_attn_tokens_per_s", "value": value,
        "unit": "tokens/s", "n_gpus": args.gpus, "steps": steps, "warmup": min(args.warmup, 1),
        "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args.workload, max(world, 1), kv, ql, Hq, Hkv),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def l2_statement(kv, hkv_local, kv_elem_bytes=2):
    """Whether one step's KV bytes per GPU exceed the L2 (no flush is done between steps)."""
    step = int(np.sum(kv)) * 2 * hkv_local * D * kv_elem_bytes
    if step > L2_BYTES:
        return f"inputs larger than L2 ({step / 1e6:.0f} MB of KV per step and GPU, L2 126 MB)"
    return (f"working set {step / 1e6:.0f} MB fits in the 126 MB L2 and nothing flushes it: "
            "L2-resident timing, reported for latency only")


def workload_config(name, world, kv, ql, Hq, Hkv):
    return {"workload": f"{name}: {len(kv)} sequences, {Hq} query / {Hkv} kv heads, head {D}, "
                        f"block {BS}, {int(np.sum(ql))} query tokens over {int(np.sum(kv))} cached "
                        f"tokens; step = KV write + paged attention",
            "sharding": f"kv heads split {world} ways, batch x{world}" if world > 1 else "single GPU",
            "l2": l2_statement(kv, Hkv // max(world, 1))}


# ---------------------------------------------------------------------------------------
def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=["c1", "c2", "c3", "c4", "c5"])
    ap.add_argument("--gather", nargs="?", const="nccl", default=None, choices=["nccl", "peer"],
                    help="all-gather the head outputs inside the step (N > 1): over NCCL, or "
                         "'peer' = the library's stores into the other ranks' buffers "
                         "(symmetric memory), checked once against NCCL")
    ap.add_argument("--fp8", action="store_true",
                    help="E4M3 KV cache (one byte per element); decode workloads only")
    ap.add_argument("--producer", action="store_true",
                    help="the step's write becomes the fused QK-norm + rotary + KV-write launch")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--seqs", type=int, default=0, help="use only the first N sequences (small captures)")
    ap.add_argument("--pool-blocks", type=int, default=0, help="override the pool size in blocks")
    ap.add_argument("--block-size", type=int, default=16, choices=[8, 16, 32],
                    help="tokens per pool block (the configurations are quoted on 16)")
    args = ap.parse_args()
    global BS
    BS = args.block_size
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

    kv, ql, Hq, Hkv, NB = workload_lengths(args.workload, world)
    if args.seqs:
        kv, ql = kv[:args.seqs], ql[:args.seqs]
    if BS != 16:  # the same pool bytes in larger blocks
        NB = max(NB * 16 // BS, int(((kv + BS - 1) // BS).sum()))
    if args.pool_blocks:
        NB = args.pool_blocks
    assert int(((kv + BS - 1) // BS).sum()) <= NB
    from paged_attn_b200 import sharding
    ka, kb = sharding.kv_head_range(rank, world, Hkv)
    qa, qb = sharding.q_head_range(rank, world, Hq, Hkv)
    hkv_l, hq_l = kb - ka, qb - qa
    S, total_q = len(kv), int(np.sum(ql))
    nblk = (kv + BS - 1) // BS
    MB = int(nblk.max())
    rng = np.random.Generator(np.random.PCG64(0))  # same tables on every rank (one host allocator)
    perm = rng.permutation(NB).astype(np.int32)
    tables_h = np.zeros((S, MB), dtype=np.int32)
    slots_all = np.empty(int(kv.sum()), dtype=np.int64)
    is_new = np.zeros(int(kv.sum()), dtype=bool)
    cu_kv = np.concatenate([[0], np.cumsum(kv)])
    cu_q = np.concatenate([[0], np.cumsum(ql)]).astype(np.int32)
    pos = 0
    for s in range(S):
        tables_h[s, :nblk[s]] = perm[pos:pos + nblk[s]]
        pos += nblk[s]
        t = np.arange(kv[s])
        slots_all[cu_kv[s]:cu_kv[s + 1]] = tables_h[s, t // BS].astype(np.int64) * BS + t % BS
        is_new[cu_kv[s + 1] - ql[s]:cu_kv[s + 1]] = True
    dev = torch.device("cuda", local_rank)
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
        k_pool = torch.zeros(NB, hkv_l, D // 16, BS, 16, dtype=torch.uint8, device=dev)
        v_pool = torch.zeros(NB, hkv_l, D, BS, dtype=torch.uint8, device=dev)
    else:
        k_pool = torch.zeros(NB, hkv_l, D // 8, BS, 8, dtype=torch.bfloat16, device=dev)
        v_pool = torch.zeros(NB, hkv_l, D, BS, dtype=torch.bfloat16, device=dev)
    cache = pa.PagedCache(BS, NB, D, hkv_l, device=local_rank, key_pools=[k_pool], value_pools=[v_pool],
                          fp8=args.fp8)
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
    k_new, v_new = k_all[new_idx].contiguous(), v_all[new_idx].contiguous()
    slots = slots_all_d[new_idx].contiguous()
    del k_all, v_all, old_slots
    q = randn_bf16(total_q, hq_l, D)
    out = torch.zeros(total_q, hq_l, D, dtype=torch.bfloat16, device=dev)
    tables = torch.from_numpy(tables_h).to(dev)
    lens = torch.from_numpy(kv.astype(np.int32)).to(dev)
    ws_bytes = cache.workspace_bytes()
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
    scale = 1.0 / math.sqrt(D)
    decode_only = bool((ql == 1).all())
    kv_i32 = np.ascontiguousarray(kv.astype(np.int32))
    do_gather = args.gather is not None and world > 1
    peer = None
    if do_gather and args.gather == "peer":
        import torch.distributed._symmetric_memory as symm_mem
        # two full-width output buffers (alternating, so that a rank never overwrites what a
        # slower rank is still reading) and the flag words, all in symmetric memory
        fulls = [symm_mem.empty((total_q, Hq, D), dtype=torch.bfloat16, device=dev) for _ in range(2)]
        flag_t = symm_mem.empty((64,), dtype=torch.int32, device=dev)
        flag_t.zero_()
        hd = [symm_mem.rendezvous(t, dist.group.WORLD) for t in fulls]
        hf = symm_mem.rendezvous(flag_t, dist.group.WORLD)
        dist.barrier()
        peer = {"fulls": fulls, "out_ptrs": [[int(p) for p in h.buffer_ptrs] for h in hd],
                "flag_ptrs": [int(p) for p in hf.buffer_ptrs], "epoch": 0}
    stream = torch.cuda.current_stream().cuda_stream

    if args.producer:
        # projections in, rotated queries out (separate buffer so every step does the same work)
        q_raw = q
        q = torch.empty_like(q_raw)
        norm_w = torch.ones(D, dtype=torch.bfloat16, device=dev)
        pos_h = np.concatenate([kv[s] - ql[s] + np.arange(ql[s]) for s in range(S)]).astype(np.int32)
        positions = torch.from_numpy(pos_h).to(dev)

    def step():
        if args.producer:
            cache.qk_norm_rope_and_cache(q, q_raw, k_new, v_new, norm_w, norm_w, 1e-6, positions,
                                         1.0e6, D, slots, total_q, hq_l, hq_l * D, hq_l * D,
                                         hkv_l * D, hkv_l * D, stream=stream)
        else:
            cache.reshape_and_cache(k_new, v_new, slots, total_q, hkv_l * D, hkv_l * D, stream=stream)
        if decode_only:
            cache.decode(out, q, tables, lens, S, hq_l, MB, scale, ws, ws_bytes, stream=stream)
        else:
            cache.varlen(out, q, tables, lens, cu_q, S, hq_l, MB, scale, ws, ws_bytes,
                         max_context_len=int(kv.max()), stream=stream, context_lens_host=kv_i32)
        if do_gather and peer is not None:
            peer["epoch"] += 1
            k = peer["epoch"] & 1
            cache.gather_heads_peer_store(out, total_q, hq_l, world, rank, peer["out_ptrs"][k],
                                          peer["flag_ptrs"], peer["epoch"], stream=stream)
        elif do_gather:
            sharding.gather_heads(out, world)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        """K steps between two events on the launching stream; returns ms (max over ranks)."""
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if dist is not None:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    for _ in range(args.warmup):
        step()
    cache.check_errors(stream)
    if peer is not None:
        torch.cuda.synchronize()
        ref_full = sharding.gather_heads(out, world)
        got_full = peer["fulls"][peer["epoch"] & 1]
        same = torch.equal(ref_full.view(torch.int16), got_full.view(torch.int16))
        flag = torch.tensor([1 if same else 0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        peer["checked"] = bool(flag.item())
        dist.barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = pa.kernel_launch_count()
    total_ms = timed(step, args.steps)
    launches = pa.kernel_launch_count() - launches0
    cache.check_errors(stream)

    # dominant kernel alone (attention call = main kernel + its merge), same inputs
    def attn_only():
        if decode_only:
            cache.decode(out, q, tables, lens, S, hq_l, MB, scale, ws, ws_bytes, stream=stream)
        else:
            cache.varlen(out, q, tables, lens, cu_q, S, hq_l, MB, scale, ws, ws_bytes,
                         max_context_len=int(kv.max()), stream=stream, context_lens_host=kv_i32)
    attn_ms = timed(attn_only, args.steps) / args.steps

    # end to end through the host-buffer entry: H2D of the step's inputs + kernels + D2H
    e2e = None
    if decode_only and not args.no_e2e:
        pin = lambda t: t.cpu().pin_memory()
        q_h, k_h, v_h, out_h = pin(q), pin(k_new), pin(v_new), torch.empty_like(q, device="cpu").pin_memory()
        slots_h, tables_p, lens_h = pin(slots), pin(tables), pin(lens)

        def host_step():
            cache.decode_step_host(out_h, q_h, k_h, v_h, slots_h, tables_p, lens_h, S, hq_l, MB, scale)
        for _ in range(3):
            host_step()
        barrier()
        t0 = time.perf_counter()
        n_e2e = max(10, min(args.steps, 100))
        for _ in range(n_e2e):
            host_step()
        barrier()
        dt = torch.tensor([(time.perf_counter() - t0) / n_e2e], device=dev)
        if dist is not None:
            dist.all_reduce(dt, op=dist.ReduceOp.MAX)
        h2d = sum(t.numel() * t.element_size() for t in (q_h, k_h, v_h, slots_h, tables_p, lens_h))
        e2e = {"value": total_q / float(dt.item()), "unit": "tokens/s",
               "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(out_h.numel() * 2),
               "ms_per_step": float(dt.item()) * 1e3,
               "timed": "host wall clock around synchronous calls, max over ranks"}
    clocks = sampler.stop() if rank == 0 else None

    # per-rank algorithmic work (this rank's heads)
    eb = 1 if args.fp8 else 2
    kv_bytes = algorithmic_bytes(kv, ql, hq_l, hkv_l, eb)
    flops = attention_flops(kv, ql, hq_l)
    hbm_peak, tf_peak, peak_kind = measured_peaks()
    tensor_bound = args.workload == "c4"
    if tensor_bound:
        achieved = flops / (attn_ms * 1e-3) / 1e12
        # ncu capture of one sequence of this workload (profiles/tile_attention_tc_kernel_c4_ncu.md):
        # 61.1 MB of DRAM traffic per sequence per launch, scaled by the sequence count
        roof = {"bound": "tensor", "achieved": achieved, "peak": tf_peak, "unit": "TFLOP/s",
                "frac": achieved / tf_peak,
                "traffic": None if args.fp8 or BS != 16 else int(61.1e6 * S * hkv_l / 8),
                "traffic_source": None if args.fp8 or BS != 16
                else "ncu dram bytes of a 1-sequence capture x sequences"}
    else:
        achieved = kv_bytes / (attn_ms * 1e-3) / 1e9
        # ncu capture of a 16-sequence case of this workload
        # (profiles/splitkv_kernel_c2_16seq_ncu_full.md): DRAM read+write = 1.021 x the
        # algorithmic bytes; traffic grows in proportion with the units processed
        # (FP8: profiles/splitkv_kernel_fp8.md, read + write = 1.047 x the algorithmic bytes)
        traffic = None if not decode_only else int((1.047 if args.fp8 else 1.021) * kv_bytes)
        roof = {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                "frac": achieved / hbm_peak, "traffic": traffic,
                "traffic_source": "ncu dram bytes of a 16-sequence capture, scaled by algorithmic bytes"
                if traffic else None}
    roof.update({"kernel": "tile_attention" if tensor_bound else "splitkv_kernel (+ merge)",
                 "peak_source": f"{peak_kind} (MEASURED_PEAKS.json)" if peak_kind == "measured"
                 else "fallback", "kernel_ms": attn_ms, "algorithmic_bytes": kv_bytes,
                 "algorithmic_flops": flops, "per": "rank"})

    cpu_base = None
    if rank == 0 and world == 1 and decode_only and not args.no_cpu_baseline and not args.fp8:
        cpu_base = cpu_baseline_and_spot_check(kv, ql, Hq, Hkv, tables_h, k_pool, v_pool, q, out,
                                               scale)
    if rank == 0:
        ms_per_step = total_ms / args.steps
        line = {
            "metric": "paged_decode_attn_tokens_per_s", "value": total_q / (ms_per_step * 1e-3),
            "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(args.workload, world, kv, ql, Hq, Hkv),
            "roofline": roof, "cpu_baseline": cpu_base, "e2e": e2e, "gpu_launches": int(launches),
            "clocks": clocks,
            "step_bytes": kv_bytes + write_bytes(ql, hkv_l, eb),
            "step_gbs": (kv_bytes + write_bytes(ql, hkv_l, eb)) / (ms_per_step * 1e-3) / 1e9,
        }
        if args.fp8:
            line["config"]["kv_cache"] = "E4M3 bytes, scales 1/32; q, out and the written k, v bf16"
            line["config"]["l2"] = l2_statement(kv, hkv_l, 1)
            line["dtype"] = "e4m3 cache, bf16 queries and output, fp32 accumulation"
        if args.producer:
            line["config"]["producer"] = "QK norm + rotary embedding fused into the KV write launch"
        if do_gather:
            line["config"]["gather"] = (
                "stores into every rank's buffer over NVLink + one flag per rank pair, inside the "
                "step; equal to an NCCL all_gather of the same outputs: " + str(peer["checked"])
                if peer is not None else "NCCL all_gather of head outputs inside the step")
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


def cpu_baseline_and_spot_check(kv, ql, Hq, Hkv, tables_h, k_pool, v_pool, q, out, scale):
    """Times the CPU path on a bounded sample of the same workload (the first n
    sequences, their blocks compacted into a small pool) and uses the same sample to
    spot-check the GPU result of this very run against the fp64 oracle."""
    import torch
    from pa_testlib import attention_oracle_rows, bf16_to_f32, check_attention, oracle, p
    from gpu_util import to_bits
    lib = oracle()
    lib.oracle_set_num_threads(len(os.sched_getaffinity(0)))
    cores = int(lib.oracle_num_threads())
    n_s = min(len(kv), max(cores, 8))
    nblk = (kv[:n_s] + BS - 1) // BS
    ids = np.concatenate([tables_h[s, :nblk[s]] for s in range(n_s)])
    idt = torch.from_numpy(ids.astype(np.int64)).to(k_pool.device)
    k_c, v_c = to_bits(k_pool[idt]), to_bits(v_pool[idt])
    tables_c = np.zeros((n_s, tables_h.shape[1]), dtype=np.int32)
    pos = 0
    for s in range(n_s):
        tables_c[s, :nblk[s]] = np.arange(pos, pos + nblk[s])
        pos += nblk[s]
    q_c = to_bits(q[:n_s])
    lens_c = np.ascontiguousarray(kv[:n_s].astype(np.int32))
    out_c = np.zeros((n_s, Hq, D), dtype=np.uint16)

    def run():
        rc = lib.baseline_mlx_paged_forward(p(out_c), p(q_c), p(k_c), p(v_c), p(tables_c), p(lens_c),
                                            n_s, Hq, Hkv, D, BS, tables_c.shape[1], scale)
        assert rc == 0
    run()
    t0 = time.perf_counter()
    reps = 0
    while reps < 3 or (time.perf_counter() - t0 < 10.0 and reps < 50):
        run()
        reps += 1
    dt = (time.perf_counter() - t0) / reps
    # spot check of the GPU output of this run: 4 rows per sampled sequence
    rows = [(s, 0, (7 * s + 3 * i) % Hq) for s in range(n_s) for i in range(4)]
    ref = attention_oracle_rows(rows, q_c, k_c, v_c, tables_c, lens_c, None, Hq, Hkv,
                                tables_c.shape[1], scale)
    got_all = bf16_to_f32(to_bits(out[:n_s]))
    got = np.stack([got_all[s, hq] for (s, _, hq) in rows])
    stats = check_attention(got, ref, "bench spot check")
    return {"value": n_s / dt, "unit": "tokens/s", "cores": cores, "kind": "port",
            "sample": f"first {n_s} of {len(kv)} sequences, attention only, {reps} repetitions",
            "ms_per_pass": dt * 1e3,
            "gpu_spot_check": {"rows": len(rows), "max_abs": stats["max_abs"],
                               "max_over_bound": stats["max_over_bound"]}}


if __name__ == "__main__":
    main()
