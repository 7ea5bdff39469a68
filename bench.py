#!/usr/bin/env python3
"""MLA decode benchmark: layer-tokens/s of one Multi-head Latent Attention layer call, with the
roofline of the latent-cache read and a host-CPU baseline beside it.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload batched|single|verify|longctx]
    python bench.py --impl reference ...      # the CPU statement of the reference math, timed

A step is one layer call (q compress/expand, kv compress + append, split-KV attention over the
paged latent cache, both output projections) for every sequence of the batch.  Default
workload: batched decode, 64 sequences per GPU, context lengths uniform in [1024, 8192], 64-token
pages with a scrambled block table, bf16 with fp32 accumulation, synthetic seeded inputs.
Under torchrun (one rank per GPU) sequences are sharded by rank with no data-path collective
(weak scaling: 64 sequences per GPU); `longctx` splits one sequence along the KV axis instead
and exchanges per-GPU partials with one all-gather.  Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

ROW_BYTES = 1152  # algorithmic bytes per cached token attended: 576 bf16, read once


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="batched", choices=["batched", "single", "verify", "longctx"])
    ap.add_argument("--batch", type=int, default=0, help="sequences per GPU (default: the workload's)")
    ap.add_argument("--ctx-lo", type=int, default=0)
    ap.add_argument("--ctx-hi", type=int, default=0)
    ap.add_argument("--attn-impl", type=int, default=0)
    ap.add_argument("--gemm-impl", type=int, default=0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--cpu-seqs", type=int, default=8, help="sequences in the bounded CPU-baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--merge-kernel", action="store_true", help="merge the split-KV partials in a kernel of its own")
    return ap.parse_args()


def workload_shape(a):
    """(batch per GPU, q_len, ctx_lo, ctx_hi, causal, description)."""
    if a.workload == "batched":
        w = (64, 1, 1024, 8192, False, "batched decode: 64 seqs/GPU, ctx~U[1024,8192], 64-token pages, scrambled block table")
    elif a.workload == "single":
        w = (1, 1, 4096, 4096, False, "decode at batch 1 over a 4096-token cache")
    elif a.workload == "verify":
        w = (32, 16, 16384, 16384, True, "speculative-verify block: 16 causal query tokens x 32 seqs over 16384-token caches")
    else:
        w = (1, 1, 131072, 131072, False, "one 131072-token sequence, split-KV across the GPUs, all-gather of partials")
    b, q, lo, hi, causal, desc = w
    return (a.batch or b, q, a.ctx_lo or lo, a.ctx_hi or hi, causal, desc)


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.idx, self.proc, self.lines = device_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.idx)], stdout=subprocess.PIPE, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def hbm_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def ncu_traffic(workload: str):
    """DRAM bytes per launch of the attention kernel from the committed ncu capture, scaled to
    this workload by cached rows (profiles/attn_traffic.json: bytes per cached row)."""
    p = os.path.join(ROOT, "profiles", "attn_traffic.json")
    if not os.path.exists(p):
        return None
    try:
        return json.load(open(p))
    except Exception:
        return None


def make_inputs(cfg, a, rank, batch, q_len, lo, hi):
    from fastar_b200 import synth
    lens = synth.context_lengths(a.seed, batch, lo, hi, (rank,))
    return lens


def cpu_sample(cfg, a, lens, q_len, causal, n_seqs, n_threads=0, target_s=10.0):
    """Times the CPU oracle on the first n_seqs sequences of this workload (bounded sample),
    repeating the pass until about target_s seconds of CPU work have been timed.
    Returns (layer-tokens/s, cores, seconds, description)."""
    from fastar_b200 import mla, synth
    from oracle import oracle as O
    ocfg = O.make_cfg(cfg.preset, n_threads=n_threads)
    w = synth.weights_rounded(synth.layer_weights_f32(cfg, a.seed, 0))
    d = mla.dims_of(cfg)
    n_seqs = min(n_seqs, len(lens))
    caches, hs = [], []
    for b in range(n_seqs):
        L = int(lens[b])
        c = np.zeros((L + q_len, d["row"]), np.float32)
        c[:L] = synth.from_bf16_bits(synth.to_bf16_bits(synth.cache_rows_f32(cfg, a.seed, b, L)))
        caches.append(c)
        hs.append(synth.from_bf16_bits(synth.to_bf16_bits(synth.hidden_f32(cfg, a.seed, q_len, (b,)))))
    O.mla_forward(ocfg, w, hs[0], int(lens[0]), caches[0], causal=causal, want_trace=False)  # warm-up
    t0 = time.perf_counter()
    passes = 0
    while True:
        for b in range(n_seqs):
            O.mla_forward(ocfg, w, hs[b], int(lens[b]), caches[b], causal=causal, want_trace=False)
        passes += 1
        dt = time.perf_counter() - t0
        if dt >= target_s or passes >= 50:
            break
    rows = int(sum(lens[:n_seqs]))
    return (passes * n_seqs * q_len / dt, O.threads(ocfg), dt,
            f"{n_seqs} of the workload's sequences ({rows} cached rows), full layer, {passes} passes")


def run_reference(a):
    """Reference arm: the CPU statement of the reference's MLA math (the reference's own code for
    this path only runs on an XDNA2 NPU), all host threads, on a bounded sample per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from fastar_b200 import mla
    batch, q_len, lo, hi, causal, desc = workload_shape(a)
    cfg = mla.make_config(mla.PRESET_BASELINE)
    lens = make_inputs(cfg, a, 0, batch, q_len, lo, hi)
    n_seqs = min(a.cpu_seqs, batch)
    if a.workload in ("verify", "longctx"):
        n_seqs = 1
    vals = []
    steps = max(1, min(a.steps, 3))
    for _ in range(max(0, min(a.warmup, 1))):
        cpu_sample(cfg, a, lens, q_len, causal, n_seqs, target_s=1.0)
    for _ in range(steps):
        v, cores, dt, sample = cpu_sample(cfg, a, lens, q_len, causal, n_seqs, target_s=5.0)
        vals.append(v)
    v = statistics.median(vals)
    line = {"impl": "reference", "metric": "mla_decode_layer_tokens_per_s", "value": v, "unit": "layer-tokens/s",
            "n_gpus": a.gpus, "steps": steps, "warmup": min(a.warmup, 1), "ms_per_step": 1e3 * n_seqs * q_len / v,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": desc, "batch_per_gpu": batch, "q_len": q_len, "ctx": [lo, hi]},
            "cpu_baseline": {"value": v, "unit": "layer-tokens/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": v, "unit": "layer-tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def main():
    a = parse()
    if a.impl == "reference":
        return run_reference(a)

    import torch
    from fastar_b200 import mla, synth, parallel

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a GPU: the MLA path has no CPU fallback")
    torch.cuda.set_device(local)
    dist = None
    if world > 1 or a.workload == "longctx":
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29531")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
    batch, q_len, lo, hi, causal, desc = workload_shape(a)
    T = batch * q_len
    longctx = a.workload == "longctx"

    lens = make_inputs(None, a, 0 if longctx else rank, batch, q_len, lo, hi)
    if longctx:
        sl = parallel.kv_slices(int(lens[0]), world)
        my_rows = [sl[rank][1] - sl[rank][0]]
    else:
        my_rows = [int(x) for x in lens]
    n_pages = sum((r + q_len + 63) // 64 for r in my_rows) + 16
    cfg = mla.make_config(mla.PRESET_BASELINE, n_pages=n_pages, max_tokens=T, max_seqs=batch + 8, device=local,
                          attn_impl=a.attn_impl, gemm_impl=a.gemm_impl)
    ctx = mla.MlaContext(cfg)
    ctx.set_stream(torch.cuda.current_stream().cuda_stream)
    if a.merge_kernel:
        ctx.set_fused_merge(False)
    ctx.set_layer_weights(0, synth.weights_to_bits(synth.layer_weights_f32(cfg, a.seed, 0)))
    # scramble the free list so that the block tables are a random page permutation
    rng = synth.rng_for(a.seed, "perm", rank)
    tmp = [ctx.seq_alloc() for _ in range(8)]
    for s in tmp:
        ctx.seq_reserve(s, 64 * (n_pages // 8))
    for s in rng.permutation(tmp):
        ctx.seq_free(int(s))
    seqs = []
    for b, rows in enumerate(my_rows):
        s = ctx.seq_alloc()
        seq_index = b if not longctx else 0
        if longctx:
            full = synth.cache_rows_f32(cfg, a.seed, 0, int(lens[0]))[sl[rank][0]:sl[rank][1]]
        else:
            full = synth.cache_rows_f32(cfg, a.seed, seq_index + 1000 * rank, rows)
        ctx.cache_write(0, s, 0, synth.to_bf16_bits(full))
        seqs.append(s)
    del full

    h_host = torch.from_numpy(synth.to_bf16_bits(synth.hidden_f32(cfg, a.seed, T, (rank,))).view(np.int16)).pin_memory()
    out_host = torch.empty_like(h_host).pin_memory()
    h_np, out_np = h_host.numpy().view(np.uint16), out_host.numpy().view(np.uint16)
    d_h = h_host.cuda()
    d_out = torch.empty_like(d_h)
    seq_arr = np.array(seqs, np.int32)
    pos_arr = np.array(my_rows, np.int32)
    qlen_arr = np.full(len(seqs), q_len, np.int32)

    if longctx:
        layer = parallel.SplitKvLayer(ctx, seqs[0], sl[rank][0], my_rows[0])
        owner = parallel.owner_of_row(int(lens[0]), int(lens[0]), world)
        layer.plan(int(lens[0]), q_len, rank == owner)

        def step_device():
            layer.run(0, d_h.data_ptr(), d_out.data_ptr())

        def step_e2e():
            layer.plan(int(lens[0]), q_len, rank == owner)
            d_h.copy_(h_host, non_blocking=True)
            layer.run(0, d_h.data_ptr(), d_out.data_ptr())
            out_host.copy_(d_out, non_blocking=True)
            ctx.sync()
    else:
        ctx.plan([(s, p, q_len) for s, p in zip(seqs, my_rows)], causal=causal)

        def step_device():
            ctx.run_device(0, d_h.data_ptr(), d_out.data_ptr())

        # the C call with its pointers converted once, as a C or C++ host would make it
        step_e2e = ctx.bind_forward(0, h_np, out_np, seq_arr, pos_arr, qlen_arr, causal)

    info = ctx.plan_info()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if dist is None:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def sum_over_ranks(x: float) -> float:
        if dist is None:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())

    # ---- device-resident timing: `value` ----
    for _ in range(max(a.warmup, 3)):
        step_device()
    ctx.sync()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)  # nvidia-smi needs a moment to deliver its first sample
    n0 = ctx.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for _ in range(a.steps):
        step_device()
    ev1.record()
    barrier()
    ms = max_over_ranks(ev0.elapsed_time(ev1))
    launches = ctx.launch_count() - n0
    # per-kernel device times: the same K steps once more with a CUDA event between every two
    # kernels on the context's stream (kept out of the timed region above, where events between
    # the kernels would undo the overlap of one kernel's prologue with its predecessor's tail)
    ctx.set_profiling(True)
    ctx.kernel_times()  # clear
    for _ in range(a.steps):
        step_device()
    ktimes = ctx.kernel_times()
    ctx.set_profiling(False)
    # nvidia-smi samples every 100 ms: when the timed region was shorter than that allows, keep
    # the same steps running (untimed) under the sampler so that the clocks are read under load
    replay_s = 0.0
    if ms < 700.0:
        t_r = time.perf_counter()
        while time.perf_counter() - t_r < 0.8:
            for _ in range(20):
                step_device()
            ctx.sync()
        replay_s = time.perf_counter() - t_r
    clocks = sampler.stop() if rank == 0 else None
    if clocks is not None:
        clocks["sampled_over"] = "timed region" if replay_s == 0 else f"timed region + {replay_s:.1f} s untimed replay of the same steps"
    ctx.sync()

    # ---- end-to-end through the host-buffer entry point: `e2e` ----
    # Every call builds and uploads its plan (what the first layer of a model step pays); the same
    # loop with the plan kept, as layers 2 .. L of a step see it, is reported beside it.
    def time_e2e():
        for _ in range(3):
            step_e2e()
        barrier()
        t0 = time.perf_counter()
        for _ in range(a.steps):
            step_e2e()
        barrier()
        return max_over_ranks(time.perf_counter() - t0)

    ctx.set_plan_reuse(False)
    e2e_s = time_e2e()
    ctx.set_plan_reuse(True)
    e2e_kept_s = time_e2e()

    tokens_per_step = sum_over_ranks(float(T)) if not longctx else float(T)
    value = tokens_per_step * a.steps / (ms * 1e-3)
    e2e = tokens_per_step * a.steps / e2e_s
    attn_ms, attn_n = ktimes["attn"]
    merge_ms, _ = ktimes["merge"]
    peak, peak_kind = hbm_peak()
    kv_bytes = ROW_BYTES * info["kv_rows"]
    achieved = kv_bytes / (attn_ms / max(attn_n, 1) * 1e-3) / 1e9 if attn_n else None
    achieved_with_merge = kv_bytes / ((attn_ms + merge_ms) / max(attn_n, 1) * 1e-3) / 1e9 if attn_n else None
    tr = ncu_traffic(a.workload)
    traffic = tr["dram_bytes_per_cached_row"] * info["kv_rows"] if tr else None

    if rank == 0:
        line = {
            "metric": "mla_decode_layer_tokens_per_s", "value": value, "unit": "layer-tokens/s", "n_gpus": world,
            "steps": a.steps, "warmup": max(a.warmup, 3), "ms_per_step": ms / a.steps, "higher_is_better": True,
            "scaling": "strong" if longctx else "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": desc, "batch_per_gpu": batch, "q_len": q_len, "ctx": [lo, hi],
                       "cached_rows_rank0": info["kv_rows"], "page_tokens": 64, "preset": "baseline",
                       "l2": "inputs larger than L2 (cache + weights read per step exceed 126 MB)"
                             if kv_bytes + 122e6 > 126e6 else "inputs smaller than L2; no flush",
                       "attn_ctas": info["n_ctas"], "attn_partials": info["n_partials"],
                       "value_excludes": "per-step plan upload (amortised over the layers of a step)",
                       "kernel_events": "second pass of the same steps, one CUDA event between kernels"},
            "e2e": {"value": e2e, "unit": "layer-tokens/s", "h2d_bytes_per_step": int(h_host.numel() * 2),
                    "d2h_bytes_per_step": int(out_host.numel() * 2), "plan": "built and uploaded in every call",
                    "value_with_plan_kept": tokens_per_step * a.steps / e2e_kept_s},
            "gpu_launches": int(launches),
            "roofline": {"bound": "hbm", "kernel": "k_attn_stream (split-KV latent attention)", "achieved": achieved,
                         "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                         "frac": achieved / peak if achieved else None, "traffic": traffic,
                         "algorithmic_bytes_per_launch": kv_bytes, "launch_ms": attn_ms / max(attn_n, 1),
                         "with_merge_GBs": achieved_with_merge, "frac_of_nominal_8TBs": achieved / 8000.0 if achieved else None},
            "kernel_ms": {k: (v[0] / v[1] if v[1] else None) for k, v in ktimes.items()},
            "clocks": clocks,
        }
        if world == 1 and not a.no_cpu_baseline:
            n = 1 if a.workload in ("verify", "longctx") else a.cpu_seqs
            v, cores, dt, sample = cpu_sample(cfg, a, lens, q_len, causal, n)
            line["cpu_baseline"] = {"value": v, "unit": "layer-tokens/s", "cores": cores, "kind": "port",
                                    "sample": sample, "seconds": dt}
        print(json.dumps(line), flush=True)
    ctx.close()
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
