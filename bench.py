#!/usr/bin/env python3
"""MLA decode benchmark: layer-tokens/s of one Multi-head Latent Attention layer call, with the
roofline of the latent-cache read and a host-CPU baseline beside it.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload batched|single|verify|longctx]
    python bench.py --impl reference ...      # the CPU statement of the reference math, timed

A step is one layer call (q compress/expand, kv compress + append, split-KV attention over the
paged latent cache, both output projections) for every sequence of the batch.  Default
workload: batched decode, batch 64, context lengths uniform in [1024, 8192], 64-token pages with
a scrambled block table, bf16 with fp32 accumulation, synthetic seeded inputs.

Under torchrun (one rank per GPU) the headline `value` is weak scaling -- every rank has its own
batch of 64 and there is no data-path collective -- and the same line carries two more
measurements of the multi-GPU forms of the path:
  strong   ONE batch of 64 split over the ranks by cached rows (no collective inside the layer)
  longctx  one 131072-token sequence split along the KV axis; every rank attends to its slice and
           the per-GPU partials are exchanged by ONE NCCL all-gather inside the C ABI
           (fst_cuda_mla_run_split_device), timed as a whole and for the exchange alone
`--workload longctx` makes the second one the headline instead.  Prints ONE JSON line on rank 0.

Timing: W untimed warm-up steps, then regions of exactly K steps, each bracketed by a barrier and
a device synchronisation, timed with CUDA events on the launching stream, maximum over ranks;
regions are repeated until about 0.25 s has been timed and the MEDIAN region is reported
(`config.timed_regions` says how many).
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
sys.path.insert(0, ROOT)

ROW_BYTES = 1152  # algorithmic bytes per cached token attended: 576 bf16, read once
METRIC = "mla_decode_layer_tokens_per_s"
UNIT = "layer-tokens/s"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="batched", choices=["batched", "single", "verify", "longctx"])
    ap.add_argument("--batch", type=int, default=0, help="sequences (default: the workload's)")
    ap.add_argument("--ctx-lo", type=int, default=0)
    ap.add_argument("--ctx-hi", type=int, default=0)
    ap.add_argument("--attn-impl", type=int, default=0)
    ap.add_argument("--gemm-impl", type=int, default=0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--cpu-seqs", type=int, default=8, help="sequences in the bounded CPU-baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the strong-scaling and long-context measurements")
    ap.add_argument("--merge-kernel", action="store_true", help="every token through its partial and the merge kernel")
    ap.add_argument("--preset", default="baseline", choices=["baseline", "v4"],
                    help="v4: the live engine's layer form (512-wide rows, head norm, sink, inverse RoPE, grouped wo_a, "
                         "214 MB of weights); GPU figures only (its parity is the tests'), no CPU legs")
    ap.add_argument("--token-schedule", action="store_true",
                    help="multi-token calls keep the token-by-token split-KV schedule (no groups of lanes sharing pages)")
    ap.add_argument("--min-timed-s", type=float, default=0.25)
    ap.add_argument("--sequential-pages", action="store_true",
                    help="leave the page pool in order (block tables ascend) instead of scrambling it")
    return ap.parse_args()


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


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            d = json.load(open(p))
            return float(d["hbm_gbs"]), float(d.get("bf16_tflops_sustained", 1399.5)), "measured"
        except Exception:
            pass
    return 6650.0, 1400.0, "fallback"


def ncu_traffic():
    """DRAM bytes per cached row of the attention kernel from the committed ncu capture
    (profiles/attn_traffic.json); the bench scales it by the rows of its own launch."""
    p = os.path.join(ROOT, "profiles", "attn_traffic.json")
    try:
        return json.load(open(p))
    except Exception:
        return None


def verify_traffic():
    """DRAM bytes per row of a SEQUENCE for the attention kernel on blocks of 16 query tokens, from
    the committed ncu capture at 8 sequences (profiles/verify_traffic.json)."""
    try:
        return json.load(open(os.path.join(ROOT, "profiles", "verify_traffic.json")))
    except Exception:
        return None


def config_dict(a, desc, batch, q_len, lo, hi):
    """What both arms print as `config`: the workload, nothing that differs between the arms."""
    return {"workload": desc, "batch": batch, "q_len": q_len, "ctx": [lo, hi], "page_tokens": 64, "preset": a.preset,
            "seed": a.seed}


# ------------------------------------------------------------------------------------------------
# CPU side: the oracle as the timed baseline and as the checker of one step's output
# ------------------------------------------------------------------------------------------------
class CpuWorkload:
    """The first n_seqs sequences of a workload for the CPU oracle (fp32 arrays of bf16 values)."""

    def __init__(self, a, name, n_seqs=None, rank=0):
        from fastar_b200 import mla, synth, workloads
        from oracle import oracle as O
        self.O = O
        batch, q_len, lo, hi, causal, desc = workloads.shape(name, a.batch, a.ctx_lo, a.ctx_hi)
        self.cfg = mla.make_config(mla.PRESET_BASELINE)
        self.ocfg = O.make_cfg(O.PRESET_BASELINE)
        lens = synth.context_lengths(a.seed, batch, lo, hi, (rank,))
        n = batch if n_seqs is None else min(n_seqs, batch)
        self.n, self.q_len, self.causal, self.batch = n, q_len, causal, batch
        self.lens = [int(x) for x in lens[:n]]
        self.w = synth.weights_rounded(synth.layer_weights_f32(self.cfg, a.seed, 0))
        row = mla.dims_of(self.cfg)["row"]
        self.caches = []
        for b in range(n):
            c = np.zeros((self.lens[b] + q_len, row), np.float32)
            key = b + 1000 * rank if name != "longctx" else 0
            c[:self.lens[b]] = synth.from_bf16_bits(synth.to_bf16_bits(synth.cache_rows_f32(self.cfg, a.seed, key, self.lens[b])))
            self.caches.append(c)
        h = synth.hidden_f32(self.cfg, a.seed, batch * q_len, (rank,))
        self.h = synth.from_bf16_bits(synth.to_bf16_bits(h[:n * q_len]))
        self.sample = (f"all {batch} sequences" if n == batch else f"the first {n} of {batch} sequences") + \
                      f" ({sum(self.lens)} cached rows), full layer, projections batched over the sample's rows"

    def step(self):
        """One layer call for the whole sample (projections as one product over all its rows)."""
        return self.O.mla_forward_batch(self.ocfg, self.w, self.h, [self.q_len] * self.n, self.lens, self.caches,
                                        causal=self.causal).out

    def cores(self):
        return self.O.threads(self.ocfg)


def reference_sample_size(name, batch):
    """Sequences per step of the CPU arm: the whole batch where a step stays around a second,
    a bounded sample for the verify block (0.5 s per sequence)."""
    return {"batched": batch, "single": batch, "longctx": batch, "verify": min(batch, 2)}[name]


def run_reference(a):
    """Reference arm.  The reference's own code for this path runs only on an XDNA2 NPU (every GEMM
    of process_mla is an NPU dispatch), so this times the CPU statement of its math -- the oracle --
    with all host threads: W warm-up steps, then K steps, each one layer call over the sample."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    from fastar_b200 import workloads
    batch, q_len, lo, hi, causal, desc = workloads.shape(a.workload, a.batch, a.ctx_lo, a.ctx_hi)
    cw = CpuWorkload(a, a.workload, reference_sample_size(a.workload, batch))
    for _ in range(a.warmup):
        cw.step()
    t0 = time.perf_counter()
    for _ in range(a.steps):
        cw.step()
    dt = time.perf_counter() - t0
    tokens = cw.n * q_len
    v = tokens * a.steps / dt
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": a.gpus, "steps": a.steps,
            "warmup": a.warmup, "ms_per_step": 1e3 * dt / a.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": config_dict(a, desc, batch, q_len, lo, hi),
            "cpu_baseline": {"value": v, "unit": UNIT, "cores": cw.cores(), "kind": "port", "sample": cw.sample,
                             "seconds": dt},
            "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# GPU side
# ------------------------------------------------------------------------------------------------
class Timer:
    """Regions of exactly K steps, bracketed by barrier + synchronise, CUDA events on the current
    stream, maximum over ranks per region; regions repeat until min_s has been timed."""

    def __init__(self, torch, dist, steps, warmup, min_s):
        self.torch, self.dist, self.K, self.W, self.min_s = torch, dist, steps, max(warmup, 3), min_s

    def barrier(self):
        if self.dist is not None:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def reduce(self, x: float, op="max") -> float:
        if self.dist is None:
            return x
        t = self.torch.tensor([x], dtype=self.torch.float64, device="cuda")
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX if op == "max" else self.dist.ReduceOp.SUM)
        return float(t.item())

    def device(self, step):
        """Median region time (ms) of a step that only enqueues work; (ms, regions)."""
        torch = self.torch
        for _ in range(self.W):
            step()
        regions, total = [], 0.0
        while True:
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self.barrier()
            ev0.record()
            for _ in range(self.K):
                step()
            ev1.record()
            self.barrier()
            ms = self.reduce(ev0.elapsed_time(ev1))
            regions.append(ms)
            total += ms
            if (total >= 1e3 * self.min_s and len(regions) >= 3) or len(regions) >= 400:
                break
        return statistics.median(regions), len(regions)

    def host(self, step):
        """The same for a step that synchronises by itself (wall clock around K calls)."""
        for _ in range(3):
            step()
        regions, total = [], 0.0
        while True:
            self.barrier()
            t0 = time.perf_counter()
            for _ in range(self.K):
                step()
            dt = time.perf_counter() - t0
            self.barrier()
            dt = self.reduce(dt)
            regions.append(dt * 1e3)
            total += dt
            if (total >= self.min_s and len(regions) >= 3) or len(regions) >= 400:
                break
        return statistics.median(regions), len(regions)


def kernel_times(ctx, step, steps):
    """Per-kernel device times: the same steps once more with a CUDA event between every two
    kernels on the context's stream (kept out of the timed regions, where events between the
    kernels would undo the overlap of one kernel's prologue with its predecessor's tail)."""
    ctx.set_profiling(True)
    ctx.kernel_times()
    for _ in range(steps):
        step()
    k = ctx.kernel_times()
    ctx.set_profiling(False)
    return {name: (v[0] / v[1] if v[1] else None) for name, v in k.items()}


def measure_longctx(a, torch, dist, timer, rank, world, local):
    """One 131072-token sequence split along the KV axis over the ranks; the exchange is the NCCL
    all-gather inside fst_cuda_mla_run_split_device."""
    from fastar_b200 import mla, parallel, workloads
    wl = workloads.build("longctx", seed=a.seed, rank=rank, world=world, device=local, attn_impl=a.attn_impl,
                         gemm_impl=a.gemm_impl, stream=torch.cuda.current_stream().cuda_stream,
                         ctx_lo=a.ctx_lo if a.workload == "longctx" else 0, ctx_hi=a.ctx_hi if a.workload == "longctx" else 0)
    ctx = wl.ctx
    L = int(wl.all_lens[0])
    owner = parallel.owner_of_row(L, L, world)
    s = wl.seqs[0]
    step_desc = (s, L - wl.slice_begin, 1, L, 1) if rank == owner else (s, wl.rows[0], 1, L, 0)
    ctx.plan([step_desc])
    d_h = torch.from_numpy(wl.h_bits.view(np.int16)).cuda()
    d_out = torch.empty_like(d_h)
    if world > 1:
        uid = [mla.comm_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(uid, src=0)
        ctx.comm_init(uid[0], rank, world)

        def step():
            ctx.run_split_device(0, d_h.data_ptr(), d_out.data_ptr())
    else:
        def step():
            ctx.run_device(0, d_h.data_ptr(), d_out.data_ptr())
    ms, regions = timer.device(step)
    kt = kernel_times(ctx, step, a.steps)
    info = ctx.plan_info()
    res = {"workload": wl.desc, "rows": L, "rows_this_rank": wl.rows[0], "ms_per_step": ms / a.steps,
           "layer_tokens_per_s": a.steps / (ms * 1e-3), "timed_regions": regions,
           "attn_us": 1e3 * kt["attn"] if kt["attn"] else None,
           "exchange_us": (1e3 * kt["exchange"] if kt.get("exchange") else None) if world > 1 else 0.0,
           "exchange_bytes_per_rank": 64 * 514 * 4 if world > 1 else 0,
           "exchange": "ncclAllGather inside fst_cuda_mla_run_split_device" if world > 1 else "none (one GPU)",
           "cache_GBs_this_rank": ROW_BYTES * info["kv_rows"] / (kt["attn"] * 1e-3) / 1e9 if kt["attn"] else None,
           "kernel_ms": kt}
    if world > 1:
        ctx.comm_destroy()
    wl.close()
    return res


def measure_noalloc(torch, rows=65536, calls=10):
    """fst_cuda_mla_attention_noalloc (decode attention without a context or any allocation, CUDA-core
    kernels, at most 31 splits: its scratch is a fixed 4 MiB array) at its largest size: us per call."""
    from fastar_b200 import mla
    g = torch.Generator(device="cuda").manual_seed(0)
    cache = torch.randn((rows, 576), generator=g, device="cuda").to(torch.bfloat16)
    q = torch.randn((64, 576), generator=g, device="cuda").to(torch.bfloat16)
    out = torch.zeros((64, 512), dtype=torch.bfloat16, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    call = lambda: mla.attention_noalloc(q.data_ptr(), cache.data_ptr(), rows, 64, 576, 512, 1.0 / math.sqrt(192.0),  # noqa: E731
                                         out.data_ptr(), st)
    for _ in range(2):
        if call():
            return {"error": mla.load_library().fst_cuda_mla_last_error().decode()}
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    ev0.record()
    for _ in range(calls):
        call()
    ev1.record()
    torch.cuda.synchronize()
    us = 1e3 * ev0.elapsed_time(ev1) / calls
    return {"what": "fst_cuda_mla_attention_noalloc, one query token over 65536 contiguous rows", "rows": rows,
            "us_per_call": us, "cache_GBs": rows * ROW_BYTES / (us * 1e-6) / 1e9, "finite": bool(torch.isfinite(out.float()).all())}


def measure_batch(a, torch, dist, timer, rank, world, local, sharding, with_e2e, with_clocks):
    """Batched workloads (batched / single / verify), replicated per rank or one batch sharded."""
    from fastar_b200 import mla, workloads
    wl = workloads.build(a.workload if a.workload != "longctx" else "batched", seed=a.seed, rank=rank, world=world,
                         sharding=sharding, device=local, batch=a.batch, ctx_lo=a.ctx_lo, ctx_hi=a.ctx_hi,
                         attn_impl=a.attn_impl, gemm_impl=a.gemm_impl, stream=torch.cuda.current_stream().cuda_stream,
                         scramble=not a.sequential_pages,
                         preset=mla.PRESET_FASTAR_V4 if a.preset == "v4" else mla.PRESET_BASELINE)
    ctx = wl.ctx
    if a.merge_kernel:
        ctx.set_fused_merge(False)
    if a.token_schedule:
        ctx.set_block_schedule(False)
    T = wl.T
    h_host = torch.from_numpy(wl.h_bits.view(np.int16)).pin_memory()
    out_host = torch.empty_like(h_host).pin_memory()
    h_np, out_np = h_host.numpy().view(np.uint16), out_host.numpy().view(np.uint16)
    d_h = h_host.cuda()
    d_out = torch.empty_like(d_h)
    seq_arr = np.array(wl.seqs, np.int32)
    pos_arr = np.array(wl.rows, np.int32)
    qlen_arr = np.full(len(wl.seqs), wl.q_len, np.int32)
    ctx.plan(wl.steps(), causal=wl.causal)
    info = ctx.plan_info() if T else {"kv_rows": 0, "n_ctas": 0, "n_partials": 0}

    def step_device():
        ctx.run_device(0, d_h.data_ptr(), d_out.data_ptr())

    sampler = ClockSampler(local)
    if with_clocks and rank == 0:
        sampler.start()
        time.sleep(0.25)  # nvidia-smi needs a moment to deliver its first sample
    n0 = ctx.launch_count()
    ms, regions = timer.device(step_device)
    launches_per_step = (ctx.launch_count() - n0) / float(regions * a.steps + timer.W)
    kt = kernel_times(ctx, step_device, a.steps)
    clocks = None
    if with_clocks:
        # nvidia-smi samples every 100 ms: keep the same steps running (untimed) under the sampler
        # until it has seen about a second under load
        t_r = time.perf_counter()
        while time.perf_counter() - t_r < 0.8:
            for _ in range(20):
                step_device()
            ctx.sync()
        if rank == 0:
            clocks = sampler.stop()
            clocks["sampled_over"] = "timed regions + 0.8 s untimed replay of the same steps"
    ctx.sync()
    tokens_all = timer.reduce(float(T), "sum")
    res = {"wl": wl, "ms": ms, "regions": regions, "kernel_ms": kt, "info": info, "clocks": clocks,
           "value": tokens_all * a.steps / (ms * 1e-3), "launches_per_step": launches_per_step,
           "rows_all": timer.reduce(float(sum(wl.rows)), "sum"), "rows_max": timer.reduce(float(sum(wl.rows)), "max"),
           "family": ctx.family_counts()}
    if with_e2e:
        # end to end through the host-buffer entry point, as a C or C++ host calls it (pointers
        # converted once); every call builds and uploads its plan.  Page-locked buffers first,
        # then pageable ones (the reference engine's own buffers are pageable vectors).
        step_e2e = ctx.bind_forward(0, h_np, out_np, seq_arr, pos_arr, qlen_arr, wl.causal)
        ctx.set_plan_reuse(False)
        e_ms, e_regions = timer.host(step_e2e)
        ctx.set_plan_reuse(True)
        k_ms, _ = timer.host(step_e2e)
        ctx.set_plan_reuse(False)
        h_pg, out_pg = wl.h_bits.copy(), np.empty_like(wl.h_bits)
        p_ms, _ = timer.host(ctx.bind_forward(0, h_pg, out_pg, seq_arr, pos_arr, qlen_arr, wl.causal))
        ctx.set_plan_reuse(True)
        res["e2e"] = {"value": tokens_all * a.steps / (e_ms * 1e-3), "unit": UNIT,
                      "h2d_bytes_per_step": int(h_host.numel() * 2), "d2h_bytes_per_step": int(out_host.numel() * 2),
                      "buffers": "page-locked host buffers (the last GEMM writes the caller's buffer)",
                      "plan": "built and uploaded in every call", "timed_regions": e_regions,
                      "value_with_plan_kept": tokens_all * a.steps / (k_ms * 1e-3),
                      "value_pageable_buffers": tokens_all * a.steps / (p_ms * 1e-3)}
        res["out_bits"] = out_np.copy()
    return res


def parity_of(a, wl, out_bits):
    """One step's output rows (through fst_cuda_mla_forward) against the oracle, for the sequences of
    the CPU sample: {cosine, max_abs}."""
    from fastar_b200 import synth
    n = min(a.cpu_seqs if a.workload != "verify" else 2, len(wl.seqs))
    cw = CpuWorkload(a, a.workload, n, rank=0)
    want = cw.step()
    got = synth.from_bf16_bits(out_bits[:n * wl.q_len])
    cos = float((got.ravel().astype(np.float64) @ want.ravel().astype(np.float64)) /
                (np.linalg.norm(got.astype(np.float64)) * np.linalg.norm(want.astype(np.float64)) + 1e-300))
    return {"cosine": cos, "max_abs": float(np.max(np.abs(got - want))), "sequences": n,
            "bar": "cosine >= 0.9999 and max_abs <= 2e-2", "ok": bool(cos >= 0.9999 and np.max(np.abs(got - want)) <= 2e-2)}, cw


def main():
    a = parse()
    if a.impl == "reference":
        return run_reference(a)

    import torch
    from fastar_b200 import workloads

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a GPU: the MLA path has no CPU fallback")
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29531")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
    timer = Timer(torch, dist, a.steps, a.warmup, a.min_timed_s)
    batch, q_len, lo, hi, causal, desc = workloads.shape(a.workload, a.batch, a.ctx_lo, a.ctx_hi)
    hbm, tensor_peak, peak_kind = peaks()

    if a.workload == "longctx":
        lc = measure_longctx(a, torch, dist, timer, rank, world, local)
        if rank == 0:
            line = {"metric": METRIC, "value": lc["layer_tokens_per_s"], "unit": UNIT, "n_gpus": world, "steps": a.steps,
                    "warmup": timer.W, "ms_per_step": lc["ms_per_step"], "higher_is_better": True, "scaling": "strong",
                    "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                    "config": config_dict(a, desc, batch, q_len, lo, hi),
                    "longctx": lc, "gpu_launches": None,
                    "roofline": {"bound": "hbm (latency-bound at this size: 151 MB of cache against 122 MB of weights and a "
                                          "131.6 KB exchange)", "achieved": lc["cache_GBs_this_rank"], "peak": hbm,
                                 "peak_kind": peak_kind, "unit": "GB/s",
                                 "frac": lc["cache_GBs_this_rank"] / hbm if lc["cache_GBs_this_rank"] else None,
                                 "traffic": None}}
            print(json.dumps(line), flush=True)
        if dist is not None:
            dist.destroy_process_group()
        return

    main_res = measure_batch(a, torch, dist, timer, rank, world, local, "replica", True, True)
    wl = main_res["wl"]
    extras = {}
    if not a.no_extras and a.workload == "batched" and a.preset == "baseline":
        if world > 1:
            st = measure_batch(a, torch, dist, timer, rank, world, local, "strong", False, False)
            st["wl"].close()
        else:
            st = main_res  # one GPU: the sharded batch IS the headline batch
        extras["strong"] = {"what": f"ONE batch of {batch} sequences split over {world} GPU(s) by cached rows, no collective",
                            "layer_tokens_per_s": st["value"], "ms_per_step": st["ms"] / a.steps,
                            "rows_total": int(st["rows_all"]), "rows_max_rank": int(st["rows_max"]),
                            "imbalance": st["rows_max"] * world / max(st["rows_all"], 1.0),
                            "attn_us_rank0": 1e3 * st["kernel_ms"]["attn"] if st["kernel_ms"]["attn"] else None}
        extras["longctx"] = measure_longctx(a, torch, dist, timer, rank, world, local)
        if world == 1:
            extras["noalloc"] = measure_noalloc(torch)

    if rank == 0:
        kt, info = main_res["kernel_ms"], main_res["info"]
        row_bytes = 1024 if a.preset == "v4" else ROW_BYTES
        kv_bytes = row_bytes * info["kv_rows"]
        attn_ms, merge_ms = kt["attn"] or 0.0, kt["merge"] or 0.0
        ach_attn = kv_bytes / (attn_ms * 1e-3) / 1e9 if attn_ms else None
        ach_both = kv_bytes / ((attn_ms + merge_ms) * 1e-3) / 1e9 if attn_ms else None
        tr = ncu_traffic()
        flops = 2.0 * 64 * ((512 if a.preset == "v4" else 576) + 512) * info["kv_rows"]
        cfg = config_dict(a, desc, batch, q_len, lo, hi)
        run = {}
        run.update({"cached_rows_rank0": info["kv_rows"], "attn_ctas": info["n_ctas"], "attn_partials": info["n_partials"],
                    "timed_regions": main_res["regions"], "timed_ms_total": main_res["ms"] * main_res["regions"],
                    "l2": "inputs larger than L2 (cache + weights read per step exceed 126 MB)"
                          if kv_bytes + 122e6 > 126e6 else "inputs smaller than L2; no flush",
                    "value_excludes": "per-step plan upload (amortised over the layers of a model step)",
                    "kernel_events": "separate pass of the same steps, one CUDA event between kernels",
                    "kernel_families": main_res["family"]})
        line = {"metric": METRIC, "value": main_res["value"], "unit": UNIT, "n_gpus": world, "steps": a.steps,
                "warmup": timer.W, "ms_per_step": main_res["ms"] / a.steps, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": cfg, "run": run, "e2e": main_res["e2e"],
                "gpu_launches": int(round(main_res["launches_per_step"] * a.steps)),
                "roofline": {"bound": "hbm", "kernel": "k_attn_stream + merge (split-KV latent attention and the merge of its partials)",
                             "achieved": ach_both, "peak": hbm, "peak_kind": peak_kind, "unit": "GB/s",
                             "frac": ach_both / hbm if ach_both else None,
                             "traffic": tr["dram_bytes_per_cached_row"] * info["kv_rows"] if tr else None,
                             "algorithmic_bytes_per_launch": kv_bytes, "launch_ms": attn_ms + merge_ms,
                             "attention_kernel_alone": {"achieved": ach_attn, "frac": ach_attn / hbm if ach_attn else None,
                                                        "launch_ms": attn_ms},
                             "frac_of_nominal_8TBs": ach_both / 8000.0 if ach_both else None,
                             "tensor": {"achieved_TFLOPs": flops / (attn_ms * 1e-3) / 1e12 if attn_ms else None,
                                        "peak_TFLOPs": tensor_peak,
                                        "frac": flops / (attn_ms * 1e-3) / 1e12 / tensor_peak if attn_ms else None}},
                "kernel_ms": kt, "clocks": main_res["clocks"]}
        if q_len > 1:
            # blocks of query tokens: the tensor cores bound the path (139 264 flop per visible row and
            # token); under the block schedule a cache page is read once per SEQUENCE, so the cache
            # bytes of a launch are those of the sequences' rows, not of every token's
            seq_rows = sum(int(r) + q_len for r in wl.rows)
            v8 = verify_traffic()
            tfl = flops / (attn_ms * 1e-3) / 1e12 if attn_ms else None
            line["roofline"] = {"bound": "tensor", "kernel": "k_attn_stream (M = 64 MMAs: half the dense rate)",
                                "achieved": tfl, "peak": tensor_peak, "peak_kind": peak_kind + ", sustained bf16 GEMM",
                                "unit": "TFLOP/s", "frac": tfl / tensor_peak if tfl else None,
                                "flops_per_launch": flops, "launch_ms": attn_ms,
                                "cache_bytes_per_launch": ROW_BYTES * seq_rows,
                                "cache_bytes_if_every_token_read_its_own": kv_bytes,
                                "traffic": v8["dram_bytes_per_sequence_row"] * seq_rows if v8 else None,
                                "cache_GBs": ROW_BYTES * seq_rows / (attn_ms * 1e-3) / 1e9 if attn_ms else None,
                                "schedule": "tokens" if a.token_schedule else "blocks"}
        line.update(extras)
        if world == 1 and not a.no_cpu_baseline and a.preset == "baseline":
            par, cw = parity_of(a, wl, main_res["out_bits"])
            line["parity"] = par
            t0, passes = time.perf_counter(), 0
            while True:
                cw.step()
                passes += 1
                dt = time.perf_counter() - t0
                if dt >= 10.0 or passes >= 200:
                    break
            line["cpu_baseline"] = {"value": passes * cw.n * cw.q_len / dt, "unit": UNIT, "cores": cw.cores(), "kind": "port",
                                    "sample": cw.sample + f", {passes} passes", "seconds": dt}
        print(json.dumps(line), flush=True)
    wl.close()
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
