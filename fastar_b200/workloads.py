"""The benchmark configurations as seeded synthetic workloads, built the same way by bench.py
and by the full-size parity tests: a context with weights, a scrambled page pool, every
sequence's cache written, the input rows of one step.

Named workloads (BASELINE preset shapes, 64-token pages):
  single   decode at batch 1 over a 4096-token cache
  batched  batch 64, context lengths uniform in [1024, 8192], scrambled block table
  verify   speculative-verify block: 16 causal query tokens x 32 sequences over 16384 rows
  longctx  one 131072-token sequence (split along the KV axis when world > 1)

Sharding of a batch over `world` ranks (one process per GPU, no data-path collective):
  replica  every rank has its own batch of the workload's size (weak scaling)
  strong   ONE batch of the workload's size is split over the ranks by cached rows
           (parallel.shard_sequences); rank r holds only its sequences
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

from . import mla, parallel, synth

SHAPES = {
    # name: (batch, q_len, ctx_lo, ctx_hi, causal, description)
    "batched": (64, 1, 1024, 8192, False,
                "batched decode: batch 64, ctx~U[1024,8192], 64-token pages, scrambled block table"),
    "single": (1, 1, 4096, 4096, False, "decode at batch 1 over a 4096-token cache"),
    "verify": (32, 16, 16384, 16384, True,
               "speculative-verify block: 16 causal query tokens x 32 seqs over 16384-token caches"),
    "longctx": (1, 1, 131072, 131072, False,
                "one 131072-token sequence, split-KV across the GPUs, all-gather of partials"),
}


def shape(name: str, batch: int = 0, ctx_lo: int = 0, ctx_hi: int = 0):
    b, q, lo, hi, causal, desc = SHAPES[name]
    return (batch or b, q, ctx_lo or lo, ctx_hi or hi, causal, desc)


@dataclass
class Workload:
    name: str
    cfg: mla.Config
    ctx: mla.MlaContext
    q_len: int
    causal: bool
    desc: str
    seqs: list            # sequence ids in the context, in batch order
    rows: list            # cached rows of each of them (this rank's slice for longctx)
    keys: list            # synth key of each sequence's cache rows (cache_rows_f32(cfg, seed, key, n))
    global_index: list    # index of each sequence in the whole batch (strong sharding)
    h_bits: np.ndarray    # [T, hidden] bf16 bits: this rank's input rows of one step
    all_lens: np.ndarray  # context lengths of the whole batch this rank's share was cut from
    seed: int = 0
    slice_begin: int = 0  # longctx: first global row of this rank's slice
    extra: dict = field(default_factory=dict)

    @property
    def T(self) -> int:
        return len(self.seqs) * self.q_len

    def steps(self):
        return [(s, r, self.q_len) for s, r in zip(self.seqs, self.rows)]

    def close(self):
        self.ctx.close()


SCRAMBLE_SEQS = 64  # throw-away sequences of scramble_pool (the context needs that many spare slots)


def scramble_pool(ctx: mla.MlaContext, n_pages: int, seed: int, rank: int) -> None:
    """Leave the free list a random permutation of the pages, page by page, so that every block
    table the workload builds afterwards is a random page list.  (The pool hands out the page that
    was freed last: pages are taken by throw-away sequences, a few hundred each, and given back one
    sequence-truncation at a time in a seeded random order: 64 ascending runs shuffled together.)"""
    rng = synth.rng_for(seed, "perm", rank)
    n_tmp = SCRAMBLE_SEQS
    per = n_pages // n_tmp
    tmp = [ctx.seq_alloc() for _ in range(n_tmp)]
    for s in tmp:
        ctx.seq_reserve(s, 64 * per)
    left = [per] * n_tmp
    # a truncation gives back the LAST page of a throw-away sequence: picking the sequence at random
    # every time interleaves the runs into one random order
    order = rng.permutation(np.repeat(np.arange(n_tmp), per))
    for i in order:
        left[i] -= 1
        ctx.seq_truncate(tmp[i], 64 * left[i])
    for s in tmp:
        ctx.seq_free(s)


def build(name: str, *, seed: int = 0, rank: int = 0, world: int = 1, sharding: str = "replica", device: int = 0,
          batch: int = 0, ctx_lo: int = 0, ctx_hi: int = 0, attn_impl: int = mla.IMPL_AUTO,
          gemm_impl: int = mla.IMPL_AUTO, preset: int = mla.PRESET_BASELINE, stream: int | None = None,
          scramble: bool = True) -> Workload:
    B, q_len, lo, hi, causal, desc = shape(name, batch, ctx_lo, ctx_hi)
    longctx = name == "longctx"
    cfg0 = mla.make_config(preset)
    slice_begin = 0
    if longctx:
        all_lens = synth.context_lengths(seed, B, lo, hi, (0,))
        sl = parallel.kv_slices(int(all_lens[0]), world)
        slice_begin = sl[rank][0]
        my_rows, keys, gidx = [sl[rank][1] - sl[rank][0]], [0], [0]
        h_f32 = synth.hidden_f32(cfg0, seed, B * q_len, (0,))
    elif sharding == "strong":
        all_lens = synth.context_lengths(seed, B, lo, hi, (0,))
        gidx = parallel.shard_sequences(all_lens, world)[rank]
        my_rows = [int(all_lens[i]) for i in gidx]
        keys = list(gidx)
        h_all = synth.hidden_f32(cfg0, seed, B * q_len, (0,))
        h_f32 = np.concatenate([h_all[i * q_len:(i + 1) * q_len] for i in gidx]) if gidx else h_all[:0]
    else:
        all_lens = synth.context_lengths(seed, B, lo, hi, (rank,))
        gidx = list(range(B))
        my_rows = [int(x) for x in all_lens]
        keys = [b + 1000 * rank for b in range(B)]
        h_f32 = synth.hidden_f32(cfg0, seed, B * q_len, (rank,))
    n_seq = len(my_rows)
    n_pages = sum((r + q_len + 63) // 64 for r in my_rows) + 16
    cfg = mla.make_config(preset, n_pages=n_pages, max_tokens=max(n_seq * q_len, 1), max_seqs=n_seq + SCRAMBLE_SEQS + 8,
                          device=device, attn_impl=attn_impl, gemm_impl=gemm_impl)
    ctx = mla.MlaContext(cfg)
    if stream is not None:
        ctx.set_stream(stream)
    ctx.set_layer_weights(0, synth.weights_to_bits(synth.layer_weights_f32(cfg, seed, 0)))
    if scramble:
        scramble_pool(ctx, n_pages, seed, rank)
    seqs = []
    for b, rows in enumerate(my_rows):
        s = ctx.seq_alloc()
        if longctx:
            full = synth.cache_rows_f32(cfg, seed, 0, int(all_lens[0]))[slice_begin:slice_begin + rows]
        else:
            full = synth.cache_rows_f32(cfg, seed, keys[b], rows)
        if rows:
            ctx.cache_write(0, s, 0, synth.to_bf16_bits(full))
        seqs.append(s)
    return Workload(name, cfg, ctx, q_len, causal, desc, seqs, my_rows, keys, gidx,
                    synth.to_bf16_bits(h_f32), np.asarray(all_lens), seed, slice_begin)
