"""Multi-GPU forms of the MLA path, one process per GPU (torch.distributed is the plumbing).

* Sequence sharding: batched decode splits by sequence; weights are replicated, every GPU
  owns the pages of its sequences, and there is no collective inside the layer.
* Split-KV: one long sequence is cut along the KV axis into page-aligned slices, one per GPU.
  Every GPU computes the (cheap) query redundantly, attends to its slice, and the per-GPU
  (max, sum, un-normalised O) partials are exchanged with ONE all-gather and merged by
  log-sum-exp on every GPU.  The reference has no counterpart (single NPU, 128 rows).
"""
from __future__ import annotations

import numpy as np


def shard_sequences(lengths, world: int) -> list[list[int]]:
    """Longest-processing-time assignment of sequences to ranks, balancing cached rows.
    Returns, per rank, the (ascending) indices of its sequences."""
    order = sorted(range(len(lengths)), key=lambda i: (-int(lengths[i]), i))
    load = [0] * world
    out = [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda k: (load[k], k))
        out[r].append(i)
        load[r] += int(lengths[i])
    return [sorted(x) for x in out]


def kv_slices(n_rows: int, world: int, page_tokens: int = 64) -> list[tuple[int, int]]:
    """Cut rows [0, n_rows) into `world` contiguous slices whose boundaries are page aligned
    (the last slice takes the ragged end).  Slices may be empty when n_rows is small."""
    n_pages = (n_rows + page_tokens - 1) // page_tokens
    out = []
    for r in range(world):
        a = (n_pages * r) // world * page_tokens
        b = (n_pages * (r + 1)) // world * page_tokens
        out.append((min(a, n_rows), min(b, n_rows)))
    return out


def owner_of_row(row: int, n_rows: int, world: int, page_tokens: int = 64) -> int:
    """Rank whose slice holds (or, for row == n_rows, will receive) the given row."""
    sl = kv_slices(max(n_rows, row + 1), world, page_tokens)
    for r, (a, b) in enumerate(sl):
        if a <= row < b:
            return r
    return world - 1


def partial_width(d_v: int) -> int:
    return 2 + d_v


def pack_partial(m: np.ndarray, l: np.ndarray, o: np.ndarray) -> np.ndarray:
    """(max[rows], sum[rows], O[rows, d_v]) -> the [rows, 2 + d_v] fp32 layout that
    fst_cuda_mla_run_partial_device writes and fst_cuda_mla_run_merge_device reads."""
    return np.concatenate([m[:, None], l[:, None], o], axis=1).astype(np.float32)


def unpack_partials(g: np.ndarray):
    """[parts, rows, 2 + d_v] -> (m[parts, rows], l[parts, rows], o[parts, rows, d_v])."""
    return g[..., 0], g[..., 1], g[..., 2:]


class SplitKvLayer:
    """Decode of one long sequence with its cache split along the KV axis over the ranks of
    a process group.  Each rank holds a context whose sequence stores only its slice."""

    def __init__(self, ctx, seq: int, slice_begin: int, slice_rows: int, group=None):
        import torch
        import torch.distributed as dist
        self.torch, self.dist = torch, dist
        self.ctx, self.seq, self.group = ctx, seq, group
        self.begin, self.rows = slice_begin, slice_rows
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        H, dv = ctx.cfg.n_heads, ctx.dims["d_v"]
        T = ctx.cfg.max_tokens
        dev = torch.device("cuda", ctx.cfg.device)
        self.partial = torch.empty((T * H, 2 + dv), dtype=torch.float32, device=dev)
        self.gathered = torch.empty((self.world * T * H, 2 + dv), dtype=torch.float32, device=dev)

    def plan(self, global_pos: int, q_len: int, append_here: bool) -> None:
        """The new tokens sit at global rows global_pos ..; only the owner of the last slice
        appends them (local row = global - slice_begin), the others attend to their slice."""
        local = global_pos - self.begin if append_here else self.rows
        self.ctx.plan([(self.seq, local, q_len, global_pos, 1 if append_here else 0)])
        if append_here:
            self.rows = local + q_len

    def run(self, lid: int, d_h_in: int, d_h_out: int) -> None:
        """Layer call: local attention partial -> all-gather -> merge + output projections."""
        T = self.ctx.plan_tokens()
        H = self.ctx.cfg.n_heads
        part = self.partial[:T * H]
        gath = self.gathered[:self.world * T * H]  # rank-major concatenation of [T*H, 2 + d_v]
        self.ctx.run_partial_device(lid, d_h_in, part.data_ptr())
        self.dist.all_gather_into_tensor(gath, part, group=self.group)
        self.ctx.run_merge_device(lid, gath.data_ptr(), self.world, d_h_out)
