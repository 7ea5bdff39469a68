"""The benchmark configurations at their FULL sizes against the CPU oracle, built exactly as
bench.py builds them (fastar_b200.workloads: seed 0, scrambled block tables): batched decode of
64 sequences with contexts in [1024, 8192], the 16-token causal verify block over 16384-row
caches, and the single 131072-row sequence on one GPU and split along the KV axis over two
contexts that stand in for two ranks.  Acceptance as everywhere: cosine >= 0.9999 and
max-abs <= 2e-2 on the bf16 outputs; appended cache rows bit-identical to the kv stage rows and
found where the block table says."""
import numpy as np
import pytest

from fastar_b200 import mla, parallel, synth, workloads
from oracle import oracle as O
from tests.helpers import check_close, oracle_cfg

pytestmark = pytest.mark.gpu


def oracle_caches(wl, which):
    """fp32 caches (bf16-representable values) of the chosen sequences, with room for the new rows."""
    d = mla.dims_of(wl.cfg)
    out = []
    for b in which:
        c = np.zeros((wl.rows[b] + wl.q_len, d["row"]), np.float32)
        c[:wl.rows[b]] = synth.from_bf16_bits(synth.to_bf16_bits(synth.cache_rows_f32(wl.cfg, wl.seed, wl.keys[b], wl.rows[b])))
        out.append(c)
    return out


def check_tables(wl):
    """Page mapping invariants: no page is owned twice, owned + free = all pages, and every
    sequence owns exactly the pages its length needs."""
    ctx, owned = wl.ctx, []
    for s, r in zip(wl.seqs, wl.rows):
        t = ctx.block_table(s)
        assert len(t) == (ctx.seq_len(s) + 63) // 64
        owned.extend(int(x) for x in t)
    assert len(owned) == len(set(owned)), "a page is owned by two sequences"
    assert all(0 <= p < wl.cfg.n_pages for p in owned)
    assert len(owned) + ctx.free_pages() == wl.cfg.n_pages


def run_and_check(wl, which, stage_ulps=2):
    """One layer call through fst_cuda_mla_forward for the whole batch; the sequences in `which`
    are compared with the oracle (output rows, o_lat, appended rows)."""
    ctx, q, H = wl.ctx, wl.q_len, wl.cfg.n_heads
    out = ctx.forward(0, wl.h_bits, wl.seqs, wl.rows, [q] * len(wl.seqs), causal=wl.causal)
    kv = ctx.get_stage(mla.STAGE_KV)
    o_lat = ctx.get_stage(mla.STAGE_OLAT)
    check_tables(wl)
    hf = synth.from_bf16_bits(wl.h_bits)
    w = synth.weights_rounded(synth.layer_weights_f32(wl.cfg, wl.seed, 0))
    caches = oracle_caches(wl, which)
    h_sel = np.concatenate([hf[b * q:(b + 1) * q] for b in which])
    r = O.mla_forward_batch(oracle_cfg(wl.cfg), w, h_sel, [q] * len(which), [wl.rows[b] for b in which], caches,
                            causal=wl.causal, want_trace=True)
    worst = (1.0, 0.0)
    for i, b in enumerate(which):
        sl, so = slice(b * q, (b + 1) * q), slice(i * q, (i + 1) * q)
        c, e = check_close(out[sl], r.out[so], f"seq {b} out")
        worst = (min(worst[0], c), max(worst[1], e))
        check_close(o_lat[b * q * H:(b + 1) * q * H], r.trace["o_lat"][i * q * H:(i + 1) * q * H], f"seq {b} o_lat")
        check_close(kv[sl], r.trace["kv"][so], f"seq {b} kv", ulps=stage_ulps)
        # the appended rows: bit for bit the kv stage rows, at the rows the block table names
        got = ctx.cache_read(0, wl.seqs[b], wl.rows[b], q)
        assert np.array_equal(got, kv[sl]), f"seq {b}: appended rows differ from the kv stage"
        table = ctx.block_table(wl.seqs[b])
        for j in (0, q - 1):
            pos = wl.rows[b] + j
            assert ctx.row_offset(wl.seqs[b], pos) == (int(table[pos // 64]) * 64 + pos % 64) * 576
    return worst


def test_config2_batched_decode_all_64_sequences():
    wl = workloads.build("batched")
    try:
        assert len(wl.seqs) == 64 and 1024 <= min(wl.rows) and max(wl.rows) <= 8192
        info_rows = sum(wl.rows)
        run_and_check(wl, list(range(64)))
        info = wl.ctx.plan_info()
        assert info["kv_rows"] == info_rows + 64  # every token also sees its own new row
    finally:
        wl.close()


def test_config3_verify_block_16_tokens_over_16384_rows():
    wl = workloads.build("verify")
    try:
        assert len(wl.seqs) == 32 and wl.q_len == 16 and all(r == 16384 for r in wl.rows)
        run_and_check(wl, [0, 13, 31])
    finally:
        wl.close()


def test_config4_one_131072_row_sequence_on_one_gpu():
    wl = workloads.build("longctx")
    try:
        assert wl.rows == [131072]
        run_and_check(wl, [0])
        assert wl.ctx.plan_info()["n_ctas"] > 100  # one sequence spread over the SMs
    finally:
        wl.close()


def test_config4_split_over_two_contexts():
    """Two contexts stand in for two ranks (one after the other on one GPU; no kernel waits on
    another): each holds its page-aligned slice, the partials are laid side by side as the
    all-gather would, and every 'rank' merges and projects."""
    import torch
    world = 2
    wls = [workloads.build("longctx", rank=r, world=world) for r in range(world)]
    try:
        L = int(wls[0].all_lens[0])
        H, dv = wls[0].cfg.n_heads, mla.dims_of(wls[0].cfg)["d_v"]
        owner = parallel.owner_of_row(L, L, world)
        d_h = torch.from_numpy(wls[0].h_bits.view(np.int16)).cuda()
        d_out = torch.empty_like(d_h)
        gathered = torch.zeros((world, H, 2 + dv), dtype=torch.float32, device="cuda")
        for r, wl in enumerate(wls):
            s = wl.seqs[0]
            if r == owner:
                wl.ctx.plan([(s, L - wl.slice_begin, 1, L, 1)])
            else:
                wl.ctx.plan([(s, wl.rows[0], 1, L, 0)])
            wl.ctx.run_partial_device(0, d_h.data_ptr(), gathered[r].data_ptr())
            wl.ctx.sync()
        full = wls[0]
        cache = np.zeros((L + 1, 576), np.float32)
        cache[:L] = synth.from_bf16_bits(synth.to_bf16_bits(synth.cache_rows_f32(full.cfg, 0, 0, L)))
        w = synth.weights_rounded(synth.layer_weights_f32(full.cfg, 0, 0))
        want = O.mla_forward(oracle_cfg(full.cfg), w, synth.from_bf16_bits(full.h_bits), L, cache)
        for wl in wls:
            wl.ctx.run_merge_device(0, gathered.data_ptr(), world, d_out.data_ptr())
            wl.ctx.sync()
            check_close(d_out.cpu().numpy().view(np.uint16), want.out, "merged output")
        new_row = wls[owner].ctx.cache_read(0, wls[owner].seqs[0], L - wls[owner].slice_begin, 1)
        check_close(new_row, want.trace["kv"], "appended row", ulps=2)
    finally:
        for wl in wls:
            wl.close()
