"""The whole MLA layer through fst_cuda_mla_forward (process_mla with host buffers) against
the CPU oracle on identical seeded inputs: stage by stage (the FST_MLA_TRACE stage list,
src/fst_engine.cpp:3396-3407, 3521-3532, 3685-3695, 3841-3851) and end to end."""
import numpy as np
import pytest

from fastar_b200 import mla, synth
from oracle import oracle as O
from tests.helpers import check_close, oracle_cfg

pytestmark = pytest.mark.gpu

IMPLS = [("simt", mla.IMPL_SIMT, mla.IMPL_SIMT), ("tensor", mla.IMPL_TENSOR, mla.IMPL_AUTO)]
_W = {}


def weights_for(preset, attn_norm=False):
    """Seed-0 weights of the preset at full size, as bits (GPU) and rounded fp32 (oracle).
    attn_norm: also the weight of the RMSNorm in front of the layer, N(1, 0.1^2)."""
    key = (preset, attn_norm)
    if key not in _W:
        cfg = mla.make_config(preset)
        w = synth.layer_weights_f32(cfg, 0, 0)
        if attn_norm:
            w["attn_norm"] = 1.0 + synth.normal_f32(0, "attn_norm", (cfg.hidden,), 0.1, (0,))
        _W[key] = (synth.weights_to_bits(w), synth.weights_rounded(w))
    return _W[key]


def run_layer(preset, impl, lens, q_len, causal, seed=0, steps=1, ulps=0, attn_norm=False, rope_yarn=False,
              yarn_by_layer_call=False):
    """`steps` consecutive layer calls (each appends q_len tokens per sequence); every call is
    compared with the oracle, and so is the cache content afterwards."""
    attn_impl, gemm_impl = impl[1], impl[2]
    B = len(lens)
    n_pages = sum((L + q_len * steps + 63) // 64 for L in lens) + 4
    cfg = mla.make_config(preset, n_pages=n_pages, max_tokens=B * q_len, max_seqs=B, attn_impl=attn_impl,
                          gemm_impl=gemm_impl, rope_yarn=rope_yarn and not yarn_by_layer_call)
    bits, rounded = weights_for(preset, attn_norm)
    ocfg = oracle_cfg(cfg)
    ocfg.rope_yarn = int(rope_yarn)
    d = mla.dims_of(cfg)
    H = cfg.n_heads
    with mla.MlaContext(cfg) as ctx:
        ctx.set_layer_weights(0, bits)
        if yarn_by_layer_call:
            ctx.set_layer_rope(0, rope_yarn)
        seqs, caches = [], []
        for b, L in enumerate(lens):
            s = ctx.seq_alloc()
            rows = synth.to_bf16_bits(synth.cache_rows_f32(cfg, seed, b, L))
            if L:
                ctx.cache_write(0, s, 0, rows)
            seqs.append(s)
            cache = np.zeros((L + q_len * steps, d["row"]), np.float32)
            cache[:L] = synth.from_bf16_bits(rows)
            caches.append(cache)
        pos = list(lens)
        for step in range(steps):
            h = synth.to_bf16_bits(synth.hidden_f32(cfg, seed, B * q_len, (step,)))
            out = ctx.forward(0, h, seqs, pos, [q_len] * B, causal=causal)
            stages = {k: ctx.get_stage(v) for k, v in (("qc", mla.STAGE_QC), ("kv", mla.STAGE_KV),
                                                      ("q_eff", mla.STAGE_QEFF), ("o_lat", mla.STAGE_OLAT),
                                                      ("low", mla.STAGE_LOW))}
            hf = synth.from_bf16_bits(h)
            for b in range(B):
                r = O.mla_forward(ocfg, rounded, hf[b * q_len:(b + 1) * q_len], pos[b], caches[b], causal=causal)
                sl = slice(b * q_len, (b + 1) * q_len)
                slh = slice(b * q_len * H, (b + 1) * q_len * H)
                # normed intermediates are O(1..8): one or two bf16 steps there exceed 2e-2
                check_close(stages["qc"][sl], r.trace["qc"], f"step {step} seq {b} qc", ulps=2)
                check_close(stages["kv"][sl], r.trace["kv"], f"step {step} seq {b} kv", ulps=2)
                check_close(stages["q_eff"][slh], r.trace["q_eff"], f"step {step} seq {b} q_eff", ulps=2)
                check_close(stages["o_lat"][slh], r.trace["o_lat"], f"step {step} seq {b} o_lat", ulps=ulps)
                check_close(stages["low"][sl], r.trace["low"], f"step {step} seq {b} low", ulps=ulps)
                check_close(out[sl], r.out, f"step {step} seq {b} out", ulps=ulps)
                # cache push: the appended rows are the kv stage rows, bit for bit, at the rows
                # the block table names
                got_rows = ctx.cache_read(0, seqs[b], pos[b], q_len)
                assert np.array_equal(got_rows, stages["kv"][sl])
                pos[b] += q_len
        # the history itself is untouched
        for b, L in enumerate(lens):
            if L:
                assert np.array_equal(ctx.cache_read(0, seqs[b], 0, L),
                                      synth.to_bf16_bits(caches[b][:L]))


@pytest.mark.parametrize("impl", IMPLS, ids=[i[0] for i in IMPLS])
def test_decode_batch1_config1(impl):
    # "decode at batch 1 over a 4096-token cache"
    run_layer(mla.PRESET_BASELINE, impl, [4096], 1, False)


@pytest.mark.parametrize("impl", IMPLS, ids=[i[0] for i in IMPLS])
def test_decode_ragged_batch(impl):
    # batched decode, ragged context lengths, two consecutive steps
    run_layer(mla.PRESET_BASELINE, impl, [1030, 64, 1, 700, 0, 129, 2047, 333], 1, False, seed=1, steps=2)


@pytest.mark.parametrize("impl", IMPLS, ids=[i[0] for i in IMPLS])
def test_verify_block_causal(impl):
    # 16 query tokens per sequence, causal among themselves, appended at L .. L+15
    run_layer(mla.PRESET_BASELINE, impl, [200, 64], 16, True, seed=2)


@pytest.mark.parametrize("preset", [mla.PRESET_BASELINE, mla.PRESET_FASTAR_V4], ids=["baseline", "v4"])
@pytest.mark.parametrize("q_len,causal", [(16, True), (5, False)], ids=["verify-16", "dense-5"])
def test_blocks_of_tokens_scheduled_by_groups_of_lanes(preset, q_len, causal):
    """Calls with G >= 4 new tokens per sequence and enough pages are cut by BLOCKS (n_sm / G groups of
    G thread blocks, lane i of a group takes token i of each sequence over the group's run of page
    columns).  Lengths around page boundaries make the causal edge bite: with 255 cached rows token 0
    of a 16-token block ends in page 3 and the others reach page 4; with 1023 the block ends
    exactly at a boundary.  Against the oracle stage by stage, two consecutive calls."""
    run_layer(preset, IMPLS[1], [255, 256, 1023, 64 * 30 + 3, 700, 0, 4000], q_len, causal, seed=7, steps=2, ulps=2)


def test_block_schedule_against_the_token_schedule():
    """The same 16-token verify call under both schedules: the block schedule uses whole groups of 16
    thread blocks and leaves most tokens in one part; outputs agree to the rounding of a bf16 step
    (the parts are cut at other rows, so the fp32 sums differ in their last bits)."""
    lens, q = [3000, 1500, 2047, 900, 4100, 64], 16
    B = len(lens)
    cfg = mla.make_config(mla.PRESET_BASELINE, n_pages=sum((L + q + 63) // 64 for L in lens) + 4, max_tokens=B * q, max_seqs=B)
    bits, _ = weights_for(mla.PRESET_BASELINE)
    with mla.MlaContext(cfg) as ctx:
        ctx.set_layer_weights(0, bits)
        seqs = []
        for b, L in enumerate(lens):
            s = ctx.seq_alloc()
            ctx.cache_write(0, s, 0, synth.to_bf16_bits(synth.cache_rows_f32(cfg, 12, b, L)))
            seqs.append(s)
        h = synth.to_bf16_bits(synth.hidden_f32(cfg, 12, B * q))
        res = {}
        for key, on in (("blocks", True), ("tokens", False), ("blocks again", True)):
            ctx.set_block_schedule(on)
            out = ctx.forward(0, h, seqs, lens, [q] * B, causal=True)
            res[key] = (out.copy(), ctx.plan_info())
            for s, L in zip(seqs, lens):
                ctx.seq_truncate(s, L)
        n_sm = res["tokens"][1]["n_ctas"]
        assert res["blocks"][1]["n_ctas"] == n_sm // q * q
        assert res["blocks"][1]["kv_rows"] == res["tokens"][1]["kv_rows"] == sum(L + i + 1 for L in lens for i in range(q))
        assert res["blocks"][1]["n_partials"] < res["tokens"][1]["n_partials"]
        assert np.array_equal(res["blocks"][0], res["blocks again"][0])
        check_close(res["blocks"][0], synth.from_bf16_bits(res["tokens"][0]), "block schedule vs token schedule", ulps=1)


@pytest.mark.parametrize("impl", IMPLS, ids=[i[0] for i in IMPLS])
def test_prefill_from_empty(impl):
    # the reference's own regime: 16-token chunks from position 0 (prefill_tiled, 2957-2984)
    run_layer(mla.PRESET_BASELINE, impl, [0], 16, True, seed=3, steps=2)


@pytest.mark.parametrize("impl", IMPLS, ids=[i[0] for i in IMPLS])
def test_fastar_v4_preset(impl):
    # the live engine's form: 512-wide rows, per-head q norm, sink, inverse RoPE, grouped wo_a
    # (its outputs reach several units: the absolute bound is two bf16 steps at that magnitude)
    run_layer(mla.PRESET_FASTAR_V4, impl, [100, 0, 129], 2, True, seed=4, steps=2, ulps=2)


@pytest.mark.parametrize("impl", IMPLS, ids=[i[0] for i in IMPLS])
@pytest.mark.parametrize("preset", [mla.PRESET_BASELINE, mla.PRESET_FASTAR_V4], ids=["baseline", "v4"])
def test_attn_norm_in_front_of_the_layer(impl, preset):
    # process_layer's attention half (src/fst_engine.cpp:2687-2689): the layer call takes the rows
    # before attn_norm and applies it itself; inputs with a row scale far from 1 so that a missing
    # norm cannot pass
    run_layer(preset, impl, [300, 65], 2, True, seed=5, steps=2, ulps=2, attn_norm=True)


@pytest.mark.parametrize("impl", IMPLS, ids=[i[0] for i in IMPLS])
@pytest.mark.parametrize("preset", [mla.PRESET_BASELINE, mla.PRESET_FASTAR_V4], ids=["baseline", "v4"])
@pytest.mark.parametrize("by_call", [False, True], ids=["config", "per-layer"])
def test_yarn_rope_tables(impl, preset, by_call):
    # the YaRN tables of the compressed layers (build_rope_lut, src/fst_engine.cpp:1995-2022) on the
    # key, the query and (V4) the inverse output rotation: new rows at positions 60..67 and
    # 4090..4097, both across a page boundary; stages kv and q_eff are compared inside run_layer.
    # Far positions matter: below a few hundred the YaRN and plain angles of the slow pairs agree
    # to bf16 precision.
    run_layer(preset, impl, [60, 4090], 8, True, seed=6, ulps=2, rope_yarn=True, yarn_by_layer_call=by_call)


def test_yarn_and_plain_tables_differ_on_the_device():
    """A context with one plain and one YaRN layer keeps both tables per plan; the same weights and
    rows give different q_eff / kv in the rope dims only."""
    cfg = mla.make_config(mla.PRESET_FASTAR_V4, n_pages=80, max_tokens=2, max_seqs=1, n_layers=2)
    bits, _ = weights_for(mla.PRESET_FASTAR_V4)
    with mla.MlaContext(cfg) as ctx:
        ctx.set_layer_weights(0, bits)
        ctx.set_layer_weights(1, bits)
        ctx.set_layer_rope(1, True)
        s = ctx.seq_alloc()
        rows = synth.to_bf16_bits(synth.cache_rows_f32(cfg, 7, 0, 4000))
        ctx.cache_write(0, s, 0, rows)
        ctx.cache_write(1, s, 0, rows)
        h = synth.to_bf16_bits(synth.hidden_f32(cfg, 7, 2))
        kv = []
        for lid in range(2):
            ctx.forward(lid, h, [s], [4000], [2])
            kv.append(ctx.get_stage(mla.STAGE_KV).copy())
        assert np.array_equal(kv[0][:, :448], kv[1][:, :448])      # the nope part does not rotate
        assert not np.array_equal(kv[0][:, 448:], kv[1][:, 448:])  # the rope tail does, differently


def test_plan_is_kept_across_the_layers_of_a_step():
    """process_layer calls process_mla once per layer with the same seq_pos_ (src/fst_engine.cpp:2687):
    the second request for the same steps keeps the plan that is on the device, gives the same bits as
    a rebuilt plan, and anything that touches a sequence makes the next request build a new one."""
    lens, B = [130, 64, 700], 3
    cfg = mla.make_config(mla.PRESET_BASELINE, n_pages=sum((L + 66) // 64 for L in lens) + 4, max_tokens=B,
                          max_seqs=B, n_layers=2)
    bits, _ = weights_for(mla.PRESET_BASELINE)
    with mla.MlaContext(cfg) as ctx:
        for lid in range(2):
            ctx.set_layer_weights(lid, bits)
        seqs = []
        for b, L in enumerate(lens):
            s = ctx.seq_alloc()
            rows = synth.to_bf16_bits(synth.cache_rows_f32(cfg, 0, b, L))
            for lid in range(2):
                ctx.cache_write(lid, s, 0, rows)
            seqs.append(s)
        h = synth.to_bf16_bits(synth.hidden_f32(cfg, 0, B, (0,)))
        c0 = ctx.plan_counts()
        out0 = ctx.forward(0, h, seqs, lens, [1] * B)        # layer 0 of the step: builds
        out1 = ctx.forward(1, h, seqs, lens, [1] * B)        # layer 1: same steps, plan kept
        c1 = ctx.plan_counts()
        assert (c1["built"] - c0["built"], c1["reused"] - c0["reused"]) == (1, 1)
        assert np.array_equal(out0, out1)                    # same weights, same cache rows in both layers
        ctx.set_plan_reuse(False)
        out2 = ctx.forward(1, h, seqs, lens, [1] * B)        # rebuilt: same bits
        c2 = ctx.plan_counts()
        assert (c2["built"] - c1["built"], c2["reused"] - c1["reused"]) == (1, 0)
        assert np.array_equal(out1, out2)
        ctx.set_plan_reuse(True)
        # the next step (positions moved on) and a rollback both ask for a new plan
        nxt = [L + 1 for L in lens]
        ctx.forward(0, h, seqs, nxt, [1] * B)
        c3 = ctx.plan_counts()
        assert c3["built"] - c2["built"] == 1
        ctx.seq_truncate(seqs[0], lens[0])
        ctx.seq_truncate(seqs[1], lens[1])
        ctx.seq_truncate(seqs[2], lens[2])
        out3 = ctx.forward(0, h, seqs, lens, [1] * B)
        c4 = ctx.plan_counts()
        assert (c4["built"] - c3["built"], c4["reused"] - c3["reused"]) == (1, 0)
        assert np.array_equal(out0, out3)


def test_page_locked_buffers_take_the_direct_paths():
    """fst_cuda_mla_forward with page-locked, device-addressable buffers (input copied straight from
    the caller's buffer, output rows written by the last GEMM itself) gives the bits of the same call
    with pageable buffers (staged copies)."""
    import torch
    lens, B = [200, 1, 64, 513], 4
    cfg = mla.make_config(mla.PRESET_BASELINE, n_pages=sum((L + 65) // 64 for L in lens) + 4, max_tokens=B, max_seqs=B)
    bits, _ = weights_for(mla.PRESET_BASELINE)
    with mla.MlaContext(cfg) as ctx:
        ctx.set_layer_weights(0, bits)
        seqs = []
        for b, L in enumerate(lens):
            s = ctx.seq_alloc()
            ctx.cache_write(0, s, 0, synth.to_bf16_bits(synth.cache_rows_f32(cfg, 0, b, L)))
            seqs.append(s)
        h = synth.to_bf16_bits(synth.hidden_f32(cfg, 0, B, (0,)))
        ref = ctx.forward(0, h, seqs, lens, [1] * B)
        for s, L in zip(seqs, lens):
            ctx.seq_truncate(s, L)
        h_pin = torch.from_numpy(h.view(np.int16).copy()).pin_memory()
        out_pin = torch.zeros_like(h_pin).pin_memory()
        call = ctx.bind_forward(0, h_pin.numpy().view(np.uint16), out_pin.numpy().view(np.uint16),
                                np.array(seqs, np.int32), np.array(lens, np.int32), np.ones(B, np.int32))
        call()
        assert np.array_equal(out_pin.numpy().view(np.uint16), ref)
        assert np.array_equal(ctx.get_stage(mla.STAGE_OUT), ref)


def test_forward_with_a_window_set_on_the_context():
    """fst_cuda_mla_set_window: process_mla attends to the last `window` rows only.  Checked on the
    attention stage: the oracle's windowed attention of the Q_eff the GPU produced; the appended row
    and the other stages do not depend on the window."""
    lens, B, W = [300, 64, 1000], 3, 100
    cfg = mla.make_config(mla.PRESET_BASELINE, n_pages=sum((L + 65) // 64 for L in lens) + 4, max_tokens=B, max_seqs=B)
    bits, _ = weights_for(mla.PRESET_BASELINE)
    ocfg, H = oracle_cfg(cfg), cfg.n_heads
    with mla.MlaContext(cfg) as ctx:
        ctx.set_layer_weights(0, bits)
        seqs = []
        for b, L in enumerate(lens):
            s = ctx.seq_alloc()
            ctx.cache_write(0, s, 0, synth.to_bf16_bits(synth.cache_rows_f32(cfg, 0, b, L)))
            seqs.append(s)
        h = synth.to_bf16_bits(synth.hidden_f32(cfg, 0, B, (0,)))
        ctx.set_window(W)
        out_w = ctx.forward(0, h, seqs, lens, [1] * B)
        q_eff = synth.from_bf16_bits(ctx.get_stage(mla.STAGE_QEFF))
        o_lat = ctx.get_stage(mla.STAGE_OLAT)
        for b, (s, L) in enumerate(zip(seqs, lens)):
            cache = synth.from_bf16_bits(ctx.cache_read(0, s, 0, L + 1))
            want = O.attention_window(ocfg, q_eff[b * H:(b + 1) * H], cache, L + 1, 1, W)
            check_close(o_lat[b * H:(b + 1) * H], want, f"window, seq {b}")
        for s, L in zip(seqs, lens):
            ctx.seq_truncate(s, L)
        ctx.set_window(0)
        out_full = ctx.forward(0, h, seqs, lens, [1] * B)
        assert not np.array_equal(out_w[0], out_full[0])      # 301 rows against the last 100
        # 65 rows: the window covers them all (the split into partials differs, so not bit for bit)
        check_close(out_w[1:2], synth.from_bf16_bits(out_full[1:2]), "window covers the context")


@pytest.mark.parametrize("preset", [mla.PRESET_BASELINE, mla.PRESET_FASTAR_V4], ids=["baseline", "v4"])
@pytest.mark.parametrize("n_seqs", [45, 150], ids=["mostly-split", "mostly-whole"])
def test_tokens_finished_by_the_attention_kernel_equal_the_merge_kernel(preset, n_seqs):
    """A token whose whole context is one segment of the split-KV schedule is normalised and written
    by the attention kernel itself; with the switch off it goes through its partial and the merge
    kernel like the split ones.  Same bits either way (o_lat and the layer output), run after run,
    with the sink and the inverse RoPE of the V4 form, empty contexts included."""
    rng = np.random.default_rng(5)
    hi = 2600 if n_seqs < 100 else 400
    lens = [int(x) for x in rng.integers(40, hi, size=n_seqs - 5)] + [0, 1, 63, 64, 65]
    B, q = len(lens), 2
    cfg = mla.make_config(preset, n_pages=sum((L + q + 63) // 64 for L in lens) + 4, max_tokens=B * q, max_seqs=B)
    bits, _ = weights_for(preset)
    with mla.MlaContext(cfg) as ctx:
        ctx.set_layer_weights(0, bits)
        seqs = []
        for b, L in enumerate(lens):
            s = ctx.seq_alloc()
            if L:
                ctx.cache_write(0, s, 0, synth.to_bf16_bits(synth.cache_rows_f32(cfg, 9, b, L)))
            seqs.append(s)
        h = synth.to_bf16_bits(synth.hidden_f32(cfg, 9, B * q))
        res = {}
        for key, direct in (("direct", True), ("kernel", False), ("direct again", True)):
            ctx.set_fused_merge(direct)
            out = ctx.forward(0, h, seqs, lens, [q] * B, causal=True)
            res[key] = (out.copy(), ctx.get_stage(mla.STAGE_OLAT).copy())
            info = ctx.plan_info()
            for s, L in zip(seqs, lens):
                ctx.seq_truncate(s, L)
        # both kinds of token are present: some split over thread blocks, some whole
        assert info["n_partials"] > B * q - 5  # split tokens are present (whole ones too: the short contexts)
        a, b, c = res["direct"], res["kernel"], res["direct again"]
        assert np.array_equal(a[1], b[1]) and np.array_equal(a[0], b[0])
        assert np.array_equal(a[1], c[1]) and np.array_equal(a[0], c[0])
