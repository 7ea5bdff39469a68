"""QK / softmax / SV over the paged cache (the qksv dispatches and the host softmax of
process_mla, src/fst_engine.cpp:3573-3683) through fst_cuda_mla_attention_only, against the
CPU oracle on the same seeded inputs.  Ragged lengths, page boundaries +-1, causal blocks."""
import numpy as np
import pytest

from fastar_b200 import mla, synth
from oracle import oracle as O
from tests.helpers import check_close, oracle_cfg

pytestmark = pytest.mark.gpu

IMPLS = [("simt", mla.IMPL_SIMT), ("tensor", mla.IMPL_TENSOR)]
PRESETS = [("baseline", mla.PRESET_BASELINE), ("v4", mla.PRESET_FASTAR_V4)]


def setup_ctx(preset, impl, n_pages, max_tokens, max_seqs=64):
    cfg = mla.make_config(preset, n_pages=n_pages, max_tokens=max_tokens, max_seqs=max_seqs, attn_impl=impl,
                          gemm_impl=mla.IMPL_SIMT)
    ctx = mla.MlaContext(cfg)
    # attention_only needs a layer with weights only for the V4 sinks; give it small real ones
    return cfg, ctx


def dummy_weights(cfg, sinks=None):
    w = {n: np.zeros(s, np.uint16) for n, s in mla.weight_shapes(cfg).items() if n != "attn_sinks"}
    if cfg.preset == mla.PRESET_FASTAR_V4:
        w["attn_sinks"] = sinks
    return w


def run_case(preset, impl, lens, q_len=1, causal=False, seed=0, q_std=1.0, shuffle_pages=True, ulps=0, windows=None):
    n_pages = sum((L + q_len + 63) // 64 for L in lens) + 8
    B = len(lens)
    cfg, ctx = setup_ctx(preset, impl, n_pages, B * q_len, max_seqs=B + 8)
    try:
        d = mla.dims_of(cfg)
        H = cfg.n_heads
        rng = np.random.default_rng(seed)
        sinks = rng.standard_normal(H).astype(np.float32) if preset == mla.PRESET_FASTAR_V4 else None
        ctx.set_layer_weights(0, dummy_weights(cfg, sinks))
        # scatter the pages: allocate throw-away sequences, free them in a shuffled order
        if shuffle_pages:
            tmp = [ctx.seq_alloc() for _ in range(4)]
            for s in tmp:
                ctx.seq_reserve(s, 64 * (n_pages // 8))
            for s in rng.permutation(tmp):
                ctx.seq_free(int(s))
        seqs, caches = [], []
        for b, L in enumerate(lens):
            s = ctx.seq_alloc()
            rows = synth.to_bf16_bits(synth.cache_rows_f32(cfg, seed, b, L + q_len))
            ctx.cache_write(0, s, 0, rows)
            seqs.append(s)
            caches.append(synth.from_bf16_bits(rows))
        windows = windows or [0] * B
        T = ctx.plan([(s, L, q_len, -1, 0 if not causal else 1, W) for s, L, W in zip(seqs, lens, windows)], causal=causal)
        assert T == B * q_len
        q = synth.to_bf16_bits((rng.standard_normal((T * H, d["d_qk"])) * q_std).astype(np.float32))
        got = ctx.attention_only(0, q)
        ocfg = oracle_cfg(cfg)
        qf = synth.from_bf16_bits(q)
        for b, L in enumerate(lens):
            kv_len = L + q_len if causal else L
            if windows[b] > 0:
                want = O.attention_window(ocfg, qf[b * q_len * H:(b + 1) * q_len * H], caches[b], kv_len, q_len,
                                          windows[b], pos0=L, causal=causal, sinks=sinks)
            else:
                want = O.attention(ocfg, qf[b * q_len * H:(b + 1) * q_len * H], caches[b], kv_len, q_len, pos0=L,
                                   causal=causal, sinks=sinks)
            if preset == mla.PRESET_FASTAR_V4:
                # the V4 output stage carries the inverse RoPE of the tail (src/fst_engine.cpp:3716)
                for r in range(q_len * H):
                    want[r, -64:] = O.rope_apply(want[r, -64:], L + r // H, inverse=True, round_bf16=True)
            check_close(got[b * q_len * H:(b + 1) * q_len * H], want, f"seq {b} (L={L})", ulps=ulps)
    finally:
        ctx.close()


@pytest.mark.parametrize("impl", IMPLS, ids=[i[0] for i in IMPLS])
@pytest.mark.parametrize("preset", PRESETS, ids=[p[0] for p in PRESETS])
def test_decode_ragged_lengths(preset, impl):
    # one token, one page, page boundary -1/0/+1, tile boundary -1/0/+1, several tiles
    run_case(preset[1], impl[1], [1, 2, 63, 64, 65, 127, 128, 129, 191, 200, 257, 700], ulps=1)


@pytest.mark.parametrize("impl", IMPLS, ids=[i[0] for i in IMPLS])
def test_decode_config1_shape(impl):
    # batch 1 over a 4096-token cache: the split-KV schedule spreads one sequence over many CTAs
    run_case(mla.PRESET_BASELINE, impl[1], [4096], seed=1)


@pytest.mark.parametrize("impl", IMPLS, ids=[i[0] for i in IMPLS])
def test_decode_sharp_softmax(impl):
    # large query norm: scores spread over hundreds of units, the running maximum moves often
    # (outputs reach several units here: the bound is one bf16 step at that magnitude)
    run_case(mla.PRESET_BASELINE, impl[1], [300, 1000, 129], seed=2, q_std=6.0, ulps=1)


@pytest.mark.parametrize("impl", IMPLS, ids=[i[0] for i in IMPLS])
@pytest.mark.parametrize("preset", PRESETS, ids=[p[0] for p in PRESETS])
def test_causal_verify_block(preset, impl):
    # 16 query tokens, causal among themselves (the speculative-verify block, 6005-6014):
    # token i sees rows <= pos0 + i (mask at 3626)
    run_case(preset[1], impl[1], [100, 128, 250], q_len=16, causal=True, seed=3, ulps=1)


@pytest.mark.parametrize("preset", PRESETS, ids=[p[0] for p in PRESETS])
def test_blocks_of_tokens_with_a_sharp_softmax(preset):
    # 16-token causal blocks over enough pages for the block schedule (groups of 16 lanes, whole-tile
    # QK issue running ahead of the softmax), with a large query norm: the reference maximum moves
    # often, also in the middle of a sequence, so the rescaling of O between the SV MMAs of
    # consecutive tiles is exercised; lengths on and beside page boundaries
    run_case(preset[1], mla.IMPL_TENSOR, [1500, 1023, 2048, 640, 3001], q_len=16, causal=True, seed=8, q_std=6.0, ulps=1)


def test_empty_batch_and_zero_context():
    cfg, ctx = setup_ctx(mla.PRESET_BASELINE, mla.IMPL_AUTO, 8, 4)
    try:
        ctx.set_layer_weights(0, dummy_weights(cfg))
        assert ctx.plan([]) == 0
        s = ctx.seq_alloc()
        # a sequence with nothing cached and nothing appended attends to nothing: output 0
        T = ctx.plan([(s, 0, 1, -1, 0)])
        q = np.zeros((T * cfg.n_heads, 576), np.uint16)
        out = ctx.attention_only(0, q)
        assert not out.any()
    finally:
        ctx.close()


@pytest.mark.parametrize("impl", IMPLS, ids=[i[0] for i in IMPLS])
def test_constant_cache_returns_the_row(impl):
    # softmax weights sum to one: if every cached row is the same, the output is that row,
    # whatever the queries, lengths or split schedule.  Size-independent check at the full
    # context length of the batched benchmark (8192 rows).
    cfg, ctx = setup_ctx(mla.PRESET_BASELINE, impl[1], 8192 // 64 * 2 + 4, 2)
    try:
        ctx.set_layer_weights(0, dummy_weights(cfg))
        rng = np.random.default_rng(4)
        row = synth.to_bf16_bits(rng.standard_normal((1, 576)).astype(np.float32))
        lens = [8192, 5000]
        seqs = []
        for L in lens:
            s = ctx.seq_alloc()
            ctx.cache_write(0, s, 0, np.repeat(row, L, axis=0))
            seqs.append(s)
        T = ctx.plan([(s, L, 1, -1, 0) for s, L in zip(seqs, lens)])
        q = synth.to_bf16_bits(rng.standard_normal((T * 64, 576)).astype(np.float32))
        out = synth.from_bf16_bits(ctx.attention_only(0, q))
        want = np.broadcast_to(synth.from_bf16_bits(row)[:, :512], out.shape)
        assert np.max(np.abs(out - want)) <= 2.0 ** -7 * np.max(np.abs(want))
    finally:
        ctx.close()


def test_many_short_segments_per_cta():
    # 240 sequences of 1 .. 200 tokens: more segments than SMs, so every CTA of the tcgen05 kernel
    # runs several one- to three-tile segments back to back (Q_eff replaced in tensor memory and a
    # partial written at every boundary) and the merge sees one part for almost every row
    rng = np.random.default_rng(11)
    lens = [int(x) for x in rng.integers(1, 201, size=240)]
    run_case(mla.PRESET_BASELINE, mla.IMPL_TENSOR, lens, seed=11, ulps=1)


def test_long_and_short_sequences_mixed():
    # one 20 000-token sequence among short ones: its tiles spread over most CTAs while the short
    # sequences share the remaining ones; the long row's parts are merged from ~140 partials
    run_case(mla.PRESET_BASELINE, mla.IMPL_TENSOR, [20000, 3, 64, 130, 65, 1], seed=12, ulps=1)


@pytest.mark.parametrize("impl", IMPLS, ids=[i[0] for i in IMPLS])
@pytest.mark.parametrize("preset", PRESETS, ids=[p[0] for p in PRESETS])
def test_sliding_window(preset, impl):
    """FstMlaSeqStep.window: every query token sees only the last `window` rows of what it may see
    (the draft model's window, src/fst_engine.cpp:2534-2576).  Windows that start inside a page, on
    a page boundary, cover the whole context, and a causal block whose window moves with the token;
    different windows in one batch."""
    preset, impl = preset[1], impl[1]
    cases = [(300, 1, False, 100), (300, 1, False, 128), (640, 1, False, 64), (70, 1, False, 4096),
             (5000, 1, False, 1000), (513, 1, False, 1), (200, 5, True, 128), (1000, 16, True, 130)]
    n_pages = sum((L + q + 63) // 64 for L, q, _, _ in cases) + 8
    for causal in (False, True):
        sub = [c for c in cases if c[2] == causal]
        groups = {}
        for c in sub:
            groups.setdefault(c[1], []).append(c)
        for q_len, grp in groups.items():
            B = len(grp)
            cfg, ctx = setup_ctx(preset, impl, n_pages, B * q_len, max_seqs=B + 8)
            try:
                d, H = mla.dims_of(cfg), cfg.n_heads
                rng = np.random.default_rng(11)
                sinks = rng.standard_normal(H).astype(np.float32) if preset == mla.PRESET_FASTAR_V4 else None
                ctx.set_layer_weights(0, dummy_weights(cfg, sinks))
                seqs, caches = [], []
                for b, (L, _, _, _) in enumerate(grp):
                    s = ctx.seq_alloc()
                    rows = synth.to_bf16_bits(synth.cache_rows_f32(cfg, 3, b, L + q_len))
                    ctx.cache_write(0, s, 0, rows)
                    seqs.append(s)
                    caches.append(synth.from_bf16_bits(rows))
                T = ctx.plan([(s, L, q_len, -1, 1 if causal else 0, W) for s, (L, _, _, W) in zip(seqs, grp)], causal=causal)
                assert T == B * q_len
                info = ctx.plan_info()
                want_rows = sum(sum(min(W, (L + i + 1) if causal else L) for i in range(q_len)) for L, _, _, W in grp)
                assert info["kv_rows"] == want_rows
                q = synth.to_bf16_bits(rng.standard_normal((T * H, d["d_qk"])).astype(np.float32))
                got = ctx.attention_only(0, q)
                ocfg, qf = oracle_cfg(cfg), synth.from_bf16_bits(q)
                for b, (L, _, _, W) in enumerate(grp):
                    kv_len = L + q_len if causal else L
                    want = O.attention_window(ocfg, qf[b * q_len * H:(b + 1) * q_len * H], caches[b], kv_len, q_len, W,
                                              pos0=L, causal=causal, sinks=sinks)
                    if preset == mla.PRESET_FASTAR_V4:
                        for r in range(q_len * H):
                            want[r, -64:] = O.rope_apply(want[r, -64:], L + r // H, inverse=True, round_bf16=True)
                    check_close(got[b * q_len * H:(b + 1) * q_len * H], want, f"L={L} q={q_len} W={W}")
            finally:
                ctx.close()


@pytest.mark.parametrize("seed", range(10))
def test_random_shapes(seed):
    """Seeded random batches through the tcgen05 kernel: ragged contexts (empty ones included), one
    token or a causal block per sequence, some sequences with a sliding window, both presets."""
    rng = np.random.default_rng(1000 + seed)
    preset = PRESETS[seed % 2][1]
    B = int(rng.integers(1, 7))
    q_len = int(rng.choice([1, 1, 1, 2, 5, 16]))
    causal = q_len > 1
    lens = [int(x) for x in rng.choice([0, 1, 63, 64, 65, 500, 1500, 3000], size=B)]
    lens = [max(L + int(rng.integers(-3, 4)), 0) for L in lens]
    if not causal:
        lens = [max(L, 1) for L in lens]  # a token that sees nothing has no softmax
    windows = [int(rng.choice([0, 0, 1, 64, 100, 777])) for _ in range(B)]
    run_case(preset, mla.IMPL_TENSOR, lens, q_len=q_len, causal=causal, seed=seed, windows=windows, ulps=1)
