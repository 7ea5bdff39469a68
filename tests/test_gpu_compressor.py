"""The V4 KV compressor and its attention columns (reference compress_token, src/fst_engine.cpp:
3171-3318; columns 3565-3586, causal rule 3630-3635) through the C ABI against the CPU oracle: a
context with a plain layer, a ratio-4 layer and a ratio-128 layer, three sequences prefilled in
causal chunks and then decoded as a batch; compressed rows, every layer output, and the undo of a
rejected speculative block."""
import numpy as np
import pytest

from fastar_b200 import mla, synth
from oracle import oracle as O
from tests.helpers import check_close, cosine, oracle_cfg
from tests.test_gpu_layer import weights_for

pytestmark = pytest.mark.gpu

RATIOS = [0, 4, 128]


def compressor_weights(cfg, ratio, seed):
    rng = np.random.default_rng(seed)
    width = 2 * cfg.kv_lora if ratio == 4 else cfg.kv_lora
    w = {"wkv": rng.standard_normal((width, cfg.hidden)).astype(np.float32) * 0.02,
         "wgate": rng.standard_normal((width, cfg.hidden)).astype(np.float32) * 0.02,
         "ape": rng.standard_normal((ratio, width)).astype(np.float32),
         "norm": (1.0 + 0.1 * rng.standard_normal(cfg.kv_lora)).astype(np.float32)}
    bits = {k: (v if k == "ape" else synth.to_bf16_bits(v)) for k, v in w.items()}
    rounded = {k: (v if k == "ape" else synth.from_bf16_bits(bits[k])) for k, v in w.items()}
    return bits, rounded


class Model:
    """GPU context and the oracle's twin state: per layer and sequence a cache and a compressor."""

    def __init__(self, n_seqs, cap, max_tokens):
        self.cfg = mla.make_config(mla.PRESET_FASTAR_V4, n_layers=3, n_pages=n_seqs * (cap // 64 + 3) + 8, max_seqs=n_seqs,
                                   max_tokens=max_tokens)
        self.bits, self.rounded = weights_for(mla.PRESET_FASTAR_V4)
        self.ctx = mla.MlaContext(self.cfg)
        self.ocfg, self.comp = [], []
        for l, r in enumerate(RATIOS):
            self.ctx.set_layer_weights(l, self.bits)
            self.ctx.set_layer_rope(l, r != 0)
            oc = oracle_cfg(self.cfg)
            oc.rope_yarn = int(r != 0)
            self.ocfg.append(oc)
            if r:
                cb, cr = compressor_weights(self.cfg, r, 100 + l)
                self.ctx.set_layer_compressor(l, r, cb["wkv"], cb["wgate"], cb["ape"], cb["norm"])
                base = O.Compressor(oc, r, cr["wkv"], cr["wgate"], cr["ape"], cr["norm"], cap=cap // r + 2)
                self.comp.append([base] + [base.fork() for _ in range(n_seqs - 1)])
            else:
                self.comp.append(None)
        self.seqs = [self.ctx.seq_alloc() for _ in range(n_seqs)]
        self.caches = [[np.zeros((cap, 512), np.float32) for _ in range(n_seqs)] for _ in RATIOS]
        self.pos = [0] * n_seqs

    def step(self, h_bits, q_lens, causal, check=True, advance=True):
        """One model step: every layer sees the same input rows; returns the GPU outputs per layer."""
        outs = []
        hf = synth.from_bf16_bits(h_bits)
        for l, r in enumerate(RATIOS):
            got = self.ctx.forward(l, h_bits, self.seqs, self.pos, q_lens, causal=causal)
            outs.append(got.copy())
            if check:
                want = O.mla_forward_batch(self.ocfg[l], self.rounded, hf, q_lens, self.pos, self.caches[l], causal=causal,
                                           compressors=self.comp[l]).out
                check_close(got, want, f"layer {l} (ratio {r}) at positions {self.pos}", ulps=2)
        if advance:
            self.pos = [p + q for p, q in zip(self.pos, q_lens)]
        return outs


def test_compressed_rows_and_mixed_attention_against_the_oracle():
    m = Model(n_seqs=3, cap=400, max_tokens=96)
    with m.ctx:
        rng = np.random.default_rng(1)
        # prefill: causal chunks, ragged (a chunk may end inside a ratio window), 262 .. 290 rows
        for q_lens in ([32, 17, 5], [32, 32, 32], [30, 32, 31], [32, 32, 32], [32, 31, 32], [32, 32, 32],
                       [32, 32, 32], [32, 32, 32], [8, 22, 32]):
            h = synth.to_bf16_bits(rng.standard_normal((sum(q_lens), 4096)).astype(np.float32))
            m.step(h, q_lens, causal=True)
        assert m.pos == [262, 262, 260]
        # decode: one row per sequence, across ratio-4 boundaries
        for _ in range(7):
            h = synth.to_bf16_bits(rng.standard_normal((3, 4096)).astype(np.float32))
            m.step(h, [1, 1, 1], causal=False)
        # the compressed rows themselves: E4M3 grid values times a power of two -- equal up to the
        # occasional neighbouring grid value where a pooled value sits on a rounding boundary
        for l, r in enumerate(RATIOS):
            for b, s in enumerate(m.seqs):
                got = m.ctx.cmp_read(l, s)
                if not r:
                    assert got.shape[0] == 0
                    continue
                want = m.comp[l][b].rows_out()
                assert got.shape[0] == want.shape[0] == m.pos[b] // r and got.shape[0] > 0
                g = synth.from_bf16_bits(got)
                assert cosine(g, want) >= 0.9995, (l, b, cosine(g, want))
                assert np.mean(g[:, :448] == want[:, :448]) > 0.97, (l, b)
                assert np.max(np.abs(g[:, :448] - want[:, :448]) / (np.abs(want[:, :448]) + 1e-3)) <= 0.14
        # page accounting: raw pages + compressed-row pages + free = all
        owned = sum(len(m.ctx.block_table(s)) for s in m.seqs)
        comp_pages = sum((p // 4 + 63) // 64 for p in m.pos)
        assert owned + comp_pages + m.ctx.free_pages() == m.cfg.n_pages


def test_a_rejected_speculative_block_is_undone():
    """Snapshot, a causal 8-row verify block, truncate back: the same block again gives the same bits
    (the compressor's window state came back with the snapshot, reference 6149-6152), and a different
    continuation matches the oracle, which never saw the rejected rows."""
    m = Model(n_seqs=2, cap=200, max_tokens=64)
    with m.ctx:
        rng = np.random.default_rng(2)
        for q_lens in ([32, 30], [32, 32], [7, 9]):
            h = synth.to_bf16_bits(rng.standard_normal((sum(q_lens), 4096)).astype(np.float32))
            m.step(h, q_lens, causal=True)
        for s in m.seqs:
            m.ctx.seq_snapshot(s)
        hb = synth.to_bf16_bits(rng.standard_normal((16, 4096)).astype(np.float32))
        first = m.step(hb, [8, 8], causal=True, check=False, advance=False)
        for s, p in zip(m.seqs, m.pos):
            m.ctx.seq_truncate(s, p)
        again = m.step(hb, [8, 8], causal=True, check=False, advance=False)
        for a, b in zip(first, again):
            assert np.array_equal(a, b)
        for s, p in zip(m.seqs, m.pos):
            m.ctx.seq_truncate(s, p)
        h2 = synth.to_bf16_bits(rng.standard_normal((6, 4096)).astype(np.float32))
        m.step(h2, [3, 3], causal=True)  # checked against the oracle
        # a call that does not continue where the compressor stands is refused
        with pytest.raises(mla.MlaError) as e:
            m.ctx.forward(1, h2, m.seqs, [p + 5 for p in m.pos], [3, 3], causal=True)
        assert e.value.code == mla.ERR_STATE and "compressor" in str(e.value)
