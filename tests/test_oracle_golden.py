"""The CPU oracle against outputs of the reference's own functions (tests/golden/)."""
import math

import numpy as np

from oracle import oracle as O


def test_f2bf_truncation_matches_reference(golden):
    # reference f2bf (src/fst_engine.cpp:27) truncates; the oracle exposes that as bf16_trunc
    x = golden["cc_f2bf_in"]
    got = np.array([O.lib().fst_oracle_bf16_trunc(float(v)) for v in x], np.float32)
    want = O.from_bf16_bits(golden["cc_f2bf_out"])
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_bf16_round_is_within_one_ulp_of_truncation(golden):
    x = golden["cc_f2bf_in"][:64]
    r = O.to_bf16_bits(x).astype(np.int64)
    t = golden["cc_f2bf_out"][:64].astype(np.int64)
    assert np.all((r - t >= 0) & (r - t <= 1))
    assert np.array_equal(O.bf16_round(x), np.array([O.lib().fst_oracle_bf16_round(float(v)) for v in x], np.float32))


def test_rmsnorm_matches_rms_cpu(golden):
    # rms_cpu (src/fst_engine.cpp:89-91): same fp32 formula, truncating store
    for d in (512, 1024):
        x = O.from_bf16_bits(golden[f"cc_rms{d}_x"])
        w = O.from_bf16_bits(golden[f"cc_rms{d}_w"])
        want = O.from_bf16_bits(golden[f"cc_rms{d}_out"])
        got = O.rmsnorm(x, w)
        # before the store the two agree to fp32 rounding; after it to one bf16 ulp
        assert np.max(np.abs(got - want) / np.abs(got).clip(1e-6)) < 2.0 ** -7
        tr = np.array([O.lib().fst_oracle_bf16_trunc(float(v)) for v in got.ravel()], np.float32)
        mism = np.mean(tr.view(np.uint32) != want.ravel().view(np.uint32))
        assert mism < 0.01  # a value that sits on a bf16 boundary may fall either way


def test_rmsnorm_matches_benchmark_host_op(golden):
    x = O.bf16_round(golden["lb_rms_x"])
    w = O.bf16_round(golden["lb_rms_w"])
    got = O.rmsnorm(x, w, round_bf16=True)
    want = golden["lb_rms_out"]
    assert np.max(np.abs(got - want)) <= 2.0 ** -7 * np.max(np.abs(want))
    assert np.mean(got != want) < 0.02


def test_rope_lut_matches_build_rope_lut(golden):
    for name, yarn in (("plain", False), ("yarn", True)):
        for inv in (False, True):
            ref = golden[f"cc_lut_{name}_{'inv' if inv else 'fwd'}"]  # [n_pos, 2, 64] bf16 bits
            for i, p in enumerate(golden["cc_lut_pos"]):
                for m in range(2):
                    got = O.rope_lut(int(p) + m, 64, 10000.0, yarn, inv, round_lut_bf16=True)
                    want = O.from_bf16_bits(ref[i, m])
                    assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (name, inv, p, m)


def test_rope_angles_match_hf_tables(golden):
    # the engine accumulates theta by repeated fp32 multiplication, the HF table multiplies
    # pos by 1/base^(2j/d): equal up to fp32 rounding of the angle
    pos = golden["hf_rope_pos"]
    for name, yarn in (("plain", False), ("yarn", True)):
        for i, p in enumerate(pos):
            lut = O.rope_lut(int(p), 64, 10000.0, yarn)
            tol = 1e-5 + 4e-7 * float(p)
            assert np.max(np.abs(lut[0::2] - golden[f"hf_rope_{name}_cos"][i])) < tol
            assert np.max(np.abs(lut[1::2] - golden[f"hf_rope_{name}_sin"][i])) < tol


def test_rope_apply_matches_apply_rotary_emb(golden):
    x = golden["hf_rot_x"]
    p0 = int(golden["hf_rot_p0"])
    for key, inv in (("hf_rot_fwd", False), ("hf_rot_inv", True)):
        want = golden[key]
        for s in range(x.shape[1]):
            for h in range(x.shape[2]):
                got = O.rope_apply(x[0, s, h], p0 + s, inverse=inv)
                assert np.max(np.abs(got - want[0, s, h])) < 2e-5


def test_rope_inverse_undoes_forward():
    rng = np.random.default_rng(1)
    x = rng.standard_normal(64).astype(np.float32)
    for p in (0, 3, 4095, 100000):
        y = O.rope_apply(O.rope_apply(x, p), p, inverse=True)
        assert np.max(np.abs(y - x)) < 1e-5


def test_sink_softmax_matches_benchmark_host_op(golden):
    # host_softmax (scripts/fst_layer_benchmark.py:25-31) == attention weights with a sink
    sc = O.bf16_round(golden["lb_sm_scores"])
    sk = O.bf16_round(golden["lb_sm_sinks"])
    want = golden["lb_sm_out"]
    n, L = sc.shape
    # attention over an identity "cache" returns the probabilities themselves
    cfg = O.make_cfg(O.PRESET_FASTAR_V4, n_heads=n, kv_lora=L, qk_rope=0, round_bf16=True,
                     softmax_scale=1.0 / math.sqrt(512.0))
    q = sc.copy()  # q . e_s = score_s
    cache = np.eye(L, dtype=np.float32)
    got = O.attention(cfg, q, cache, L, 1, sinks=sk)
    assert np.max(np.abs(got - want)) <= 2.0 ** -8
    assert np.mean(got != want) < 0.05


def test_attention_matches_sparse_attn(golden):
    q, kv, sink = golden["hf_attn_q"], golden["hf_attn_kv"], golden["hf_attn_sink"]
    want = golden["hf_attn_out"]  # [1, nq, H, 512]
    nq, H, L = q.shape[1], q.shape[2], kv.shape[1]
    cfg = O.make_cfg(O.PRESET_FASTAR_V4, n_heads=H, round_bf16=False)
    got = O.attention(cfg, q.reshape(nq * H, 512), kv[0], L, nq, pos0=L - nq, causal=True, sinks=sink)
    assert np.max(np.abs(got.reshape(want.shape) - want)) < 2e-5
    # and the split-KV form merges to the same thing
    parts = [O.attention_partial(cfg, q.reshape(nq * H, 512), kv[0], a, b, nq, L - nq, True)
             for a, b in ((0, 10), (10, 11), (11, 37))]
    m = np.stack([p[0] for p in parts])
    l = np.stack([p[1] for p in parts])
    o = np.stack([p[2] for p in parts])
    merged = O.merge_partials(cfg, m, l, o, sinks=sink)
    assert np.max(np.abs(merged.reshape(want.shape) - want)) < 2e-5


def test_attn_norm_is_rmsnorm_in_front_of_the_layer():
    """The oracle with an attn_norm weight equals the oracle fed with rms_cpu-normed rows
    (process_layer calls npu_rmsnorm_weighted and then process_mla, src/fst_engine.cpp:2687-2689)."""
    cfg = O.make_cfg(O.PRESET_BASELINE, hidden=256, n_heads=4, q_lora=64, kv_lora=64, qk_nope=32, qk_rope=16,
                     v_head=32, round_bf16=True)
    rng = np.random.default_rng(7)
    d = O.dims_of(cfg) if hasattr(O, "dims_of") else None
    shapes = {"wq_a": (64, 256), "wq_b": (4 * 48, 64), "wkv_a": (80, 256), "wkv_b": (4 * 64, 64),
              "wo_b": (256, 4 * 32), "q_norm": (64,), "kv_norm": (64,)}
    w = {k: O.bf16_round((rng.standard_normal(s) * (1.0 if "norm" in k else 0.05)).astype(np.float32)) for k, s in shapes.items()}
    g = O.bf16_round((1.0 + 0.2 * rng.standard_normal(256)).astype(np.float32))
    h = O.bf16_round((3.0 * rng.standard_normal((3, 256))).astype(np.float32))
    cache_a = np.zeros((8, 80), np.float32)
    cache_b = np.zeros((8, 80), np.float32)
    fused = O.mla_forward(cfg, dict(w, attn_norm=g), h, 0, cache_a, causal=True)
    normed = O.rmsnorm(h, g, round_bf16=True)
    plain = O.mla_forward(cfg, w, normed, 0, cache_b, causal=True)
    assert np.array_equal(fused.out.view(np.uint32), plain.out.view(np.uint32))
    assert np.array_equal(cache_a.view(np.uint32), cache_b.view(np.uint32))
    assert not np.array_equal(fused.out, O.mla_forward(cfg, w, h, 0, np.zeros((8, 80), np.float32), causal=True).out)


def test_window_attention_is_attention_over_the_last_rows():
    """attention_window: a window that covers everything equals attention(); a shorter one equals
    attention() over a cache cut to the window's rows (softmax does not care where the rows sit).
    Outputs are bf16-rounded and the partial + merge route rounds P against a per-slice maximum, so
    the two may differ by one bf16 step (values here are below 4: 2^-6 = 1.6e-2)."""
    cfg = O.make_cfg(O.PRESET_BASELINE)
    rng = np.random.default_rng(5)
    H, L = cfg.n_heads, 300
    cache = O.bf16_round(rng.standard_normal((L, 576)).astype(np.float32))
    q = O.bf16_round(rng.standard_normal((H, 576)).astype(np.float32))
    full = O.attention(cfg, q, cache, L, 1)
    assert np.allclose(O.attention_window(cfg, q, cache, L, 1, 0), full, atol=1.6e-2)
    assert np.allclose(O.attention_window(cfg, q, cache, L, 1, 4096), full, atol=1.6e-2)
    for W in (1, 63, 64, 100, 299):
        cut = np.ascontiguousarray(cache[L - W:])
        assert np.allclose(O.attention_window(cfg, q, cache, L, 1, W), O.attention(cfg, q, cut, W, 1), atol=1.6e-2), W


# ---- the V4 layer and its KV compressor against the reference's own Python (tests/golden/make_golden_v4.py) ----
import os  # noqa: E402

import pytest  # noqa: E402

_V4 = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_v4_layer.npz")
GEOM = dict(hidden=128, n_heads=4, q_lora=64, kv_lora=192, qk_rope=64, o_groups=2, o_lora=32)


@pytest.fixture(scope="module")
def v4():
    return np.load(_V4)


def _layer_weights(v4, tag):
    g = lambda n: v4[f"{tag}_w_{n}"]  # noqa: E731
    return {"wq_a": g("attn.wq_a.weight"), "wq_b": g("attn.wq_b.weight"), "wkv_a": g("attn.wkv.weight"),
            "wo_a": g("attn.wo_a.weight"), "wo_b": g("attn.wo_b.weight"), "q_norm": g("attn.q_norm.weight"),
            "kv_norm": g("attn.kv_norm.weight"), "attn_sinks": g("attn.attn_sink")}


def _compressor(cfg, v4, tag, ratio, **kw):
    g = lambda n: v4[f"{tag}_w_attn.compressor.{n}"]  # noqa: E731
    return O.Compressor(cfg, ratio, g("wkv.weight"), g("wgate.weight"), g("ape"), g("norm.weight"), **kw)


def test_e4m3_round_trip_is_the_fp8_cast():
    # e4m3_roundtrip (src/fst_engine.cpp:3084-3100) == a cast to float8_e4m3fn and back, ties to even
    import torch
    rng = np.random.default_rng(3)
    x = np.concatenate([rng.uniform(-448, 448, 4000), rng.standard_normal(2000) * 0.01, [0.0, 448.0, -448.0, 500.0],
                        np.arange(0, 16, 0.0625)]).astype(np.float32)
    want = torch.from_numpy(np.clip(x, -448, 448)).to(torch.float8_e4m3fn).to(torch.float32).numpy()
    got = np.array([O.e4m3_roundtrip(v) for v in x], np.float32)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("tag,ratio", [("cmp4", 4), ("cmp128", 128)])
def test_compressor_matches_the_reference_compressor(v4, tag, ratio):
    """compress_token (src/fst_engine.cpp:3171-3318) streamed token by token == the HF model's
    Compressor.forward (scripts/hf_gen_ref.py:266-353) on the same rows, with the score state started
    at -inf as that model starts it.  Nope values are E4M3 grid values times a power of two: equal
    up to an occasional neighbouring grid value where the pooled value sits on a rounding boundary."""
    cfg = O.make_cfg(O.PRESET_FASTAR_V4, round_bf16=False, rope_yarn=True, **GEOM)
    comp = _compressor(cfg, v4, tag, ratio, score_init=-np.inf)
    x = v4[f"{tag}_x"]
    emitted = [comp.push(cfg, x[t], t) for t in range(x.shape[0])]
    assert emitted == [1 if (t + 1) % ratio == 0 else 0 for t in range(x.shape[0])]
    got, want = comp.rows_out(), v4[f"{tag}_rows"]
    assert got.shape == want.shape and got.shape[0] == x.shape[0] // ratio
    nope = slice(0, 128)
    same = np.isclose(got[:, nope], want[:, nope], rtol=0, atol=0)
    assert same.mean() > 0.995
    assert np.max(np.abs(got[:, nope] - want[:, nope]) / (np.abs(want[:, nope]) + 1e-6)) <= 0.13  # one grid step
    # the rotated tail: fp32 there, rounded to bf16 here
    assert np.max(np.abs(got[:, 128:] - want[:, 128:])) <= 2.0 ** -8 * np.max(np.abs(want[:, 128:])) + 1e-6


def test_engine_starts_the_compressor_state_at_zero(v4):
    """reset_compressor_state (3160-3169) zeroes the states, so the empty lane of the very first
    ratio-4 window takes part in the pool with score 0 and value 0: the first row differs from the
    HF model's, later rows do not."""
    cfg = O.make_cfg(O.PRESET_FASTAR_V4, round_bf16=False, rope_yarn=True, **GEOM)
    x = v4["cmp4_x"]
    a, b = _compressor(cfg, v4, "cmp4", 4, score_init=0.0), _compressor(cfg, v4, "cmp4", 4, score_init=-np.inf)
    for t in range(12):
        a.push(cfg, x[t], t)
        b.push(cfg, x[t], t)
    assert not np.allclose(a.rows_out()[0], b.rows_out()[0])
    assert np.array_equal(a.rows_out()[1:], b.rows_out()[1:])


def test_v4_layer_composition_matches_layer_attn_forward(v4):
    """The whole V4 attention layer -- head layout [M, 64, 512], per-head q norm before RoPE, sink
    in the softmax, inverse RoPE on the output tail, grouped wo_a -- against LayerAttn.forward
    (scripts/hf_gen_ref.py:389-467): a causal prefill of 11 rows, then two decode steps."""
    cfg = O.make_cfg(O.PRESET_FASTAR_V4, round_bf16=False, rope_yarn=False, **GEOM)
    w = _layer_weights(v4, "layer0")
    x, want = v4["layer0_x"], v4["layer0_out"]
    cache = np.zeros((x.shape[0], 192), np.float32)
    for start, n in v4["layer0_plan"]:
        got = O.mla_forward(cfg, w, x[start:start + n], int(start), cache, causal=n > 1, want_trace=False).out
        ref = want[start:start + n]
        assert np.max(np.abs(got - ref)) <= 2e-4 * np.max(np.abs(ref)), (start, n)


def test_v4_layer_with_compressor_matches_layer_attn_forward(v4):
    """A ratio-4 layer (YaRN tables) decoded token by token from position 0: the compressed rows join
    the attention as extra columns (src/fst_engine.cpp:3565-3586), as LayerAttn.forward does it."""
    cfg = O.make_cfg(O.PRESET_FASTAR_V4, round_bf16=False, rope_yarn=True, **GEOM)
    w = _layer_weights(v4, "layer2")
    comp = _compressor(cfg, v4, "layer2", 4, score_init=-np.inf)
    x, want = v4["layer2_x"], v4["layer2_out"]
    cache = np.zeros((x.shape[0], 192), np.float32)
    for t in range(x.shape[0]):
        got = O.mla_forward_batch(cfg, w, x[t:t + 1], [1], [t], [cache], compressors=[comp]).out
        assert np.max(np.abs(got - want[t:t + 1])) <= 5e-3 * np.max(np.abs(want[t:t + 1])), t
    assert comp.n_comp == x.shape[0] // 4
    assert np.max(np.abs(comp.rows_out() - v4["layer2_cmp_rows"])) <= 0.13 * np.max(np.abs(v4["layer2_cmp_rows"]))
