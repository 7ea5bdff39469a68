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
