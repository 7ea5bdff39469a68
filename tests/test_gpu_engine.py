"""The C++ host class FSTEngine (fastar_b200/host) driven the way the reference drives it:
prefill in 16-token chunks with is_prefill_ set (prefill_tiled, src/fst_engine.cpp:2957-2984),
then single-token decode steps (6251-6262), rollback of rejected speculative rows (6132-6147),
reset_session (2992-3012) and the random-matrix GEMM probe (586-685)."""
import ctypes as C
import os

import numpy as np
import pytest

from fastar_b200 import mla, synth
from oracle import oracle as O
from tests.helpers import check_close, oracle_cfg
from tests.test_gpu_layer import weights_for

pytestmark = pytest.mark.gpu

LIB = os.path.join(os.path.dirname(mla.LIB_PATH), "libfst_engine.so")


def load():
    L = C.CDLL(LIB)
    L.fst_engine_create.restype = C.c_void_p
    L.fst_engine_create.argtypes = [C.c_int] * 8
    L.fst_engine_destroy.argtypes = [C.c_void_p]
    L.fst_engine_last_error.restype = C.c_char_p
    L.fst_engine_set_weight.argtypes = [C.c_void_p, C.c_int, C.c_char_p, C.POINTER(C.c_uint16), C.c_size_t]
    L.fst_engine_set_sinks.argtypes = [C.c_void_p, C.c_int, C.POINTER(C.c_float), C.c_size_t]
    L.fst_engine_preload.argtypes = [C.c_void_p]
    L.fst_engine_process_mla.argtypes = [C.c_void_p, C.c_int, C.POINTER(C.c_uint16), C.c_int]
    L.fst_engine_reset_session.argtypes = [C.c_void_p]
    L.fst_engine_seq_pos.argtypes = [C.c_void_p]
    L.fst_engine_advance.argtypes = [C.c_void_p, C.c_int]
    L.fst_engine_set_prefill.argtypes = [C.c_void_p, C.c_int]
    L.fst_engine_rollback.argtypes = [C.c_void_p, C.c_int]
    L.fst_engine_set_window.argtypes = [C.c_void_p, C.c_int]
    L.fst_engine_randmat_test.argtypes = [C.c_void_p] + [C.POINTER(C.c_double)] * 3 + [C.c_int]
    return L


def make_engine(L, preset, max_seq=128):
    e = L.fst_engine_create(preset, 1, max_seq, 1, 16, 0, mla.IMPL_AUTO, mla.IMPL_AUTO)
    assert e, L.fst_engine_last_error()
    bits, rounded = weights_for(preset)
    for name, a in bits.items():
        if name == "attn_sinks":
            a = np.ascontiguousarray(a, np.float32)
            assert L.fst_engine_set_sinks(e, 0, a.ctypes.data_as(C.POINTER(C.c_float)), a.size) == 0
        else:
            a = np.ascontiguousarray(a, np.uint16)
            assert L.fst_engine_set_weight(e, 0, name.encode(), a.ctypes.data_as(C.POINTER(C.c_uint16)), a.size) == 0
    assert L.fst_engine_preload(e) == 0, L.fst_engine_last_error()
    return e, rounded


def process(L, e, h_bits):
    buf = np.ascontiguousarray(h_bits, np.uint16).copy()
    rc = L.fst_engine_process_mla(e, 0, buf.ctypes.data_as(C.POINTER(C.c_uint16)), buf.shape[0])
    assert rc == 0, L.fst_engine_last_error()
    return buf  # overwritten in place, as the reference does (3889)


@pytest.mark.parametrize("preset", [mla.PRESET_FASTAR_V4, mla.PRESET_BASELINE], ids=["v4", "baseline"])
def test_prefill_then_decode_like_the_engine(preset):
    L = load()
    e, rounded = make_engine(L, preset)
    try:
        cfg = mla.make_config(preset)
        ocfg = oracle_cfg(cfg)
        cache = np.zeros((128, mla.dims_of(cfg)["row"]), np.float32)
        ulps = 2 if preset == mla.PRESET_FASTAR_V4 else 0
        # prefill: two chunks (16 + 5 rows), causal inside each chunk
        L.fst_engine_set_prefill(e, 1)
        for step, M in enumerate((16, 5)):
            h = synth.to_bf16_bits(synth.hidden_f32(cfg, 7, M, (step,)))
            pos = L.fst_engine_seq_pos(e)
            got = process(L, e, h)
            want = O.mla_forward(ocfg, rounded, synth.from_bf16_bits(h), pos, cache, causal=True, want_trace=False).out
            check_close(got, want, f"prefill chunk {step}", ulps=ulps)
            L.fst_engine_advance(e, M)
        # decode: one row at a time, no mask
        L.fst_engine_set_prefill(e, 0)
        for step in range(3):
            h = synth.to_bf16_bits(synth.hidden_f32(cfg, 8, 1, (step,)))
            pos = L.fst_engine_seq_pos(e)
            got = process(L, e, h)
            want = O.mla_forward(ocfg, rounded, synth.from_bf16_bits(h), pos, cache, causal=False, want_trace=False).out
            check_close(got, want, f"decode step {step}", ulps=ulps)
            L.fst_engine_advance(e, 1)
        assert L.fst_engine_seq_pos(e) == 24
        # speculative verify of 4 rows, 2 rejected: roll back, then decode again from the kept length
        L.fst_engine_set_prefill(e, 1)
        h = synth.to_bf16_bits(synth.hidden_f32(cfg, 9, 4))
        process(L, e, h)
        O.mla_forward(ocfg, rounded, synth.from_bf16_bits(h), 24, cache, causal=True, want_trace=False)
        assert L.fst_engine_rollback(e, 26) == 0
        cache[26:] = 0  # the reference zeroes the rejected rows
        L.fst_engine_set_prefill(e, 0)
        h = synth.to_bf16_bits(synth.hidden_f32(cfg, 10, 1))
        got = process(L, e, h)
        want = O.mla_forward(ocfg, rounded, synth.from_bf16_bits(h), 26, cache, causal=False, want_trace=False).out
        check_close(got, want, "decode after rollback", ulps=ulps)
        # a window that covers the whole context changes nothing; a negative one is an error
        assert L.fst_engine_set_window(e, 4096) == 0
        check_close(process(L, e, h), want, "window over the whole context", ulps=ulps)
        assert L.fst_engine_set_window(e, -1) != 0
        assert L.fst_engine_set_window(e, 0) == 0
        # the reference asserts seq_pos_ + M <= max_seq: here it is an error, not a crash
        L.fst_engine_advance(e, 128)
        buf = np.zeros((1, 4096), np.uint16)
        assert L.fst_engine_process_mla(e, 0, buf.ctypes.data_as(C.POINTER(C.c_uint16)), 1) != 0
        assert b"max_seq" in L.fst_engine_last_error()
        # a new session starts from an empty, zeroed cache
        assert L.fst_engine_reset_session(e) == 0
        assert L.fst_engine_seq_pos(e) == 0
        cache[:] = 0
        L.fst_engine_set_prefill(e, 1)
        h = synth.to_bf16_bits(synth.hidden_f32(cfg, 11, 3))
        got = process(L, e, h)
        want = O.mla_forward(ocfg, rounded, synth.from_bf16_bits(h), 0, cache, causal=True, want_trace=False).out
        check_close(got, want, "first chunk of a new session", ulps=ulps)
    finally:
        L.fst_engine_destroy(e)


def test_randmat_probe_passes_the_reference_gate():
    L = load()
    e = L.fst_engine_create(mla.PRESET_FASTAR_V4, 1, 128, 1, 16, 0, 0, 0)
    assert e, L.fst_engine_last_error()
    try:
        cos = (C.c_double * 8)()
        ratio = (C.c_double * 8)()
        err = (C.c_double * 8)()
        n = L.fst_engine_randmat_test(e, cos, ratio, err, 8)
        assert n == 6, L.fst_engine_last_error()
        for i in range(n):
            # the reference's gate: cos >= 0.999, |npu|/|ref| ~ 1 (src/fst_engine.cpp:582-585)
            assert cos[i] >= 0.99999 and abs(ratio[i] - 1) < 1e-3
    finally:
        L.fst_engine_destroy(e)


def _write_fst(path, n_layers, tensors):
    """A `.fst` file in the reference's layout (scripts/fst_converter.py:173-176, 685-716, 1464-1500):
    128-byte header, 64-byte directory entries, page-aligned payloads.  tensors: (tid, layer, sub,
    qtype, ndarray) with BF16 payloads given as uint16 bits and F32 as float32."""
    import struct
    page = lambda x: (x + 4095) & ~4095  # noqa: E731
    dir_off = page(128)
    off = page(dir_off + 64 * len(tensors))
    entries = []
    with open(path, "wb") as f:
        for tid, layer, sub, qtype, a in tensors:
            shape = (tuple(a.shape) + (1, 1, 1))[:3]
            f.seek(off)
            f.write(a.tobytes())
            entries.append(struct.pack("<IHHHHIQQQQQQ", tid, layer, sub, qtype, a.ndim, 0, *shape, off, a.nbytes, 0))
            off = page(off + a.nbytes)
        f.seek(dir_off)
        f.write(b"".join(entries))
        f.seek(0)
        f.write(struct.pack("<4sIIIIIIIIIIIQffQQQQQQQQ", b"FST\x00", 2, 4096, n_layers, 0, 8, 64, 1, 512, 0, 1, 0, 1000,
                            1e-6, 10000.0, dir_off, len(tensors), off, 0, 0, 0, 0, 0))
        f.truncate(off)


def test_weights_loaded_from_a_fst_file(tmp_path):
    """FSTEngine::load_shared_weights / load_norm_override (src/fst_engine.cpp:1503-1642, 1873-1900): an
    engine that read its MLA tensors from a `.fst` file (norms and sinks from the sidecar) computes the
    same bits as one that was handed the same arrays; a file whose tensors do not fit is an error."""
    L = load()
    L.fst_engine_load_shared_weights.argtypes = [C.c_void_p, C.c_char_p]
    L.fst_engine_load_norm_override.argtypes = [C.c_void_p, C.c_char_p]
    bits, _ = weights_for(mla.PRESET_FASTAR_V4)
    tid = {"wq_a": (5, 0), "wq_b": (5, 1), "wkv_a": (6, 0), "wo_a": (8, 0), "wo_b": (8, 1), "q_norm": (14, 0),
           "kv_norm": (15, 0)}
    main = [(t, 0, s, 2, np.ascontiguousarray(bits[n], np.uint16)) for n, (t, s) in tid.items()]
    # the main file carries norms that the sidecar must replace, and no sinks
    main[-2] = (14, 0, 0, 2, np.full_like(bits["q_norm"], 0x3C00))
    main[-1] = (15, 0, 0, 2, np.full_like(bits["kv_norm"], 0x3C00))
    side = [(14, 0, 0, 2, np.ascontiguousarray(bits["q_norm"], np.uint16)),
            (15, 0, 0, 2, np.ascontiguousarray(bits["kv_norm"], np.uint16)),
            (22, 0, 0, 3, np.ascontiguousarray(bits["attn_sinks"], np.float32))]
    p_main, p_side = str(tmp_path / "m.fst"), str(tmp_path / "m.fst.norm")
    _write_fst(p_main, 1, main)
    _write_fst(p_side, 1, side)
    e_ref, _ = make_engine(L, mla.PRESET_FASTAR_V4)
    e = L.fst_engine_create(mla.PRESET_FASTAR_V4, 1, 128, 1, 16, 0, mla.IMPL_AUTO, mla.IMPL_AUTO)
    try:
        assert L.fst_engine_load_shared_weights(e, p_main.encode()) == 0, L.fst_engine_last_error()
        assert L.fst_engine_load_norm_override(e, p_side.encode()) == 0, L.fst_engine_last_error()
        assert L.fst_engine_preload(e) == 0, L.fst_engine_last_error()
        cfg = mla.make_config(mla.PRESET_FASTAR_V4)
        h = synth.to_bf16_bits(synth.hidden_f32(cfg, 21, 5))
        L.fst_engine_set_prefill(e, 1)
        L.fst_engine_set_prefill(e_ref, 1)
        assert np.array_equal(process(L, e, h), process(L, e_ref, h))
        # a file of another model size is refused, with the tensor named
        golden = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "tiny_mla.fst")
        assert L.fst_engine_load_shared_weights(e, golden.encode()) != 0
        assert b"configuration wants" in L.fst_engine_last_error()
    finally:
        L.fst_engine_destroy(e)
        L.fst_engine_destroy(e_ref)


@pytest.mark.parametrize("with_compressor", [False, True], ids=["plain", "compressor"])
def test_rope_kind_follows_each_layers_compress_ratio(tmp_path, with_compressor):
    """build_rope_lut chooses per layer (src/fst_engine.cpp:1979-1982): plain RoPE with the file's
    rope_freq_base for layers whose compress ratio is 0, YaRN for the others.  A three-layer engine
    reads ratios {0, 0, 4} (TID 40) and a non-default base from a file written in the converter's
    other form (wq_a / wq_b and wo_a / wo_b under one tensor id AND sub id 0, found by shape as the
    engine finds them, 1610-1615); every layer is prefilled in 15-row chunks -- rows 60..74 straddle
    a page boundary -- and compared with the oracle that uses that layer's RoPE kind.  With the
    compressor switched on (the reference gates it behind FST_COMPRESSOR, 3565) layer 2 also reads
    its compressor tensors (TIDs 32-35, 1657-1690) and attends to its compressed rows."""
    import struct
    L = load()
    L.fst_engine_load_shared_weights.argtypes = [C.c_void_p, C.c_char_p]
    bits, rounded = weights_for(mla.PRESET_FASTAR_V4)
    theta = 50000.0
    tensors = []
    for l in range(3):
        tensors += [(5, l, 0, 2, bits["wq_a"]), (5, l, 0, 2, bits["wq_b"]), (6, l, 0, 2, bits["wkv_a"]),
                    (8, l, 0, 2, bits["wo_a"]), (8, l, 0, 2, bits["wo_b"]), (14, l, 0, 2, bits["q_norm"]),
                    (15, l, 0, 2, bits["kv_norm"]), (22, l, 0, 3, np.ascontiguousarray(bits["attn_sinks"], np.float32))]
    tensors.append((40, 0xFFFF, 0, 3, np.array([0.0, 0.0, 4.0], np.float32)))
    cfg = mla.make_config(mla.PRESET_FASTAR_V4)
    comp = None
    if with_compressor:
        from tests.test_gpu_compressor import compressor_weights
        cb, cr = compressor_weights(cfg, 4, 77)
        tensors += [(32, 2, 0, 3, cb["ape"]), (33, 2, 0, 2, cb["wkv"]), (34, 2, 0, 2, cb["wgate"]), (35, 2, 0, 2, cb["norm"])]
    path = str(tmp_path / "three.fst")
    _write_fst(path, 3, [(t, l, s, q, np.ascontiguousarray(a)) for t, l, s, q, a in tensors])
    with open(path, "r+b") as f:  # the header's rope_freq_base
        f.seek(struct.calcsize("<4sIIIIIIIIIIIQf"))
        f.write(struct.pack("<f", theta))
    e = L.fst_engine_create(mla.PRESET_FASTAR_V4, 3, 128, 1, 16, 0, mla.IMPL_AUTO, mla.IMPL_AUTO)
    assert e, L.fst_engine_last_error()
    try:
        L.fst_engine_enable_compressor.argtypes = [C.c_void_p, C.c_int]
        L.fst_engine_layer_cmp_ratio.argtypes = [C.c_void_p, C.c_int]
        L.fst_engine_enable_compressor(e, int(with_compressor))
        assert L.fst_engine_load_shared_weights(e, path.encode()) == 0, L.fst_engine_last_error()
        assert L.fst_engine_preload(e) == 0, L.fst_engine_last_error()
        assert [L.fst_engine_layer_cmp_ratio(e, l) for l in range(3)] == [0, 0, 4]
        caches = [np.zeros((128, 512), np.float32) for _ in range(3)]
        ocfgs = []
        for l in range(3):
            oc = oracle_cfg(cfg)
            oc.rope_yarn = 1 if l == 2 else 0
            oc.rope_theta = theta
            ocfgs.append(oc)
        if with_compressor:
            comp = O.Compressor(ocfgs[2], 4, cr["wkv"], cr["wgate"], cr["ape"], cr["norm"], cap=40)
        L.fst_engine_set_prefill(e, 1)
        outs = {}
        for chunk in range(5):
            pos = L.fst_engine_seq_pos(e)
            assert pos == 15 * chunk
            h = synth.to_bf16_bits(synth.hidden_f32(cfg, 31, 15, (chunk,)))
            for l in range(3):
                buf = np.ascontiguousarray(h, np.uint16).copy()
                rc = L.fst_engine_process_mla(e, l, buf.ctypes.data_as(C.POINTER(C.c_uint16)), 15)
                assert rc == 0, L.fst_engine_last_error()
                want = O.mla_forward_batch(ocfgs[l], rounded, synth.from_bf16_bits(h), [15], [pos], [caches[l]], causal=True,
                                           compressors=[comp] if (comp is not None and l == 2) else None).out
                check_close(buf, want, f"chunk {chunk} layer {l}", ulps=2)
                outs[chunk, l] = buf
            L.fst_engine_advance(e, 15)
        # same weights, same rows: the layers differ only by their RoPE kind, and layer 2 must differ
        assert np.array_equal(outs[4, 0], outs[4, 1])
        assert not np.array_equal(outs[4, 0], outs[4, 2])
    finally:
        L.fst_engine_destroy(e)


@pytest.mark.parametrize("window", [128, 8], ids=["inside-the-window", "window-slides"])
def test_draft_model_attention(window):
    """process_draft_mla (src/fst_engine.cpp:4884-5131): the projected main hidden row becomes the KV
    row at the anchor; a block of candidates at anchor+1 .. attends densely to the last window_size
    main rows and to itself, with no per-head q norm and the q / output rotation on head 0 only; the
    block's own rows are dropped again.  Against the oracle, anchor after anchor, with a window that
    never fills (the reference's own regime) and one that slides."""
    L = load()
    L.fst_engine_set_draft.argtypes = [C.c_void_p, C.c_int]
    L.fst_engine_process_draft_mla.argtypes = [C.c_void_p, C.c_int, C.POINTER(C.c_uint16), C.c_int, C.POINTER(C.c_uint16)]
    e = L.fst_engine_create(mla.PRESET_FASTAR_V4, 1, 128, 1, 16, 0, mla.IMPL_AUTO, mla.IMPL_AUTO)
    assert e, L.fst_engine_last_error()
    try:
        L.fst_engine_set_draft(e, window)
        bits, rounded = weights_for(mla.PRESET_FASTAR_V4)
        for name, a in bits.items():
            if name == "attn_sinks":
                a = np.ascontiguousarray(a, np.float32)
                assert L.fst_engine_set_sinks(e, 0, a.ctypes.data_as(C.POINTER(C.c_float)), a.size) == 0
            else:
                a = np.ascontiguousarray(a, np.uint16)
                assert L.fst_engine_set_weight(e, 0, name.encode(), a.ctypes.data_as(C.POINTER(C.c_uint16)), a.size) == 0
        assert L.fst_engine_preload(e) == 0, L.fst_engine_last_error()
        cfg = mla.make_config(mla.PRESET_FASTAR_V4)
        main_cfg = oracle_cfg(cfg)                      # the KV side is the main layer's
        draft_cfg = oracle_cfg(cfg)
        draft_cfg.draft_form = 1
        cache = np.zeros((128, 512), np.float32)
        rng = np.random.default_rng(9)
        M = 5
        for anchor in range(14):
            assert L.fst_engine_seq_pos(e) == anchor
            main_x = synth.to_bf16_bits(rng.standard_normal((1, 4096)).astype(np.float32))
            h = synth.to_bf16_bits(rng.standard_normal((M, 4096)).astype(np.float32))
            buf = h.copy()
            rc = L.fst_engine_process_draft_mla(e, 0, buf.ctypes.data_as(C.POINTER(C.c_uint16)), M,
                                                main_x.ctypes.data_as(C.POINTER(C.c_uint16)))
            assert rc == 0, L.fst_engine_last_error()
            # oracle: the main row enters the cache at the anchor; the block sees [window ; block]
            O.mla_forward(main_cfg, rounded, synth.from_bf16_bits(main_x), anchor, cache, want_trace=False)
            scratch = cache.copy()
            draft_cfg.window = window + M if anchor + 1 > window else 0
            want = O.mla_forward(draft_cfg, rounded, synth.from_bf16_bits(h), anchor + 1, scratch, causal=False,
                                 want_trace=False).out
            check_close(buf, want, f"anchor {anchor}", ulps=2)
            L.fst_engine_advance(e, 1)
        # only the main rows stayed in the cache
        ctx = L.fst_engine_ctx
        ctx.restype = C.c_void_p
        n = C.c_int32()
        lib = mla.load_library()
        assert lib.fst_cuda_mla_seq_len(C.c_void_p(ctx(e)), 0, C.byref(n)) == 0 and n.value == 14
    finally:
        L.fst_engine_destroy(e)
