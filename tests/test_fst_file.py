"""The `.fst` reader for MLA tensors (fastar_b200/fst_file.py) against fixtures written with the
reference's own converter primitives (tests/golden/make_fst_fixture.py; format and loader:
scripts/fst_converter.py:173-176, 511-546, 685-716, 1464-1500; src/fst_engine.cpp:1503-1642,
1873-1900).  The fixture's float values are seeded, so they are rebuilt here and compared."""
import os
import shutil

import numpy as np
import pytest

from fastar_b200 import fst_file as F
from fastar_b200 import mla

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
MAIN, SIDE = os.path.join(GOLD, "tiny_mla.fst"), os.path.join(GOLD, "tiny_mla.fst.norm")
N_LAYERS, HIDDEN, HEADS, Q_LORA, KV, HEAD_DIM, O_LOW = 2, 64, 4, 32, 24, 24, 48


def main_values(seed=0):
    """The generator's sequence of draws, in its order: {(layer, name): float32 array}."""
    rng = np.random.default_rng(seed)
    n = lambda *s: rng.standard_normal(s).astype(np.float32)  # noqa: E731
    out = {}
    for l in range(N_LAYERS):
        out[l, "attn_norm"] = 1.0 + 0.1 * n(HIDDEN)
        out[l, "moe_norm"] = 1.0 + 0.1 * n(HIDDEN)
        out[l, "wq_a"] = 0.05 * n(Q_LORA, HIDDEN)
        out[l, "wq_b"] = 0.05 * n(HEADS * HEAD_DIM, Q_LORA)
        out[l, "wkv_a"] = 0.05 * n(KV, HIDDEN)
        out[l, "wo_a"] = 0.05 * n(O_LOW, HEADS * HEAD_DIM // 2)
        out[l, "wo_b"] = 0.05 * n(HIDDEN, O_LOW)
        out[l, "q_norm"] = 1.0 + 0.1 * n(Q_LORA)
        out[l, "kv_norm"] = 1.0 + 0.1 * n(KV)
        out[l, "attn_sinks"] = n(HEADS)
    return out


def side_values(seed=1):
    rng = np.random.default_rng(seed)
    n = lambda *s: rng.standard_normal(s).astype(np.float32)  # noqa: E731
    out = {}
    for l in range(N_LAYERS):
        out[l, "attn_norm"] = 1.2 + 0.1 * n(HIDDEN)
        out[l, "q_norm"] = 0.9 + 0.1 * n(Q_LORA)
        out[l, "kv_norm"] = 1.1 + 0.1 * n(KV)
        out[l, "attn_sinks"] = n(HEADS)
    return out


def trunc_bits(x):
    return (np.ascontiguousarray(x, np.float32).view(np.uint32) >> 16).astype(np.uint16)


def from_bits(b):
    return (b.astype(np.uint32) << 16).view(np.float32)


def test_header_and_directory():
    h = F.read_header(MAIN)
    assert (h.version, h.hidden_dim, h.n_layers, h.n_q_heads, h.head_dim, h.vocab_size) == (2, 64, 2, 4, 24, 100)
    assert h.rope_freq_base == 10000.0 and abs(h.rms_eps - 1e-6) < 1e-12
    assert (h.dir_offset, h.dir_count) == (4096, 20)
    es = F.read_directory(MAIN)
    assert len(es) == 20 and all(e.offset % 4096 == 0 for e in es)   # page-aligned payloads
    e = F.find(es, F.TID_Q_PROJ, 1, 1)
    assert (e.layer, e.qtype, e.shape) == (1, F.QTYPE_Q8_0, (96, 32)) and e.size == 96 * 32 // 32 * 34
    assert F.find(es, 4, 0).shape == (64,) and F.find(es, 99, 0) is None


def test_bf16_and_f32_tensors_are_the_stored_bits():
    want = main_values()
    for l in range(N_LAYERS):
        w = F.load_mla_layer(MAIN, l)
        for name in ("wq_a", "wkv_a", "wo_b", "q_norm", "kv_norm", "attn_norm"):
            assert w[name].dtype == np.uint16 and np.array_equal(w[name], trunc_bits(want[l, name])), (l, name)
        assert w["attn_sinks"].dtype == np.float32 and np.array_equal(w["attn_sinks"], want[l, "attn_sinks"])
        assert "moe_norm" not in w   # TID 4 is not the attention's


def test_q8_0_tensors_expand_as_the_engine_does():
    """All fp16 scales first, then the int8 values; value * scale, truncated to bf16: within half a
    quantisation step (+ the bf16 truncation) of the float the converter was given."""
    want = main_values()
    for l in range(N_LAYERS):
        w = F.load_mla_layer(MAIN, l)
        for name in ("wq_b", "wo_a"):
            x = want[l, name]
            got = from_bits(w[name])
            assert got.shape == x.shape
            step = (np.abs(x.reshape(-1, 32)).max(axis=1) / 127.0)[:, None]
            err = np.abs(got.reshape(-1, 32) - x.reshape(-1, 32))
            assert (err <= 0.51 * step + 2.0 ** -7 * np.abs(x.reshape(-1, 32)) + 1e-7).all(), (l, name, err.max())
            assert np.corrcoef(got.ravel(), x.ravel())[0, 1] > 0.9999


def test_norm_sidecar_overrides_norms_and_sinks_only():
    main, side = main_values(), side_values()
    for l in range(N_LAYERS):
        w = F.load_mla_layer(MAIN, l, norm_path=SIDE)
        for name in ("attn_norm", "q_norm", "kv_norm"):
            assert np.array_equal(w[name], trunc_bits(side[l, name]))
        assert np.array_equal(w["attn_sinks"], side[l, "attn_sinks"])
        assert np.array_equal(w["wq_a"], trunc_bits(main[l, "wq_a"]))


def test_shapes_against_a_configuration():
    cfg = mla.make_config(mla.PRESET_FASTAR_V4, hidden=HIDDEN, n_heads=HEADS, q_lora=Q_LORA, kv_lora=KV, qk_rope=8,
                          o_groups=2, o_lora=O_LOW // 2)
    w = F.load_mla_layer(MAIN, 0)
    F.check_mla_shapes(w, mla.weight_shapes(cfg))
    bad = mla.make_config(mla.PRESET_FASTAR_V4, hidden=HIDDEN, n_heads=HEADS, q_lora=Q_LORA * 2, kv_lora=KV, qk_rope=8,
                          o_groups=2, o_lora=O_LOW // 2)
    with pytest.raises(F.FstFormatError, match="wq_a"):
        F.check_mla_shapes(w, mla.weight_shapes(bad))


def _write_fst(path, n_layers, tensors, theta=10000.0):
    """A `.fst` file in the reference's layout (scripts/fst_converter.py:173-176, 685-716, 1464-1500):
    128-byte header, 64-byte directory entries, page-aligned payloads.  tensors: (tid, layer, sub,
    qtype, ndarray), BF16 payloads as uint16 bits and F32 as float32."""
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
        f.write(struct.pack("<4sIIIIIIIIIIIQffQQQQQQQQ", b"FST\x00", 2, HIDDEN, n_layers, 0, 8, HEADS, 1, HEAD_DIM, 0, 1, 0,
                            100, 1e-6, theta, dir_off, len(tensors), off, 0, 0, 0, 0, 0))
        f.truncate(off)


def test_tensors_stored_under_one_sub_id_are_told_apart_by_shape(tmp_path):
    """One converter path (scripts/fst_converter.py:636-644) writes wq_a and wq_b both as (TID 5, sub 0)
    and wo_a and wo_b both as (TID 8, sub 0); the engine finds each by its shape
    (src/fst_engine.cpp:1553-1558, 1610-1615), takes the compress ratios from TID 40 (1559-1590) and
    the RoPE base from the header (1505).  Given the expected shapes the reader does the same; without
    them it falls back to sub ids and, for such a file, finds no wq_b."""
    rng = np.random.default_rng(5)
    bits = lambda *s: trunc_bits(rng.standard_normal(s).astype(np.float32))  # noqa: E731
    t = {"wq_a": bits(Q_LORA, HIDDEN), "wq_b": bits(HEADS * HEAD_DIM, Q_LORA), "wkv_a": bits(KV, HIDDEN),
         "wo_a": bits(O_LOW, HEADS * HEAD_DIM // 2), "wo_b": bits(HIDDEN, O_LOW)}
    tensors = []
    for l in range(3):
        tensors += [(5, l, 0, F.QTYPE_BF16, t["wq_b"] + l), (5, l, 0, F.QTYPE_BF16, t["wq_a"] + l),
                    (6, l, 0, F.QTYPE_BF16, t["wkv_a"] + l),
                    (8, l, 0, F.QTYPE_BF16, t["wo_b"] + l), (8, l, 0, F.QTYPE_BF16, t["wo_a"] + l)]
    tensors.append((F.TID_COMPRESS_RATIOS, F.GLOBAL_LAYER, 0, F.QTYPE_F32, np.array([0.0, 0.0, 4.0], np.float32)))
    path = str(tmp_path / "sub0.fst")
    _write_fst(path, 3, tensors, theta=50000.0)
    shapes = {k: v.shape for k, v in t.items()}
    for l in range(3):
        w = F.load_mla_layer(path, l, shapes=shapes)
        for k in t:
            assert np.array_equal(w[k], t[k] + l), (l, k)
    plain = F.load_mla_layer(path, 1)
    assert "wq_b" not in plain and "wo_b" not in plain      # (TID, sub 1) does not exist in this form
    assert F.compress_ratios(path, 3) == [0, 0, 4]
    assert F.read_header(path).rope_freq_base == 50000.0
    # a file without TID 40: the engine's default pattern
    assert F.compress_ratios(MAIN, 6) == [0, 0, 4, 128, 4, 128]
    assert F.compress_ratios(MAIN, 43)[40:] == [4, 0, 0]


def test_malformed_files_are_errors(tmp_path):
    p = tmp_path / "bad.fst"
    p.write_bytes(b"nope" + bytes(200))
    with pytest.raises(F.FstFormatError, match="magic"):
        F.read_header(str(p))
    p.write_bytes(b"FST")
    with pytest.raises(F.FstFormatError, match="header"):
        F.read_header(str(p))
    cut = tmp_path / "cut.fst"
    shutil.copy(MAIN, cut)
    with open(cut, "r+b") as f:
        f.truncate(20000)   # the directory survives, most payloads do not
    with pytest.raises(F.FstFormatError, match="out of bounds"):
        F.read_directory(str(cut))


def _engine_lib():
    import ctypes as C
    L = C.CDLL(os.path.join(os.path.dirname(mla.LIB_PATH), "libfst_engine.so"))
    L.fst_file_read_tensor.argtypes = [C.c_char_p, C.c_uint32, C.c_int, C.c_int, C.POINTER(C.c_uint16),
                                       C.POINTER(C.c_float), C.c_int64, C.POINTER(C.c_int64), C.POINTER(C.c_int)]
    L.fst_engine_last_error.restype = C.c_char_p
    return L


def test_cpp_reader_agrees_with_the_python_reader(tmp_path):
    """The host mirror's reader (fastar_b200/host/fst_file.cpp, what FSTEngine::load_shared_weights and
    load_norm_override use) returns the same bits as fst_file.py for every tensor of both fixtures."""
    import ctypes as C
    L = _engine_lib()
    for path in (MAIN, SIDE):
        for e in F.read_directory(path):
            want = F.load_tensor(path, e)
            n = C.c_int64(0)
            qt = C.c_int(0)
            bits = np.zeros(e.n_elements, np.uint16)
            f32 = np.zeros(e.n_elements, np.float32)
            rc = L.fst_file_read_tensor(path.encode(), e.tid, e.layer, e.sub, bits.ctypes.data_as(C.POINTER(C.c_uint16)),
                                        f32.ctypes.data_as(C.POINTER(C.c_float)), e.n_elements, C.byref(n), C.byref(qt))
            assert rc == 0, L.fst_engine_last_error()
            assert (n.value, qt.value) == (e.n_elements, e.qtype)
            if e.qtype == F.QTYPE_F32:
                assert np.array_equal(f32, want.ravel()) and np.array_equal(bits, trunc_bits(want).ravel())
            else:
                assert np.array_equal(bits, want.ravel()), (e.tid, e.layer, e.sub)
                assert np.array_equal(trunc_bits(f32), want.ravel())
    # a tensor the file does not hold: zero elements, no error; a broken file: an error with its reason
    n = C.c_int64(7)
    assert L.fst_file_read_tensor(MAIN.encode(), 99, 0, 0, None, None, 0, C.byref(n), None) == 0 and n.value == 0
    bad = tmp_path / "bad.fst"
    bad.write_bytes(b"nope" + bytes(200))
    assert L.fst_file_read_tensor(str(bad).encode(), 5, 0, 0, None, None, 0, C.byref(n), None) != 0
    assert b"magic" in L.fst_engine_last_error()
