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
