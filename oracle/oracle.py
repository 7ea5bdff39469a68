"""ctypes binding of the CPU oracle (libfst_mla_oracle.so).  TEST INFRASTRUCTURE ONLY.

Imported by tests/, by __graft_entry__.smoke() and by the cpu_baseline / reference legs of
bench.py -- always as the checker or the timed CPU baseline, never by the shipped package.
"""
from __future__ import annotations

import ctypes as C
import math
import os
import subprocess
from dataclasses import dataclass

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libfst_mla_oracle.so")
_REF_PATH = os.path.join(_HERE, "_ref", "libfst_ref_snippets.so")

PRESET_BASELINE = 0
PRESET_FASTAR_V4 = 1


def reference_tree() -> str | None:
    """The FaStar source tree: $FST_REFERENCE, else a folder `reference` beside this repository;
    None when neither holds the engine source."""
    for d in (os.environ.get("FST_REFERENCE"), os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")):
        if d and os.path.exists(os.path.join(d, "src", "fst_engine.cpp")):
            return d
    return None


def build(with_ref: bool = True) -> None:
    """Compile the oracle (and the reference snippets when the reference tree is there)."""
    subprocess.run(["make", "-C", _HERE, "-s"], check=True)
    ref = reference_tree() if with_ref else None
    if ref:
        subprocess.run(["make", "-C", _HERE, "-s", "ref", f"REF={ref}"], check=True)


class OracleCfg(C.Structure):
    _fields_ = [
        ("preset", C.c_int32), ("hidden", C.c_int32), ("n_heads", C.c_int32),
        ("q_lora", C.c_int32), ("kv_lora", C.c_int32), ("qk_nope", C.c_int32),
        ("qk_rope", C.c_int32), ("v_head", C.c_int32), ("o_groups", C.c_int32),
        ("o_lora", C.c_int32), ("softmax_scale", C.c_float), ("rope_theta", C.c_float),
        ("rms_eps", C.c_float), ("rope_yarn", C.c_int32), ("use_sink", C.c_int32),
        ("round_bf16", C.c_int32), ("n_threads", C.c_int32), ("draft_form", C.c_int32),
        ("window", C.c_int32),
    ]


class _Weights(C.Structure):
    _fields_ = [(n, C.POINTER(C.c_float)) for n in
                ("wq_a", "wq_b", "wkv_a", "wkv_b", "wo_a", "wo_b", "q_norm", "kv_norm", "attn_sinks", "attn_norm")]


class _CompressorW(C.Structure):
    _fields_ = [("ratio", C.c_int32)] + [(n, C.POINTER(C.c_float)) for n in ("wkv", "wgate", "ape", "norm")]


class _CompressorState(C.Structure):
    _fields_ = [("state_kv", C.POINTER(C.c_float)), ("state_sc", C.POINTER(C.c_float)),
                ("cache", C.POINTER(C.c_float)), ("n_comp", C.c_int32), ("cap", C.c_int32)]


class _Trace(C.Structure):
    _fields_ = [(n, C.POINTER(C.c_float)) for n in ("qc", "kv", "q_eff", "o_lat", "low")]


def make_cfg(preset: int = PRESET_BASELINE, *, round_bf16: bool = True, n_threads: int = 0,
             hidden: int = 4096, n_heads: int = 64, q_lora: int = 1024, kv_lora: int = 512,
             qk_nope: int = 128, qk_rope: int = 64, v_head: int = 128, o_groups: int = 8,
             o_lora: int = 1024, rope_yarn: bool = False, use_sink: bool | None = None,
             softmax_scale: float | None = None, draft_form: bool = False) -> OracleCfg:
    """Configuration of either preset.  BASELINE: 576-wide rows, scale 1/sqrt(nope+rope),
    no sink.  FASTAR_V4: 512-wide rows with a RoPE tail, scale 1/sqrt(512), sink on."""
    if preset == PRESET_BASELINE:
        scale = 1.0 / math.sqrt(qk_nope + qk_rope)
        sink = False
    else:
        scale = 1.0 / math.sqrt(kv_lora)
        sink = True
        qk_nope = kv_lora - qk_rope
    if softmax_scale is not None:
        scale = softmax_scale
    if use_sink is not None:
        sink = use_sink
    return OracleCfg(preset, hidden, n_heads, q_lora, kv_lora, qk_nope, qk_rope, v_head, o_groups,
                     o_lora, scale, 10000.0, 1e-6, int(rope_yarn), int(sink), int(round_bf16),
                     n_threads, int(draft_form), 0)


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build(with_ref=False)
        L = C.CDLL(_LIB_PATH)
        fp = C.POINTER(C.c_float)
        cp = C.POINTER(OracleCfg)
        L.fst_oracle_bf16_round.restype = C.c_float
        L.fst_oracle_bf16_round.argtypes = [C.c_float]
        L.fst_oracle_bf16_trunc.restype = C.c_float
        L.fst_oracle_bf16_trunc.argtypes = [C.c_float]
        L.fst_oracle_bf16_round_array.argtypes = [fp, C.c_int64]
        L.fst_oracle_rmsnorm.argtypes = [fp, fp, fp, C.c_int, C.c_int, C.c_float, C.c_int]
        L.fst_oracle_rope_lut.argtypes = [fp, C.c_int, C.c_int, C.c_float, C.c_int, C.c_int, C.c_int]
        L.fst_oracle_rope_apply.argtypes = [fp, C.c_int, C.c_int, C.c_float, C.c_int, C.c_int, C.c_int]
        L.fst_oracle_gemm.argtypes = [fp, fp, fp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]
        L.fst_oracle_attention.argtypes = [cp, fp, fp, C.c_int, C.c_int, C.c_int, C.c_int, fp, fp]
        L.fst_oracle_attention_partial.argtypes = [cp, fp, fp, C.c_int, C.c_int, C.c_int, C.c_int,
                                                   C.c_int, fp, fp, fp]
        L.fst_oracle_merge_partials.argtypes = [cp, fp, fp, fp, C.c_int, C.c_int, fp, fp]
        L.fst_oracle_mla_forward.argtypes = [cp, C.POINTER(_Weights), fp, C.c_int, C.c_int, C.c_int,
                                             fp, C.c_int, fp, C.POINTER(_Trace)]
        L.fst_oracle_mla_forward.restype = C.c_int
        i32p = C.POINTER(C.c_int32)
        L.fst_oracle_mla_forward_batch.argtypes = [cp, C.POINTER(_Weights), fp, C.c_int, i32p, i32p, C.c_int,
                                                   C.POINTER(fp), i32p, fp, C.POINTER(_Trace)]
        L.fst_oracle_mla_forward_batch.restype = C.c_int
        L.fst_oracle_mla_forward_batch_cmp.argtypes = [cp, C.POINTER(_Weights), C.POINTER(_CompressorW),
                                                       C.POINTER(_CompressorState), fp, C.c_int, i32p, i32p, C.c_int,
                                                       C.POINTER(fp), i32p, fp, C.POINTER(_Trace)]
        L.fst_oracle_mla_forward_batch_cmp.restype = C.c_int
        L.fst_oracle_compress_token.argtypes = [cp, C.POINTER(_CompressorW), C.POINTER(_CompressorState), fp, C.c_int]
        L.fst_oracle_compress_token.restype = C.c_int
        L.fst_oracle_e4m3_roundtrip.argtypes = [C.c_float]
        L.fst_oracle_e4m3_roundtrip.restype = C.c_float
        L.fst_oracle_compressor_width.argtypes = [C.c_int, C.c_int]
        L.fst_oracle_compressor_rows.argtypes = [C.c_int]
        for n in ("row_width", "d_qk", "d_v", "low_dim", "threads"):
            getattr(L, "fst_oracle_" + n).argtypes = [cp]
        L.fst_oracle_pager_create.restype = C.c_void_p
        L.fst_oracle_pager_create.argtypes = [C.c_int, C.c_int, C.c_int]
        L.fst_oracle_pager_destroy.argtypes = [C.c_void_p]
        L.fst_oracle_pager_seq_alloc.argtypes = [C.c_void_p]
        L.fst_oracle_pager_seq_free.argtypes = [C.c_void_p, C.c_int]
        L.fst_oracle_pager_reserve.argtypes = [C.c_void_p, C.c_int, C.c_int]
        L.fst_oracle_pager_truncate.argtypes = [C.c_void_p, C.c_int, C.c_int]
        L.fst_oracle_pager_table.argtypes = [C.c_void_p, C.c_int, C.POINTER(C.c_int32), C.c_int]
        L.fst_oracle_pager_free_pages.argtypes = [C.c_void_p]
        _lib = L
    return _lib


def ref_lib() -> C.CDLL | None:
    """The reference's own bf16 helpers, rms_cpu and build_rope_lut, when they were built."""
    if not os.path.exists(_REF_PATH):
        return None
    L = C.CDLL(_REF_PATH)
    u16 = C.POINTER(C.c_uint16)
    L.fst_ref_f2bf.restype = C.c_uint16
    L.fst_ref_f2bf.argtypes = [C.c_float]
    L.fst_ref_bf16f.restype = C.c_float
    L.fst_ref_bf16f.argtypes = [C.c_uint16]
    L.fst_ref_rms_cpu.argtypes = [u16, u16, u16, C.c_int, C.c_int]
    L.fst_ref_build_rope_lut.argtypes = [u16, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]
    return L


def _f(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a: np.ndarray | None):
    return None if a is None else a.ctypes.data_as(C.POINTER(C.c_float))


# ---- bf16 helpers in numpy (round-to-nearest-even), shared by tests --------------------
def bf16_round(x: np.ndarray) -> np.ndarray:
    """fp32 -> nearest bf16 value, returned as fp32."""
    b = _f(x).view(np.uint32).astype(np.uint64)
    b = (b + 0x7FFF + ((b >> 16) & 1)) & 0xFFFF0000
    return b.astype(np.uint32).view(np.float32).reshape(np.shape(x))


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """fp32 -> bf16 bit pattern (uint16), round-to-nearest-even."""
    b = _f(x).view(np.uint32).astype(np.uint64)
    b = (b + 0x7FFF + ((b >> 16) & 1)) >> 16
    return b.astype(np.uint16).reshape(np.shape(x))


def from_bf16_bits(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def dims(cfg: OracleCfg) -> dict:
    L = lib()
    return {"row": L.fst_oracle_row_width(C.byref(cfg)), "d_qk": L.fst_oracle_d_qk(C.byref(cfg)),
            "d_v": L.fst_oracle_d_v(C.byref(cfg)), "low": L.fst_oracle_low_dim(C.byref(cfg))}


def threads(cfg: OracleCfg) -> int:
    return lib().fst_oracle_threads(C.byref(cfg))


def rmsnorm(x, w, eps=1e-6, round_bf16=False):
    x = _f(x)
    rows, d = x.reshape(-1, x.shape[-1]).shape
    y = np.empty_like(x)
    wv = None if w is None else _f(w)
    lib().fst_oracle_rmsnorm(_p(x), _p(wv), _p(y), rows, d, eps, int(round_bf16))
    return y


def rope_lut(pos, rope_dim=64, theta=10000.0, yarn=False, inverse=False, round_lut_bf16=False):
    lut = np.empty(rope_dim, np.float32)
    lib().fst_oracle_rope_lut(_p(lut), pos, rope_dim, theta, int(yarn), int(inverse),
                              int(round_lut_bf16))
    return lut


def rope_apply(x, pos, theta=10000.0, yarn=False, inverse=False, round_bf16=False):
    y = _f(x).copy()
    lib().fst_oracle_rope_apply(_p(y), pos, y.shape[-1], theta, int(yarn), int(inverse),
                                int(round_bf16))
    return y


def gemm(A, B, b_kn=False, round_bf16=False, n_threads=0):
    A, B = _f(A), _f(B)
    M, K = A.shape
    N = B.shape[1] if b_kn else B.shape[0]
    Cm = np.empty((M, N), np.float32)
    lib().fst_oracle_gemm(_p(A), _p(B), _p(Cm), M, N, K, int(b_kn), int(round_bf16), n_threads)
    return Cm


def attention(cfg, q_eff, cache, kv_len, n_q, pos0=0, causal=False, sinks=None):
    d = dims(cfg)
    q_eff, cache = _f(q_eff), _f(cache)
    out = np.empty((n_q * cfg.n_heads, d["d_v"]), np.float32)
    sk = None if sinks is None else _f(sinks)
    lib().fst_oracle_attention(C.byref(cfg), _p(q_eff), _p(cache), kv_len, n_q, pos0, int(causal),
                               _p(sk), _p(out))
    return out


def attention_partial(cfg, q_eff, cache, s0, s1, n_q, pos0=0, causal=False):
    d = dims(cfg)
    q_eff, cache = _f(q_eff), _f(cache)
    rows = n_q * cfg.n_heads
    m = np.empty(rows, np.float32)
    l = np.empty(rows, np.float32)
    o = np.empty((rows, d["d_v"]), np.float32)
    lib().fst_oracle_attention_partial(C.byref(cfg), _p(q_eff), _p(cache), s0, s1, n_q, pos0,
                                       int(causal), _p(m), _p(l), _p(o))
    return m, l, o


def merge_partials(cfg, m, l, o, sinks=None):
    d = dims(cfg)
    m, l, o = _f(m), _f(l), _f(o)
    n_parts, rows = m.shape
    out = np.empty((rows, d["d_v"]), np.float32)
    sk = None if sinks is None else _f(sinks)
    lib().fst_oracle_merge_partials(C.byref(cfg), _p(m), _p(l), _p(o), n_parts, rows, _p(sk), _p(out))
    return out


def attention_window(cfg, q_eff, cache, kv_len, n_q, window, pos0=0, causal=False, sinks=None):
    """Sliding-window attention (the draft model keeps only the last `window_size` rows, reference
    src/fst_engine.cpp:2534-2576): query token i sees the last `window` rows of what attention()
    lets it see.  A composition of attention_partial over [lo, hi) and merge_partials, per token."""
    H = cfg.n_heads
    q_eff = _f(q_eff)
    out = np.empty((n_q * H, dims(cfg)["d_v"]), np.float32)
    for i in range(n_q):
        hi = min(kv_len, pos0 + i + 1) if causal else kv_len
        lo = max(0, hi - window) if window > 0 else 0
        m, l, o = attention_partial(cfg, q_eff[i * H:(i + 1) * H], cache, lo, hi, 1)
        out[i * H:(i + 1) * H] = merge_partials(cfg, m[None], l[None], o[None], sinks)
    return out


@dataclass
class ForwardResult:
    out: np.ndarray
    trace: dict


def mla_forward(cfg, weights: dict, h, pos0, cache, causal=False, want_trace=True) -> ForwardResult:
    """Run the layer for one sequence.  `cache` is a float32 [cap, row] array updated in place
    (rows pos0 .. pos0+M-1 are appended).  weights: name -> float32 array (missing = None)."""
    d = dims(cfg)
    h = _f(h)
    M = h.shape[0]
    assert cache.dtype == np.float32 and cache.flags.c_contiguous
    keep = {k: _f(v) for k, v in weights.items() if v is not None}
    w = _Weights(**{k: _p(v) for k, v in keep.items()})
    out = np.empty((M, cfg.hidden), np.float32)
    H = cfg.n_heads
    tr = {}
    t = _Trace()
    if want_trace:
        tr = {"qc": np.empty((M, cfg.q_lora), np.float32), "kv": np.empty((M, d["row"]), np.float32),
              "q_eff": np.empty((M * H, d["d_qk"]), np.float32),
              "o_lat": np.empty((M * H, d["d_v"]), np.float32),
              "low": np.empty((M, d["low"]), np.float32)}
        t = _Trace(**{k: _p(v) for k, v in tr.items()})
    rc = lib().fst_oracle_mla_forward(C.byref(cfg), C.byref(w), _p(h), M, pos0, int(causal),
                                      _p(cache), cache.shape[0], _p(out), C.byref(t))
    if rc != 0:
        raise ValueError("oracle: pos0 + M exceeds the cache capacity")
    return ForwardResult(out, tr)


class Compressor:
    """Weights of one layer's KV compressor (wkv, wgate [width, hidden]; ape [ratio, width];
    norm [kv_lora]) and the streaming state of ONE sequence: window state, compressed rows."""

    def __init__(self, cfg, ratio: int, wkv, wgate, ape, norm, cap: int = 4096, score_init: float = 0.0):
        self.ratio, self.kv_lora = ratio, cfg.kv_lora
        self.width = lib().fst_oracle_compressor_width(ratio, cfg.kv_lora)
        self.rows = lib().fst_oracle_compressor_rows(ratio)
        self.wkv, self.wgate, self.ape, self.norm = _f(wkv), _f(wgate), _f(ape), _f(norm)
        assert self.wkv.shape == (self.width, cfg.hidden) and self.ape.shape == (ratio, self.width)
        self.w = _CompressorW(ratio, _p(self.wkv), _p(self.wgate), _p(self.ape), _p(self.norm))
        self.cap, self.score_init = cap, score_init
        self.reset()

    def reset(self):
        # the engine starts both states at zero (reset_compressor_state, src/fst_engine.cpp:3160-3169);
        # the HF model starts the scores at -inf (score_init)
        self.state_kv = np.zeros((self.rows, self.width), np.float32)
        self.state_sc = np.full((self.rows, self.width), self.score_init, np.float32)
        self.cache = np.zeros((self.cap, self.kv_lora), np.float32)
        self.st = _CompressorState(_p(self.state_kv), _p(self.state_sc), _p(self.cache), 0, self.cap)

    def fork(self):
        """A second sequence with the same weights and a fresh state."""
        o = object.__new__(Compressor)
        o.__dict__.update(self.__dict__)
        o.reset()
        return o

    @property
    def n_comp(self) -> int:
        return self.st.n_comp

    def rows_out(self) -> np.ndarray:
        return self.cache[:self.st.n_comp]

    def push(self, cfg, hidden_normed, pos: int) -> int:
        return lib().fst_oracle_compress_token(C.byref(cfg), C.byref(self.w), C.byref(self.st), _p(_f(hidden_normed)), pos)


def e4m3_roundtrip(v: float) -> float:
    return lib().fst_oracle_e4m3_roundtrip(float(v))


def mla_forward_batch(cfg, weights: dict, h, q_lens, pos0, caches, causal=False, want_trace=False,
                      compressors=None) -> ForwardResult:
    """The layer for B sequences in one call: h [sum q_lens, hidden] holds the sequences' rows back to
    back, caches[b] is sequence b's float32 [cap_b, row] array (updated in place).  Row for row the
    arithmetic of mla_forward; the projections run over all rows at once."""
    d = dims(cfg)
    h = _f(h)
    q = np.ascontiguousarray(q_lens, np.int32)
    p0 = np.ascontiguousarray(pos0, np.int32)
    B, T = len(q), int(q.sum())
    assert h.shape == (T, cfg.hidden) and len(caches) == B and len(p0) == B
    for c in caches:
        assert c.dtype == np.float32 and c.flags.c_contiguous and c.shape[1] == d["row"]
    caps = np.array([c.shape[0] for c in caches], np.int32)
    fp = C.POINTER(C.c_float)
    cptr = (fp * max(B, 1))(*[_p(c) for c in caches])
    keep = {k: _f(v) for k, v in weights.items() if v is not None}
    w = _Weights(**{k: _p(v) for k, v in keep.items()})
    out = np.empty((T, cfg.hidden), np.float32)
    H = cfg.n_heads
    tr = {}
    t = _Trace()
    if want_trace:
        tr = {"qc": np.empty((T, cfg.q_lora), np.float32), "kv": np.empty((T, d["row"]), np.float32),
              "q_eff": np.empty((T * H, d["d_qk"]), np.float32),
              "o_lat": np.empty((T * H, d["d_v"]), np.float32),
              "low": np.empty((T, d["low"]), np.float32)}
        t = _Trace(**{k: _p(v) for k, v in tr.items()})
    i32p = C.POINTER(C.c_int32)
    if compressors is not None:
        # one Compressor per sequence (same weights, own state): the layer's KV compressor
        assert len(compressors) == B
        sts = (_CompressorState * B)(*[c.st for c in compressors])
        rc = lib().fst_oracle_mla_forward_batch_cmp(C.byref(cfg), C.byref(w), C.byref(compressors[0].w), sts, _p(h), B,
                                                    q.ctypes.data_as(i32p), p0.ctypes.data_as(i32p), int(causal), cptr,
                                                    caps.ctypes.data_as(i32p), _p(out), C.byref(t))
        for c, st in zip(compressors, sts):
            c.st.n_comp = st.n_comp
    else:
        rc = lib().fst_oracle_mla_forward_batch(C.byref(cfg), C.byref(w), _p(h), B, q.ctypes.data_as(i32p),
                                                p0.ctypes.data_as(i32p), int(causal), cptr, caps.ctypes.data_as(i32p),
                                                _p(out), C.byref(t))
    if rc != 0:
        raise ValueError("oracle: a sequence's pos0 + q_len exceeds its cache capacity")
    return ForwardResult(out, tr)


class Pager:
    """Host twin of the paged-cache bookkeeping (LIFO free list)."""

    def __init__(self, n_pages, page_tokens=64, max_seqs=256):
        self._h = lib().fst_oracle_pager_create(n_pages, page_tokens, max_seqs)
        if not self._h:
            raise ValueError("bad pager arguments")
        self._cap = n_pages

    def __del__(self):
        if getattr(self, "_h", None):
            lib().fst_oracle_pager_destroy(self._h)
            self._h = None

    def seq_alloc(self):
        return lib().fst_oracle_pager_seq_alloc(self._h)

    def seq_free(self, s):
        return lib().fst_oracle_pager_seq_free(self._h, s)

    def reserve(self, s, n):
        return lib().fst_oracle_pager_reserve(self._h, s, n)

    def truncate(self, s, n):
        return lib().fst_oracle_pager_truncate(self._h, s, n)

    def table(self, s):
        buf = (C.c_int32 * max(self._cap, 1))()
        n = lib().fst_oracle_pager_table(self._h, s, buf, self._cap)
        if n < 0:
            raise KeyError(s)
        return np.array(buf[:n], np.int32)

    def free_pages(self):
        return lib().fst_oracle_pager_free_pages(self._h)
