"""ctypes binding of the C ABI (include/fst_cuda_mla.h) and a thin object wrapper.

The wrapper mirrors how the engine drives the path: weights once, a sequence per chat,
`forward(lid, h, seq_ids, pos0, q_lens)` per layer call.  There is no CPU fallback: without the
built library, or without a GPU, construction raises.
"""
from __future__ import annotations

import ctypes as C
import math
import os

import numpy as np

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libfst_cuda_mla.so")

PRESET_BASELINE = 0
PRESET_FASTAR_V4 = 1
IMPL_AUTO, IMPL_TENSOR, IMPL_SIMT = 0, 1, 2
STAGE_QC, STAGE_KV, STAGE_QEFF, STAGE_OLAT, STAGE_LOW, STAGE_OUT = range(6)
KERNEL_NAMES = ["compress", "norm_append", "q_expand", "q_absorb", "attn", "merge", "exchange", "merge_gathered",
                "oproj_a", "oproj_b"]
K_ATTN, K_MERGE = 4, 5

ERR_ARG, ERR_PAGES, ERR_CAPACITY, ERR_CUDA, ERR_DEVICE_CHECK, ERR_STATE, ERR_NO_DEVICE = -1, -2, -3, -4, -5, -6, -7
ERR_COMM = -8
GATHER_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p)


class MlaError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"fst_cuda_mla error {code}: {msg}")
        self.code = code


class Config(C.Structure):
    _fields_ = [
        ("preset", C.c_int32), ("hidden", C.c_int32), ("n_heads", C.c_int32), ("q_lora", C.c_int32),
        ("kv_lora", C.c_int32), ("qk_nope", C.c_int32), ("qk_rope", C.c_int32), ("v_head", C.c_int32),
        ("o_groups", C.c_int32), ("o_lora", C.c_int32), ("softmax_scale", C.c_float),
        ("rope_theta", C.c_float), ("rms_eps", C.c_float), ("rope_yarn", C.c_int32),
        ("n_layers", C.c_int32), ("page_tokens", C.c_int32), ("n_pages", C.c_int32),
        ("max_seqs", C.c_int32), ("max_tokens", C.c_int32), ("device", C.c_int32),
        ("attn_impl", C.c_int32), ("gemm_impl", C.c_int32),
    ]


class Weights(C.Structure):
    _fields_ = [(n, C.POINTER(C.c_uint16)) for n in
                ("wq_a", "wq_b", "wkv_a", "wkv_b", "wo_a", "wo_b", "q_norm", "kv_norm")] + \
               [("attn_sinks", C.POINTER(C.c_float)), ("attn_norm", C.POINTER(C.c_uint16))]


class CompressorW(C.Structure):
    _fields_ = [("ratio", C.c_int32), ("wkv", C.POINTER(C.c_uint16)), ("wgate", C.POINTER(C.c_uint16)),
                ("ape", C.POINTER(C.c_float)), ("norm", C.POINTER(C.c_uint16))]


class SeqStep(C.Structure):
    _fields_ = [("seq", C.c_int32), ("pos0", C.c_int32), ("q_len", C.c_int32),
                ("rope_pos0", C.c_int32), ("append", C.c_int32), ("window", C.c_int32)]


def make_config(preset=PRESET_BASELINE, *, n_layers=1, n_pages=256, max_seqs=64, max_tokens=64, device=0,
                hidden=4096, n_heads=64, q_lora=1024, kv_lora=512, qk_nope=128, qk_rope=64, v_head=128,
                o_groups=8, o_lora=1024, page_tokens=64, rope_yarn=False, attn_impl=IMPL_AUTO,
                gemm_impl=IMPL_AUTO, softmax_scale=0.0) -> Config:
    return Config(preset, hidden, n_heads, q_lora, kv_lora, qk_nope, qk_rope, v_head, o_groups, o_lora,
                  softmax_scale, 10000.0, 1e-6, int(rope_yarn), n_layers, page_tokens, n_pages, max_seqs,
                  max_tokens, device, attn_impl, gemm_impl)


_lib = None


def load_library() -> C.CDLL:
    """Load libfst_cuda_mla.so.  Fails loudly when it was not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(f"{LIB_PATH} is missing: run `python -m fastar_b200.build` "
                           "(the MLA path has no fallback without its CUDA library)")
    L = C.CDLL(LIB_PATH)
    vp, i32, i64 = C.c_void_p, C.c_int32, C.c_int64
    u16p, i32p = C.POINTER(C.c_uint16), C.POINTER(C.c_int32)
    L.fst_cuda_mla_last_error.restype = C.c_char_p
    L.fst_cuda_mla_create.argtypes = [C.POINTER(Config), C.POINTER(vp)]
    L.fst_cuda_mla_destroy.argtypes = [vp]
    L.fst_cuda_mla_destroy.restype = None
    L.fst_cuda_mla_set_stream.argtypes = [vp, vp]
    L.fst_cuda_mla_sync.argtypes = [vp]
    L.fst_cuda_mla_set_layer_weights.argtypes = [vp, C.c_int, C.POINTER(Weights)]
    L.fst_cuda_mla_seq_alloc.argtypes = [vp, i32p]
    L.fst_cuda_mla_seq_free.argtypes = [vp, i32]
    L.fst_cuda_mla_seq_reserve.argtypes = [vp, i32, i32]
    L.fst_cuda_mla_seq_truncate.argtypes = [vp, i32, i32]
    L.fst_cuda_mla_seq_len.argtypes = [vp, i32, i32p]
    L.fst_cuda_mla_reset.argtypes = [vp]
    L.fst_cuda_mla_block_table.argtypes = [vp, i32, i32p, i32, i32p]
    L.fst_cuda_mla_free_pages.argtypes = [vp, i32p]
    L.fst_cuda_mla_row_offset.argtypes = [vp, i32, i32, C.POINTER(i64)]
    L.fst_cuda_mla_cache_write.argtypes = [vp, C.c_int, i32, i32, i32, u16p]
    L.fst_cuda_mla_cache_read.argtypes = [vp, C.c_int, i32, i32, i32, u16p]
    L.fst_cuda_mla_pool_read.argtypes = [vp, C.c_int, u16p, C.c_size_t]
    L.fst_cuda_mla_plan.argtypes = [vp, C.POINTER(SeqStep), i32, i32]
    L.fst_cuda_mla_run_device.argtypes = [vp, C.c_int, vp, vp]
    L.fst_cuda_mla_forward.argtypes = [vp, C.c_int, u16p, u16p, i32p, i32p, i32p, i32, i32]
    L.fst_cuda_mla_attention_only.argtypes = [vp, C.c_int, u16p, u16p]
    L.fst_cuda_mla_run_partial_device.argtypes = [vp, C.c_int, vp, vp]
    L.fst_cuda_mla_run_merge_device.argtypes = [vp, C.c_int, vp, i32, vp]
    L.fst_cuda_mla_plan_tokens.argtypes = [vp, i32p]
    L.fst_cuda_mla_get_stage.argtypes = [vp, C.c_int, u16p, C.c_size_t]
    L.fst_cuda_mla_gemm.argtypes = [vp, u16p, u16p, u16p, C.c_int, C.c_int, C.c_int, C.c_int]
    L.fst_cuda_mla_launch_count.argtypes = [vp, C.POINTER(i64)]
    L.fst_cuda_mla_set_profiling.argtypes = [vp, C.c_int]
    L.fst_cuda_mla_kernel_times.argtypes = [vp, C.POINTER(C.c_float), i32p]
    L.fst_cuda_mla_plan_info.argtypes = [vp, i32p, i32p, C.POINTER(i64)]
    L.fst_cuda_mla_set_plan_reuse.argtypes = [vp, i32]
    L.fst_cuda_mla_set_window.argtypes = [vp, i32]
    L.fst_cuda_mla_set_fused_merge.argtypes = [vp, i32]
    L.fst_cuda_mla_set_block_schedule.argtypes = [vp, i32]
    L.fst_cuda_mla_debug_schedule.argtypes = [i32, i32p, i32p, i32, i32, i32, i32p, i32, i32p, i32p, i32p]
    L.fst_cuda_mla_plan_counts.argtypes = [vp, C.POINTER(i64), C.POINTER(i64)]
    L.fst_cuda_mla_set_layer_rope.argtypes = [vp, C.c_int, i32]
    L.fst_cuda_mla_set_rope_theta.argtypes = [vp, C.c_float]
    L.fst_cuda_mla_set_layer_compressor.argtypes = [vp, C.c_int, C.POINTER(CompressorW)]
    L.fst_cuda_mla_set_layer_draft_form.argtypes = [vp, C.c_int, i32]
    L.fst_cuda_mla_append_rows.argtypes = [vp, C.c_int, u16p, i32p, i32p, i32p, i32]
    L.fst_cuda_mla_cmp_read.argtypes = [vp, C.c_int, i32, u16p, i32, i32p]
    L.fst_cuda_mla_seq_snapshot.argtypes = [vp, i32]
    L.fst_cuda_mla_comm_unique_id.argtypes = [C.POINTER(C.c_uint8)]
    L.fst_cuda_mla_comm_init.argtypes = [vp, C.POINTER(C.c_uint8), i32, i32]
    L.fst_cuda_mla_comm_set_gather.argtypes = [vp, GATHER_FN, vp, i32, i32]
    L.fst_cuda_mla_comm_destroy.argtypes = [vp]
    L.fst_cuda_mla_run_split_device.argtypes = [vp, C.c_int, vp, vp]
    L.fst_cuda_mla_forward_split.argtypes = [vp, C.c_int, u16p, u16p, C.POINTER(SeqStep), i32, i32]
    L.fst_cuda_mla_family_counts.argtypes = [vp, C.POINTER(i64), C.POINTER(i64)]
    L.fst_cuda_mla_selftest_wait_expiry.argtypes = [vp, i32]
    L.fst_cuda_mla_debug_set_status.argtypes = [vp, i32]
    L.fst_cuda_mla_debug_attr_first_use.argtypes = [C.c_uint64, i32, i64]
    L.fst_cuda_mla_attention_noalloc.argtypes = [vp, vp, i32, i32, i32, i32, C.c_float, vp, vp]
    _lib = L
    return L


def _u16(a: np.ndarray):
    return a.ctypes.data_as(C.POINTER(C.c_uint16))


def _i32(a: np.ndarray):
    return a.ctypes.data_as(C.POINTER(C.c_int32))


def dims_of(cfg: Config) -> dict:
    v4 = cfg.preset == PRESET_FASTAR_V4
    row = cfg.kv_lora if v4 else cfg.kv_lora + cfg.qk_rope
    return {"row": row, "d_qk": row, "d_v": cfg.kv_lora,
            "q_head": cfg.kv_lora if v4 else cfg.qk_nope + cfg.qk_rope,
            "low": cfg.o_groups * cfg.o_lora if v4 else cfg.n_heads * cfg.v_head}


def weight_shapes(cfg: Config) -> dict:
    """name -> shape of every weight the preset uses (reference layout: [N_out, K_in])."""
    d = dims_of(cfg)
    H = cfg.n_heads
    sh = {"wq_a": (cfg.q_lora, cfg.hidden), "wq_b": (H * d["q_head"], cfg.q_lora),
          "wkv_a": (d["row"], cfg.hidden), "wo_b": (cfg.hidden, d["low"]),
          "q_norm": (cfg.q_lora,), "kv_norm": (cfg.kv_lora,)}
    if cfg.preset == PRESET_FASTAR_V4:
        sh["wo_a"] = (d["low"], H * d["d_v"] // cfg.o_groups)
        sh["attn_sinks"] = (H,)
    else:
        sh["wkv_b"] = (H * (cfg.qk_nope + cfg.v_head), cfg.kv_lora)
    return sh


def debug_schedule(n_sm: int, pos0, q_lens, causal: bool, by_blocks: bool = True):
    """The split-KV schedule of a call as the library cuts it, on the host alone (no device needed):
    (segments [n, 5] = token, first row, end row, partial slot, thread block; number of thread blocks;
    whether the block schedule cut it)."""
    L = load_library()
    p0 = np.ascontiguousarray(pos0, np.int32)
    ql = np.ascontiguousarray(q_lens, np.int32)
    cap = int(ql.sum()) + n_sm + 8
    segs = np.zeros((cap, 5), np.int32)
    n, k, b = C.c_int32(0), C.c_int32(0), C.c_int32(0)
    i32p = C.POINTER(C.c_int32)
    rc = L.fst_cuda_mla_debug_schedule(n_sm, p0.ctypes.data_as(i32p), ql.ctypes.data_as(i32p), len(p0), int(causal),
                                       int(by_blocks), segs.ctypes.data_as(i32p), cap, C.byref(n), C.byref(k), C.byref(b))
    if rc:
        raise MlaError(rc, L.fst_cuda_mla_last_error().decode())
    return segs[:n.value].copy(), k.value, bool(b.value)


class MlaContext:
    """One GPU's MLA state: weights, paged latent cache, workspaces."""

    def __init__(self, cfg: Config):
        self.lib = load_library()
        self.cfg = cfg
        self.dims = dims_of(cfg)
        self._h = C.c_void_p()
        self._check(self.lib.fst_cuda_mla_create(C.byref(cfg), C.byref(self._h)))

    # -- plumbing --
    def _check(self, rc: int) -> None:
        if rc != 0:
            raise MlaError(rc, self.lib.fst_cuda_mla_last_error().decode())

    def close(self) -> None:
        if getattr(self, "_h", None) and self._h.value:
            self.lib.fst_cuda_mla_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def set_stream(self, cuda_stream: int) -> None:
        self._check(self.lib.fst_cuda_mla_set_stream(self._h, C.c_void_p(cuda_stream)))

    def sync(self) -> None:
        self._check(self.lib.fst_cuda_mla_sync(self._h))

    # -- weights --
    def set_layer_weights(self, lid: int, weights: dict) -> None:
        """weights: name -> uint16 bf16-bit arrays (attn_sinks: float32)."""
        keep = {}
        w = Weights()
        for name, _ in Weights._fields_:
            a = weights.get(name)
            if a is None:
                continue
            if name == "attn_sinks":
                a = np.ascontiguousarray(a, np.float32)
                setattr(w, name, a.ctypes.data_as(C.POINTER(C.c_float)))
            else:
                a = np.ascontiguousarray(a, np.uint16)
                setattr(w, name, _u16(a))
            keep[name] = a
        self._check(self.lib.fst_cuda_mla_set_layer_weights(self._h, lid, C.byref(w)))

    def set_layer_rope(self, lid: int, yarn: bool) -> None:
        """RoPE kind of one layer: plain, or the YaRN tables of the compressed V4 layers."""
        self._check(self.lib.fst_cuda_mla_set_layer_rope(self._h, lid, 1 if yarn else 0))

    def set_layer_compressor(self, lid: int, ratio: int, wkv=None, wgate=None, ape=None, norm=None) -> None:
        """The layer's V4 KV compressor: wkv / wgate bf16 bits [width, hidden], ape fp32 [ratio, width],
        norm bf16 bits [kv_lora]; ratio 0 removes it."""
        if not ratio:
            self._check(self.lib.fst_cuda_mla_set_layer_compressor(self._h, lid, None))
            return
        wkv, wgate = np.ascontiguousarray(wkv, np.uint16), np.ascontiguousarray(wgate, np.uint16)
        ape, norm = np.ascontiguousarray(ape, np.float32), np.ascontiguousarray(norm, np.uint16)
        w = CompressorW(ratio, _u16(wkv), _u16(wgate), ape.ctypes.data_as(C.POINTER(C.c_float)), _u16(norm))
        self._check(self.lib.fst_cuda_mla_set_layer_compressor(self._h, lid, C.byref(w)))

    def set_layer_draft_form(self, lid: int, on: bool = True) -> None:
        """The draft model's form of the layer: no per-head q norm, q / output rotation on head 0 only."""
        self._check(self.lib.fst_cuda_mla_set_layer_draft_form(self._h, lid, 1 if on else 0))

    def append_rows(self, lid: int, h: np.ndarray, seq_ids, pos0, q_lens) -> None:
        """KV side of the layer alone: rows -> kv compress, kv_norm, key RoPE, cache append."""
        h = np.ascontiguousarray(h, np.uint16)
        s, p, q = (np.ascontiguousarray(x, np.int32) for x in (seq_ids, pos0, q_lens))
        self._check(self.lib.fst_cuda_mla_append_rows(self._h, lid, _u16(h), _i32(s), _i32(p), _i32(q), len(s)))

    def cmp_read(self, lid: int, seq: int) -> np.ndarray:
        """The compressed rows of a sequence in one layer, uint16 bf16 bits [n, kv_lora]."""
        n = C.c_int32()
        self._check(self.lib.fst_cuda_mla_cmp_read(self._h, lid, seq, None, 0, C.byref(n)))
        out = np.empty((n.value, self.dims["row"]), np.uint16)
        if n.value:
            self._check(self.lib.fst_cuda_mla_cmp_read(self._h, lid, seq, _u16(out), n.value, C.byref(n)))
        return out

    def seq_snapshot(self, seq: int) -> None:
        self._check(self.lib.fst_cuda_mla_seq_snapshot(self._h, seq))

    def set_rope_theta(self, theta: float) -> None:
        self._check(self.lib.fst_cuda_mla_set_rope_theta(self._h, theta))

    # -- paged cache --
    def seq_alloc(self) -> int:
        s = C.c_int32()
        self._check(self.lib.fst_cuda_mla_seq_alloc(self._h, C.byref(s)))
        return s.value

    def seq_free(self, seq: int) -> None:
        self._check(self.lib.fst_cuda_mla_seq_free(self._h, seq))

    def seq_reserve(self, seq: int, n: int) -> None:
        self._check(self.lib.fst_cuda_mla_seq_reserve(self._h, seq, n))

    def seq_truncate(self, seq: int, n: int) -> None:
        self._check(self.lib.fst_cuda_mla_seq_truncate(self._h, seq, n))

    def seq_len(self, seq: int) -> int:
        n = C.c_int32()
        self._check(self.lib.fst_cuda_mla_seq_len(self._h, seq, C.byref(n)))
        return n.value

    def reset(self) -> None:
        self._check(self.lib.fst_cuda_mla_reset(self._h))

    def block_table(self, seq: int) -> np.ndarray:
        buf = np.zeros(max(self.cfg.n_pages, 1), np.int32)
        n = C.c_int32()
        self._check(self.lib.fst_cuda_mla_block_table(self._h, seq, _i32(buf), buf.size, C.byref(n)))
        return buf[:n.value].copy()

    def free_pages(self) -> int:
        n = C.c_int32()
        self._check(self.lib.fst_cuda_mla_free_pages(self._h, C.byref(n)))
        return n.value

    def row_offset(self, seq: int, pos: int) -> int:
        o = C.c_int64()
        self._check(self.lib.fst_cuda_mla_row_offset(self._h, seq, pos, C.byref(o)))
        return o.value

    def cache_write(self, lid: int, seq: int, pos0: int, rows: np.ndarray) -> None:
        rows = np.ascontiguousarray(rows, np.uint16)
        assert rows.ndim == 2 and rows.shape[1] == self.dims["row"]
        self._check(self.lib.fst_cuda_mla_cache_write(self._h, lid, seq, pos0, rows.shape[0], _u16(rows)))

    def cache_read(self, lid: int, seq: int, pos0: int, n: int) -> np.ndarray:
        out = np.empty((n, self.dims["row"]), np.uint16)
        self._check(self.lib.fst_cuda_mla_cache_read(self._h, lid, seq, pos0, n, _u16(out)))
        return out

    def pool_read(self, lid: int) -> np.ndarray:
        out = np.empty((self.cfg.n_pages * self.cfg.page_tokens, self.dims["row"]), np.uint16)
        self._check(self.lib.fst_cuda_mla_pool_read(self._h, lid, _u16(out), out.nbytes))
        return out

    # -- the layer --
    def plan(self, steps, causal: bool = False) -> int:
        """steps: iterable of (seq, pos0, q_len[, rope_pos0[, append[, window]]]).  Returns T."""
        arr = (SeqStep * len(steps))()
        for i, s in enumerate(steps):
            s = tuple(s)
            arr[i] = SeqStep(s[0], s[1], s[2], s[3] if len(s) > 3 else -1, s[4] if len(s) > 4 else 1,
                             s[5] if len(s) > 5 else 0)
        self._check(self.lib.fst_cuda_mla_plan(self._h, arr, len(steps), int(causal)))
        return self.plan_tokens()

    def plan_tokens(self) -> int:
        t = C.c_int32()
        self._check(self.lib.fst_cuda_mla_plan_tokens(self._h, C.byref(t)))
        return t.value

    def set_plan_reuse(self, on: bool) -> None:
        """Whether a plan request equal to the valid plan keeps it (default) or rebuilds it."""
        self._check(self.lib.fst_cuda_mla_set_plan_reuse(self._h, 1 if on else 0))

    def set_block_schedule(self, on: bool) -> None:
        """Calls with G >= 4 new tokens per sequence: thread blocks in groups of G lanes that share pages."""
        self._check(self.lib.fst_cuda_mla_set_block_schedule(self._h, 1 if on else 0))

    def set_fused_merge(self, on: bool) -> None:
        """Let the attention kernel finish tokens that have a single partial itself (default)."""
        self._check(self.lib.fst_cuda_mla_set_fused_merge(self._h, 1 if on else 0))

    def set_window(self, window: int) -> None:
        """Sliding window that forward() applies to every sequence (0: none)."""
        self._check(self.lib.fst_cuda_mla_set_window(self._h, int(window)))

    def plan_counts(self) -> dict:
        built, reused = C.c_int64(0), C.c_int64(0)
        self._check(self.lib.fst_cuda_mla_plan_counts(self._h, C.byref(built), C.byref(reused)))
        return {"built": built.value, "reused": reused.value}

    def plan_info(self) -> dict:
        a, b, c = C.c_int32(), C.c_int32(), C.c_int64()
        self._check(self.lib.fst_cuda_mla_plan_info(self._h, C.byref(a), C.byref(b), C.byref(c)))
        return {"n_partials": a.value, "n_ctas": b.value, "kv_rows": c.value}

    def run_device(self, lid: int, d_in: int, d_out: int) -> None:
        self._check(self.lib.fst_cuda_mla_run_device(self._h, lid, C.c_void_p(d_in), C.c_void_p(d_out)))

    def run_partial_device(self, lid: int, d_in: int, d_partial: int) -> None:
        self._check(self.lib.fst_cuda_mla_run_partial_device(self._h, lid, C.c_void_p(d_in), C.c_void_p(d_partial)))

    def run_merge_device(self, lid: int, d_partials: int, n_parts: int, d_out: int) -> None:
        self._check(self.lib.fst_cuda_mla_run_merge_device(self._h, lid, C.c_void_p(d_partials), n_parts,
                                                          C.c_void_p(d_out)))

    # -- split-KV across GPUs --
    def comm_init(self, unique_id: bytes, rank: int, world: int) -> None:
        """Join an NCCL communicator of `world` ranks (collective).  unique_id: comm_unique_id() of rank 0."""
        buf = (C.c_uint8 * 128).from_buffer_copy(unique_id)
        self._check(self.lib.fst_cuda_mla_comm_init(self._h, buf, rank, world))

    def comm_set_gather(self, fn, rank: int, world: int) -> None:
        """A host-supplied all-gather: fn(d_send, d_recv, bytes_per_rank, stream) -> 0."""
        self._gather_cb = GATHER_FN(lambda user, s, r, n, st: int(fn(s, r, n, st) or 0))
        self._check(self.lib.fst_cuda_mla_comm_set_gather(self._h, self._gather_cb, None, rank, world))

    def comm_destroy(self) -> None:
        self._check(self.lib.fst_cuda_mla_comm_destroy(self._h))

    def run_split_device(self, lid: int, d_in: int, d_out: int) -> None:
        self._check(self.lib.fst_cuda_mla_run_split_device(self._h, lid, C.c_void_p(d_in), C.c_void_p(d_out)))

    def forward_split(self, lid: int, h: np.ndarray, steps, causal: bool = False) -> np.ndarray:
        """The split-KV layer call with host buffers; steps as for plan()."""
        h = np.ascontiguousarray(h, np.uint16)
        out = np.empty_like(h)
        arr = (SeqStep * len(steps))()
        for i, s in enumerate(steps):
            s = tuple(s)
            arr[i] = SeqStep(s[0], s[1], s[2], s[3] if len(s) > 3 else -1, s[4] if len(s) > 4 else 1,
                             s[5] if len(s) > 5 else 0)
        self._check(self.lib.fst_cuda_mla_forward_split(self._h, lid, _u16(h), _u16(out), arr, len(steps), int(causal)))
        return out

    def forward(self, lid: int, h: np.ndarray, seq_ids, pos0, q_lens, causal: bool = False) -> np.ndarray:
        """process_mla with host buffers.  h: uint16 [T, hidden] bf16 bits.  Returns the same shape."""
        h = np.ascontiguousarray(h, np.uint16)
        out = np.empty_like(h)
        s = np.ascontiguousarray(seq_ids, np.int32)
        p = np.ascontiguousarray(pos0, np.int32)
        q = np.ascontiguousarray(q_lens, np.int32)
        assert h.shape == (int(q.sum()), self.cfg.hidden)
        self._check(self.lib.fst_cuda_mla_forward(self._h, lid, _u16(h), _u16(out), _i32(s), _i32(p), _i32(q),
                                                  len(s), int(causal)))
        return out

    def forward_into(self, lid: int, h: np.ndarray, out: np.ndarray, s, p, q, causal: bool = False) -> None:
        """forward() without allocating: all arrays prepared by the caller (timed loops)."""
        self._check(self.lib.fst_cuda_mla_forward(self._h, lid, _u16(h), _u16(out), _i32(s), _i32(p), _i32(q),
                                                  len(s), int(causal)))

    def bind_forward(self, lid: int, h: np.ndarray, out: np.ndarray, s, p, q, causal: bool = False):
        """forward_into() with the argument conversion done once: returns a callable that makes
        exactly the C call (for loops that reuse the same page-locked buffers, as a host that
        calls the C ABI directly would)."""
        keep = (h, out, s, p, q)  # the arrays must outlive the pointers
        args = (self._h, lid, _u16(h), _u16(out), _i32(s), _i32(p), _i32(q), len(s), int(causal))
        fn, check = self.lib.fst_cuda_mla_forward, self._check

        def call(_keep=keep):
            check(fn(*args))
        return call

    def attention_only(self, lid: int, q_eff: np.ndarray) -> np.ndarray:
        q_eff = np.ascontiguousarray(q_eff, np.uint16)
        T = self.plan_tokens()
        assert q_eff.shape == (T * self.cfg.n_heads, self.dims["d_qk"])
        out = np.empty((T * self.cfg.n_heads, self.dims["d_v"]), np.uint16)
        self._check(self.lib.fst_cuda_mla_attention_only(self._h, lid, _u16(q_eff), _u16(out)))
        return out

    def get_stage(self, stage: int) -> np.ndarray:
        T, H, d, c = self.plan_tokens(), self.cfg.n_heads, self.dims, self.cfg
        shape = {STAGE_QC: (T, c.q_lora), STAGE_KV: (T, d["row"]), STAGE_QEFF: (T * H, d["d_qk"]),
                 STAGE_OLAT: (T * H, d["d_v"]), STAGE_LOW: (T, d["low"]), STAGE_OUT: (T, c.hidden)}[stage]
        out = np.empty(shape, np.uint16)
        self._check(self.lib.fst_cuda_mla_get_stage(self._h, stage, _u16(out), out.nbytes))
        return out

    def gemm(self, A: np.ndarray, B: np.ndarray, b_kn: bool = False) -> np.ndarray:
        """npu_gemm_mla_vec: C = A @ B.T (B is [N, K]) or A @ B (b_kn: B is [K, N])."""
        A = np.ascontiguousarray(A, np.uint16)
        B = np.ascontiguousarray(B, np.uint16)
        M, K = A.shape
        N = B.shape[1] if b_kn else B.shape[0]
        Cm = np.empty((M, N), np.uint16)
        self._check(self.lib.fst_cuda_mla_gemm(self._h, _u16(Cm), _u16(A), _u16(B), M, N, K, int(b_kn)))
        return Cm

    # -- measurement --
    def launch_count(self) -> int:
        n = C.c_int64()
        self._check(self.lib.fst_cuda_mla_launch_count(self._h, C.byref(n)))
        return n.value

    def family_counts(self) -> dict:
        """GEMM and attention launches so far by kernel family."""
        a, b = C.c_int64(0), C.c_int64(0)
        self._check(self.lib.fst_cuda_mla_family_counts(self._h, C.byref(a), C.byref(b)))
        return {"tensor": a.value, "simt": b.value}

    def selftest_wait_expiry(self, polls: int = 2000) -> None:
        self._check(self.lib.fst_cuda_mla_selftest_wait_expiry(self._h, polls))

    def debug_set_status(self, code: int) -> None:
        self._check(self.lib.fst_cuda_mla_debug_set_status(self._h, code))

    def set_profiling(self, on: bool) -> None:
        self._check(self.lib.fst_cuda_mla_set_profiling(self._h, int(on)))

    def kernel_times(self) -> dict:
        ms = (C.c_float * len(KERNEL_NAMES))()
        n = (C.c_int32 * len(KERNEL_NAMES))()
        self._check(self.lib.fst_cuda_mla_kernel_times(self._h, ms, n))
        return {k: (ms[i], n[i]) for i, k in enumerate(KERNEL_NAMES)}


def attention_noalloc(d_q_eff: int, d_cache: int, n_rows: int, n_heads: int, d_qk: int, d_v: int, scale: float,
                      d_o_lat: int, stream: int = 0) -> int:
    """Decode attention of one query token over a contiguous device cache, for callers that must
    not allocate (see include/fst_cuda_mla.h).  Device pointers as integers; returns the status."""
    return load_library().fst_cuda_mla_attention_noalloc(C.c_void_p(d_q_eff), C.c_void_p(d_cache), n_rows, n_heads,
                                                         d_qk, d_v, scale, C.c_void_p(d_o_lat), C.c_void_p(stream))


def comm_unique_id() -> bytes:
    """The 128 bytes rank 0 creates for comm_init (ncclGetUniqueId)."""
    buf = (C.c_uint8 * 128)()
    rc = load_library().fst_cuda_mla_comm_unique_id(buf)
    if rc != 0:
        raise MlaError(rc, load_library().fst_cuda_mla_last_error().decode())
    return bytes(buf)


def default_scale(cfg: Config) -> float:
    if cfg.softmax_scale > 0:
        return cfg.softmax_scale
    return 1.0 / math.sqrt(cfg.kv_lora if cfg.preset == PRESET_FASTAR_V4 else cfg.qk_nope + cfg.qk_rope)
