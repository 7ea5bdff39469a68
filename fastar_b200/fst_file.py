"""Reader for the MLA tensors of a FaStar `.fst` checkpoint (the input side of process_mla).

File layout, as the reference's converter writes it (scripts/fst_converter.py:173-176, 685-716,
1464-1500) and its engine reads it (src/fst_engine.cpp:1503-1642, 1873-1900):
  * a 128-byte little-endian header at offset 0: magic "FST\\0", version, hidden_dim, n_layers,
    n_experts, top_k, n_q_heads, n_kv_heads, head_dim, expert_inter_dim, n_shared_experts, 0,
    vocab_size (u64), rms_eps (f32), rope_freq_base (f32), shared-directory offset and count (u64),
    expert bank offset, block bytes, block stride, expert count, two reserved words (u64);
  * a directory of 64-byte entries: tensor id (u32), layer (u16; 0xFFFF = global), sub id, qtype,
    ndim (u16), pad (u32), shape[3], payload offset, payload size, 0 (u64);
  * page-aligned payloads: BF16 (qtype 2, the upper 16 bits of the fp32 value), F32 (qtype 3) or
    Q8_0 (qtype 1): ALL fp16 block scales first, then all int8 values, 32 values per block.

The engine finds its tensors by shape string and layer (1590-1616); the `.norm` sidecar is read by
tensor id (1873-1900) because two norms share the shape "4096x1x1".  This reader goes by tensor id
and sub id for everything (the converter's table, scripts/fst_converter.py:1134-1165):
  TID 5 sub 0 / 1 = wq_a / wq_b, TID 6 = wkv, TID 8 sub 0 / 1 = wo_a / wo_b, TID 14 = q_norm,
  TID 15 = kv_norm, TID 22 = attn_sink (F32), TID 3 = attn_norm.
Q8_0 is expanded as the engine does it (1593-1597): value * scale with a zero scale read as 1, then
fp32 -> bf16 by truncation.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass

import numpy as np

HEADER_FMT = "<4sIIIIIIIIIIIQffQQQQQQQQ"
HEADER_SIZE = struct.calcsize(HEADER_FMT)   # 128
ENTRY_FMT = "<IHHHHIQQQQQQ"
ENTRY_SIZE = struct.calcsize(ENTRY_FMT)     # 64
MAGIC = b"FST\x00"
QTYPE_Q8_0, QTYPE_BF16, QTYPE_F32 = 1, 2, 3
GLOBAL_LAYER = 0xFFFF

TID_INPUT_NORM, TID_Q_PROJ, TID_K_PROJ, TID_O_PROJ = 3, 5, 6, 8
TID_Q_NORM, TID_KV_NORM, TID_ATTN_SINK = 14, 15, 22

# name in a layer's weight dict -> (tensor id, sub id)
MLA_TENSORS = {"wq_a": (TID_Q_PROJ, 0), "wq_b": (TID_Q_PROJ, 1), "wkv_a": (TID_K_PROJ, 0),
               "wo_a": (TID_O_PROJ, 0), "wo_b": (TID_O_PROJ, 1), "q_norm": (TID_Q_NORM, 0),
               "kv_norm": (TID_KV_NORM, 0), "attn_sinks": (TID_ATTN_SINK, 0), "attn_norm": (TID_INPUT_NORM, 0)}
# what the `.norm` sidecar overrides (src/fst_engine.cpp:1873-1885; TIDs 1 and 4 are not MLA's)
NORM_SIDECAR = ("attn_norm", "q_norm", "kv_norm", "attn_sinks")


class FstFormatError(ValueError):
    pass


@dataclass(frozen=True)
class FstHeader:
    version: int
    hidden_dim: int
    n_layers: int
    n_experts: int
    top_k: int
    n_q_heads: int
    n_kv_heads: int
    head_dim: int
    vocab_size: int
    rms_eps: float
    rope_freq_base: float
    dir_offset: int
    dir_count: int


@dataclass(frozen=True)
class FstEntry:
    tid: int
    layer: int
    sub: int
    qtype: int
    shape: tuple
    offset: int
    size: int

    @property
    def n_elements(self) -> int:
        return int(np.prod(self.shape)) if self.shape else 1


def read_header(path: str) -> FstHeader:
    with open(path, "rb") as f:
        raw = f.read(HEADER_SIZE)
    if len(raw) < HEADER_SIZE:
        raise FstFormatError(f"{path}: {len(raw)} bytes, a header has {HEADER_SIZE}")
    h = struct.unpack(HEADER_FMT, raw)
    if h[0] != MAGIC:
        raise FstFormatError(f"{path}: magic {h[0]!r}, expected {MAGIC!r}")
    # the engine falls back to 10000 when the stored base is not positive (src/fst_engine.cpp:1505)
    theta = h[14] if h[14] > 0.0 else 10000.0
    return FstHeader(version=h[1], hidden_dim=h[2], n_layers=h[3], n_experts=h[4], top_k=h[5], n_q_heads=h[6],
                     n_kv_heads=h[7], head_dim=h[8], vocab_size=h[12], rms_eps=h[13], rope_freq_base=theta,
                     dir_offset=h[15], dir_count=h[16])


def read_directory(path: str, header: FstHeader | None = None) -> list:
    header = header or read_header(path)
    with open(path, "rb") as f:
        f.seek(0, 2)
        file_size = f.tell()
        f.seek(header.dir_offset)
        raw = f.read(header.dir_count * ENTRY_SIZE)
    if len(raw) != header.dir_count * ENTRY_SIZE:
        raise FstFormatError(f"{path}: directory of {header.dir_count} entries is cut short")
    out = []
    for i in range(header.dir_count):
        tid, layer, sub, qtype, ndim, _, s0, s1, s2, off, size, _ = struct.unpack_from(ENTRY_FMT, raw, i * ENTRY_SIZE)
        if ndim > 3 or off + size > file_size:
            raise FstFormatError(f"{path}: entry {i} (tid {tid}) is out of bounds")
        out.append(FstEntry(tid, layer, sub, qtype, tuple((s0, s1, s2)[:ndim]), off, size))
    return out


def load_tensor(path: str, e: FstEntry) -> np.ndarray:
    """The tensor of a directory entry: uint16 bf16 bits (BF16, Q8_0) or float32 (F32), in its shape."""
    with open(path, "rb") as f:
        f.seek(e.offset)
        raw = f.read(e.size)
    if len(raw) != e.size:
        raise FstFormatError(f"{path}: payload of tid {e.tid} layer {e.layer} is cut short")
    n = e.n_elements
    if e.qtype == QTYPE_BF16:
        if e.size < 2 * n:
            raise FstFormatError(f"tid {e.tid}: {e.size} bytes for {n} bf16 values")
        return np.frombuffer(raw, np.uint16, n).reshape(e.shape).copy()
    if e.qtype == QTYPE_F32:
        if e.size < 4 * n:
            raise FstFormatError(f"tid {e.tid}: {e.size} bytes for {n} fp32 values")
        return np.frombuffer(raw, np.float32, n).reshape(e.shape).copy()
    if e.qtype == QTYPE_Q8_0:
        nb = (n + 31) // 32
        if e.size < nb * 34:
            raise FstFormatError(f"tid {e.tid}: {e.size} bytes for {nb} Q8_0 blocks")
        scale = np.frombuffer(raw, np.float16, nb).astype(np.float32)
        scale = np.where(np.abs(scale) < 1e-12, np.float32(1.0), scale)     # src/fst_engine.cpp:1595
        q = np.frombuffer(raw, np.int8, nb * 32, offset=nb * 2).astype(np.float32).reshape(nb, 32)
        val = (q * scale[:, None]).reshape(-1)[:n]
        return (val.view(np.uint32) >> 16).astype(np.uint16).reshape(e.shape)  # f2bf truncates (27)
    raise FstFormatError(f"tid {e.tid}: unknown qtype {e.qtype}")


def find(entries, tid: int, layer: int, sub: int = 0):
    """First entry with this tensor id and sub id for the layer (or stored as global)."""
    for e in entries:
        if e.tid == tid and e.sub == sub and e.layer in (layer, GLOBAL_LAYER):
            return e
    return None


def find_shape(entries, tid: int, layer: int, shape):
    """First entry of this tensor id for the layer whose stored shape is `shape`: the way the engine
    tells wq_a from wq_b and wo_a from wo_b (src/fst_engine.cpp:1553-1558, 1610-1615) -- one converter
    path (scripts/fst_converter.py:636-644) stores both under the same tensor id AND sub id 0."""
    shape = tuple(int(x) for x in shape)
    for e in entries:
        if e.tid == tid and e.layer in (layer, GLOBAL_LAYER) and tuple(e.shape) == shape:
            return e
    return None


TID_COMPRESS_RATIOS = 40


def compress_ratios(path: str, n_layers: int, entries=None) -> list:
    """The per-layer KV compress ratios: TID 40 (F32 [n_layers], float -> int) when the file has
    it, else the engine's default pattern 0, 0, 4, 128, 4, ... with layers from 41 on uncompressed
    (src/fst_engine.cpp:1559-1590)."""
    entries = entries if entries is not None else read_directory(path)
    for e in entries:
        if e.tid == TID_COMPRESS_RATIOS:
            r = np.asarray(load_tensor(path, e)).reshape(-1)
            if r.dtype == np.uint16:
                r = (r.astype(np.uint32) << 16).view(np.float32)
            return [int(r[l]) if l < r.size else 0 for l in range(n_layers)]
    return [0 if (l < 2 or l >= 41) else (4 if l % 2 == 0 else 128) for l in range(n_layers)]


def load_mla_layer(path: str, lid: int, norm_path: str | None = None, entries=None, shapes: dict | None = None) -> dict:
    """The MLA weights of layer `lid` as set_layer_weights takes them: bf16 bits in the reference's
    [N_out, K_in] layout, `attn_sinks` fp32.  Tensors the file does not hold are left out.  With
    norm_path, the norm weights and sinks found in that sidecar replace the main file's
    (load_norm_override, src/fst_engine.cpp:1873).  `shapes` ({name: shape}, what the model
    configuration expects) makes the lookup shape-first, as the engine's is: a tensor is the entry
    of its tensor id with the expected shape, and only failing that the entry with its sub id."""
    entries = entries if entries is not None else read_directory(path)
    out = {}
    for name, (tid, sub) in MLA_TENSORS.items():
        e = find_shape(entries, tid, lid, shapes[name]) if shapes and name in shapes else None
        if e is None:
            e = find(entries, tid, lid, sub)
        if e is not None:
            out[name] = load_tensor(path, e)
    if norm_path is not None:
        side = read_directory(norm_path)
        for name in NORM_SIDECAR:
            tid, sub = MLA_TENSORS[name]
            e = find(side, tid, lid, sub)
            if e is not None:
                out[name] = load_tensor(norm_path, e)
    if "attn_sinks" in out and out["attn_sinks"].dtype != np.float32:
        out["attn_sinks"] = (out["attn_sinks"].astype(np.uint32) << 16).view(np.float32)  # stored as bf16
    return out


def check_mla_shapes(weights: dict, shapes: dict) -> None:
    """Raises when a loaded tensor does not have the shape the configuration expects."""
    for name, want in shapes.items():
        if name not in weights:
            raise FstFormatError(f"{name} is missing from the file")
        if tuple(weights[name].shape) != tuple(want):
            raise FstFormatError(f"{name}: file has {tuple(weights[name].shape)}, the configuration wants {tuple(want)}")
