"""Writes tests/golden/tiny_mla.fst and tiny_mla.fst.norm with the REFERENCE's own converter
primitives (scripts/fst_converter.py: _pack_header, _quant_shared, align_up, SHARED_ENTRY_FMT, the
TID_* / QTYPE_* constants), following the writer loop of convert_full_model_v4
(scripts/fst_converter.py:1464-1500): header page, directory page, page-aligned payloads.

Run where the FaStar tree is:
    FST_REFERENCE=/path/to/FaStar python tests/golden/make_fst_fixture.py
The tensors are tiny (hidden 64, 4 heads) and seeded, so the test can rebuild the float values and
check what the reader returns against them; shapes are free in the format.
"""
import os
import struct
import sys

import numpy as np

REF = os.environ.get("FST_REFERENCE")
if not REF:
    sys.exit("set FST_REFERENCE to the FaStar source tree")
sys.path.insert(0, os.path.join(REF, "scripts"))
sys.argv = sys.argv[:1]
import fst_converter as F  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
N_LAYERS, HIDDEN, HEADS, Q_LORA, KV, HEAD_DIM, O_LOW = 2, 64, 4, 32, 24, 24, 48


def tensors(seed: int = 0):
    """(tid, layer, sub, qtype, float32 array) in file order; seeded."""
    rng = np.random.default_rng(seed)
    out = []
    for l in range(N_LAYERS):
        n = lambda *s: rng.standard_normal(s).astype(np.float32)  # noqa: E731
        out += [
            (F.TID_INPUT_NORM, l, 0, F.QTYPE_BF16, 1.0 + 0.1 * n(HIDDEN)),
            (F.TID_POST_ATTN_NORM, l, 0, F.QTYPE_BF16, 1.0 + 0.1 * n(HIDDEN)),   # not MLA: must be skipped
            (F.TID_Q_PROJ, l, 0, F.QTYPE_BF16, 0.05 * n(Q_LORA, HIDDEN)),         # wq_a
            (F.TID_Q_PROJ, l, 1, F.QTYPE_Q8_0, 0.05 * n(HEADS * HEAD_DIM, Q_LORA)),  # wq_b, quantised
            (F.TID_K_PROJ, l, 0, F.QTYPE_BF16, 0.05 * n(KV, HIDDEN)),             # wkv
            (F.TID_O_PROJ, l, 0, F.QTYPE_Q8_0, 0.05 * n(O_LOW, HEADS * HEAD_DIM // 2)),  # wo_a, quantised
            (F.TID_O_PROJ, l, 1, F.QTYPE_BF16, 0.05 * n(HIDDEN, O_LOW)),          # wo_b
            (F.TID_Q_NORM, l, 0, F.QTYPE_BF16, 1.0 + 0.1 * n(Q_LORA)),
            (F.TID_KV_NORM, l, 0, F.QTYPE_BF16, 1.0 + 0.1 * n(KV)),
            (F.TID_ATTN_SINK, l, 0, F.QTYPE_F32, n(HEADS)),
        ]
    return out


def norm_sidecar(seed: int = 1):
    """The .norm sidecar carries only norm TIDs and sinks (src/fst_engine.cpp:1873-1885)."""
    rng = np.random.default_rng(seed)
    out = []
    for l in range(N_LAYERS):
        n = lambda *s: rng.standard_normal(s).astype(np.float32)  # noqa: E731
        out += [(F.TID_INPUT_NORM, l, 0, F.QTYPE_BF16, 1.2 + 0.1 * n(HIDDEN)),
                (F.TID_Q_NORM, l, 0, F.QTYPE_BF16, 0.9 + 0.1 * n(Q_LORA)),
                (F.TID_KV_NORM, l, 0, F.QTYPE_BF16, 1.1 + 0.1 * n(KV)),
                (F.TID_ATTN_SINK, l, 0, F.QTYPE_F32, n(HEADS))]
    return out


def write(path: str, entries) -> None:
    cfg = {"hidden_dim": HIDDEN, "num_layers": N_LAYERS, "num_experts": 0, "top_k": 8, "num_q_heads": HEADS,
           "num_kv_heads": 1, "head_dim": HEAD_DIM, "vocab_size": 100, "rms_eps": 1e-6, "rope_freq_base": 10000.0}
    dir_off = F.align_up(F.HEADER_SIZE)
    data_off0 = F.align_up(dir_off + len(entries) * F.SHARED_ENTRY_SIZE)
    with open(path, "wb") as f:
        f.write(b"\x00" * data_off0)
        packed = []
        for tid, lid, sub, qtype, t in entries:
            shape = F._shape_of(t)
            shape3 = (shape + (1, 1, 1))[:3]
            data = F._quant_shared(t, qtype)
            off = F.align_up(f.tell())
            f.seek(off)
            f.write(data)
            packed.append(struct.pack(F.SHARED_ENTRY_FMT, tid, lid, sub, qtype, len(shape), 0, int(shape3[0]),
                                      int(shape3[1]), int(shape3[2]), int(off), int(len(data)), 0))
        end = F.align_up(f.tell())
        f.seek(dir_off)
        f.write(b"".join(packed))
        f.seek(0)
        f.write(F._pack_header(cfg, dir_off, len(entries), end, 0))
        f.truncate(max(end, f.tell()))


if __name__ == "__main__":
    write(os.path.join(HERE, "tiny_mla.fst"), tensors())
    write(os.path.join(HERE, "tiny_mla.fst.norm"), norm_sidecar())
    for n in ("tiny_mla.fst", "tiny_mla.fst.norm"):
        print(n, os.path.getsize(os.path.join(HERE, n)), "bytes")
