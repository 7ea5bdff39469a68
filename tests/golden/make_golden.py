#!/usr/bin/env python3
"""Regenerates tests/golden/ref_vectors.npz from the reference's own code.

Run where the FaStar tree is (FST_REFERENCE=/path/to/FaStar):
    make -C oracle ref && python tests/golden/make_golden.py

Two sources, both executed unmodified:
  * Python functions of the reference, taken out of their modules by name with `ast`
    (the modules themselves cannot be imported: they open model weights or an NPU at
    import time): sparse_attn, precompute_freqs_cis, apply_rotary_emb
    (scripts/hf_gen_ref.py:194-241) and host_rms_norm, host_softmax
    (scripts/fst_layer_benchmark.py:20-31).
  * C++ functions of the engine compiled from where they lie by oracle/Makefile:
    f2bf / bf16f (src/fst_engine.cpp:26-27), rms_cpu (89-91), build_rope_lut (1970-2023).
Inputs are seeded; inputs and outputs are stored together, so the fixture is self-contained.
"""
import ast
import ctypes as C
import math
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
REF = os.environ.get("FST_REFERENCE")
if not REF:
    sys.exit("set FST_REFERENCE to the FaStar source tree")


def load_functions(path, names, namespace):
    tree = ast.parse(open(path).read(), path)
    picked = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name in names]
    assert {n.name for n in picked} == set(names), (path, names)
    exec(compile(ast.Module(picked, []), path, "exec"), namespace)
    return [namespace[n] for n in names]


def main():
    import torch
    from ml_dtypes import bfloat16
    from oracle import oracle as O

    out = {}
    rng = np.random.default_rng(20240607)

    # ---- reference Python functions ----------------------------------------------------
    ns = {"torch": torch, "math": math, "F": torch.nn.functional}
    sparse_attn, precompute_freqs_cis, apply_rotary_emb = load_functions(
        os.path.join(REF, "scripts/hf_gen_ref.py"),
        ["sparse_attn", "precompute_freqs_cis", "apply_rotary_emb"], ns)
    ns2 = {"np": np, "bfloat16": bfloat16, "HEAD_DIM": 512}
    host_rms_norm, host_softmax = load_functions(
        os.path.join(REF, "scripts/fst_layer_benchmark.py"), ["host_rms_norm", "host_softmax"], ns2)

    # RoPE angle tables: plain (base 10000) and YaRN (base 160000, factor 16, 65536, 32/1).
    pos = np.array([0, 1, 2, 7, 63, 127, 128, 1000, 4095], np.int64)
    fc = precompute_freqs_cis(64, 4096, 0, 10000.0, 16, 32, 1)
    out["hf_rope_pos"] = pos
    out["hf_rope_plain_cos"] = fc.real[pos].numpy().astype(np.float32)
    out["hf_rope_plain_sin"] = fc.imag[pos].numpy().astype(np.float32)
    fy = precompute_freqs_cis(64, 4096, 65536, 160000.0, 16, 32, 1)
    out["hf_rope_yarn_cos"] = fy.real[pos].numpy().astype(np.float32)
    out["hf_rope_yarn_sin"] = fy.imag[pos].numpy().astype(np.float32)

    # Rotation of [1, s, heads, 64] at positions p0 .. p0+s-1, forward and inverse.
    p0, s, nh = 37, 4, 3
    x = rng.standard_normal((1, s, nh, 64)).astype(np.float32)
    out["hf_rot_x"] = x
    out["hf_rot_p0"] = np.int64(p0)
    out["hf_rot_fwd"] = apply_rotary_emb(torch.from_numpy(x), fc[p0:p0 + s]).numpy()
    out["hf_rot_inv"] = apply_rotary_emb(torch.from_numpy(x), fc[p0:p0 + s], inverse=True).numpy()

    # Latent attention with a sink (the V4 core): 2 query tokens, 4 heads, 37 cached rows,
    # causal among the 2 new tokens (rows 35, 36 are theirs).
    nq, H, L = 2, 4, 37
    q = (rng.standard_normal((1, nq, H, 512)) * 0.5).astype(np.float32)
    kv = rng.standard_normal((1, L, 512)).astype(np.float32)
    sink = rng.standard_normal(H).astype(np.float32)
    idx = np.full((1, nq, L), -1, np.int32)
    for i in range(nq):
        n_vis = L - nq + i + 1
        idx[0, i, :n_vis] = np.arange(n_vis)
    scale = 1.0 / math.sqrt(512.0)
    out["hf_attn_q"], out["hf_attn_kv"], out["hf_attn_sink"] = q, kv, sink
    out["hf_attn_out"] = sparse_attn(torch.from_numpy(q), torch.from_numpy(kv), torch.from_numpy(sink),
                                     torch.from_numpy(idx), scale).numpy()

    # Benchmark-harness host ops (bf16 results, stored as fp32).
    xr = rng.standard_normal((4, 512)).astype(np.float32)
    wr = (1.0 + 0.1 * rng.standard_normal(512)).astype(np.float32)
    out["lb_rms_x"], out["lb_rms_w"] = xr, wr
    out["lb_rms_out"] = host_rms_norm(xr.astype(bfloat16), wr.astype(bfloat16)).astype(np.float32)
    sc = (rng.standard_normal((8, 40)) * 30).astype(np.float32)
    sk = rng.standard_normal(8).astype(np.float32)
    out["lb_sm_scores"], out["lb_sm_sinks"] = sc, sk
    out["lb_sm_out"] = host_softmax(sc.astype(bfloat16), sk.astype(bfloat16)).astype(np.float32)

    # ---- reference C++ functions -------------------------------------------------------
    R = O.ref_lib()
    assert R is not None, "run `make -C oracle ref` first"
    fl = np.concatenate([rng.standard_normal(64).astype(np.float32) * 10,
                         np.array([0.0, -0.0, 1.0, 1.0039062, 3.3895314e38, 1e-40], np.float32)])
    out["cc_f2bf_in"] = fl
    out["cc_f2bf_out"] = np.array([R.fst_ref_f2bf(float(v)) for v in fl], np.uint16)
    for d in (512, 1024):
        xi = O.to_bf16_bits(rng.standard_normal((3, d)).astype(np.float32) * 2)
        wi = O.to_bf16_bits(1.0 + 0.1 * rng.standard_normal(d).astype(np.float32))
        oo = np.zeros_like(xi)
        u16 = C.POINTER(C.c_uint16)
        R.fst_ref_rms_cpu(oo.ctypes.data_as(u16), xi.ctypes.data_as(u16), wi.ctypes.data_as(u16), d, 3)
        out[f"cc_rms{d}_x"], out[f"cc_rms{d}_w"], out[f"cc_rms{d}_out"] = xi, wi, oo
    lut_pos = np.array([0, 1, 5, 127, 4095, 131071], np.int64)
    out["cc_lut_pos"] = lut_pos
    for name, comp in (("plain", 0), ("yarn", 1)):
        for inv in (0, 1):
            rows = []
            for p in lut_pos:
                lut = np.zeros((2, 64), np.uint16)
                R.fst_ref_build_rope_lut(lut.ctypes.data_as(C.POINTER(C.c_uint16)), 2, int(p), 64, comp, inv)
                rows.append(lut)
            out[f"cc_lut_{name}_{'inv' if inv else 'fwd'}"] = np.stack(rows)

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_vectors.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()
