#!/usr/bin/env python3
"""Regenerates tests/golden/ref_v4_layer.npz: the V4 attention layer and its KV compressor as the
REFERENCE's own Python states them (scripts/hf_gen_ref.py), run on small seeded tensors.

    FST_REFERENCE=/path/to/FaStar python tests/golden/make_golden_v4.py

The module cannot be imported (it opens a 160 GB checkpoint at import time), so the pieces are taken
out of it by name with `ast` and run unmodified: the classes `LayerAttn` (389-467 is its forward)
and `Compressor` (266-353) and the functions they call (`rmsnorm`, `act_quant_rt`, `sparse_attn`,
`precompute_freqs_cis`, `apply_rotary_emb`, the two top-k index helpers).  What is replaced, and why:
  * `get_tensor`    -> seeded small tensors (the checkpoint is not here); the module-level shape
                       constants are set to a small geometry (4 heads of 192 = 128 nope + 64 rope)
  * `fp8_linear`    -> plain `x @ W.T`, `fp8_dequant` -> the weight itself: the checkpoint's FP8
                       weight format and the activation quantisation in front of every projection
                       are the HF model's, the engine's process_mla applies neither
                       (src/fst_engine.cpp:3362-3473 multiply bf16 weights by bf16 rows)
  * `act_quant_rt`  -> identity INSIDE LayerAttn.forward only (the raw cached row; the engine keeps
                       it unquantised, 3534-3544); the Compressor keeps the real one (3256-3267)
Stored: inputs, weights and outputs, so the fixture is self-contained.
"""
import ast
import math
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
REF = os.environ.get("FST_REFERENCE")
if not REF:
    sys.exit("set FST_REFERENCE to the FaStar source tree")

GEOM = dict(DIM=128, N_HEADS=4, HEAD_DIM=192, ROPE_HEAD_DIM=64, NOPE_HEAD_DIM=128, Q_LORA=64, O_LORA=32, O_GROUPS=2,
            NORM_EPS=1e-6, WINDOW=128, MAX_SEQ=256, ORIG_SEQ_LEN=65536, ROPE_FACTOR=16.0, BETA_FAST=32, BETA_SLOW=1,
            ROPE_THETA=10000.0, COMPRESS_ROPE_THETA=160000.0, FP8_MAX=448.0, FP8_BLOCK=128,
            COMPRESS_RATIOS=[0, 0, 4, 128], USE_COMPRESSOR=True)
GEOM["SOFTMAX_SCALE"] = GEOM["HEAD_DIM"] ** -0.5


def load(path, names, namespace):
    tree = ast.parse(open(path).read(), path)
    picked = [n for n in tree.body if isinstance(n, (ast.FunctionDef, ast.ClassDef)) and n.name in names]
    assert {n.name for n in picked} == set(names), (set(names) - {n.name for n in picked})
    exec(compile(ast.Module(picked, []), path, "exec"), namespace)


def shapes(L, ratio):
    g = GEOM
    coff = 2 if ratio == 4 else 1
    p = f"layers.{L}.attn."
    sh = {p + "wq_a.weight": (g["Q_LORA"], g["DIM"]), p + "wq_b.weight": (g["N_HEADS"] * g["HEAD_DIM"], g["Q_LORA"]),
          p + "wkv.weight": (g["HEAD_DIM"], g["DIM"]),
          p + "wo_a.weight": (g["O_GROUPS"] * g["O_LORA"], g["N_HEADS"] * g["HEAD_DIM"] // g["O_GROUPS"]),
          p + "wo_b.weight": (g["DIM"], g["O_GROUPS"] * g["O_LORA"]), p + "q_norm.weight": (g["Q_LORA"],),
          p + "kv_norm.weight": (g["HEAD_DIM"],), p + "attn_sink": (g["N_HEADS"],),
          f"layers.{L}.attn_norm.weight": (g["DIM"],)}
    if ratio:
        c = p + "compressor."
        sh.update({c + "ape": (ratio, coff * g["HEAD_DIM"]), c + "wkv.weight": (coff * g["HEAD_DIM"], g["DIM"]),
                   c + "wgate.weight": (coff * g["HEAD_DIM"], g["DIM"]), c + "norm.weight": (g["HEAD_DIM"],)})
    return sh


def main():
    import torch
    import torch.nn.functional as F
    src = os.path.join(REF, "scripts/hf_gen_ref.py")
    rng = np.random.default_rng(20250101)
    store = {}

    def make_tensors(L, ratio):
        t = {}
        for k, s in shapes(L, ratio).items():
            if k.endswith("norm.weight"):
                a = 1.0 + 0.1 * rng.standard_normal(s)
            elif k.endswith("attn_sink") or k.endswith("ape"):
                a = rng.standard_normal(s)
            else:
                a = rng.standard_normal(s) / math.sqrt(s[-1])
            t[k] = torch.from_numpy(a.astype(np.float32))
        return t

    tensors = {}

    def get_tensor(key):
        if key.endswith(".scale"):
            return torch.ones(1)
        return tensors[key]

    base = dict(GEOM, torch=torch, F=F, math=math, os=os, get_tensor=get_tensor)
    # the compressor with the real activation quantiser
    ns_cmp = dict(base)
    load(src, ["act_quant_rt", "apply_rotary_emb", "precompute_freqs_cis", "Compressor"], ns_cmp)
    # the layer: plain products for the projections, the raw row left unquantised
    ns_layer = dict(base, fp8_linear=lambda x, w, s: x.float() @ w.float().T, fp8_dequant=lambda w, s: w.float(),
                    act_quant_rt=lambda x, block: x, Compressor=ns_cmp["Compressor"])
    load(src, ["rmsnorm", "sparse_attn", "apply_rotary_emb", "precompute_freqs_cis", "get_window_topk_idxs",
               "get_compress_topk_idxs", "LayerAttn"], ns_layer)

    def keep_weights(tag, L, only=""):
        for k, v in tensors.items():
            if only in k:
                store[f"{tag}_w_{k.split(f'layers.{L}.')[1]}"] = v.numpy()

    # ---- A. the compressor alone, streamed one token at a time (ratio 4: YaRN layer; ratio 128) ----
    for tag, L, ratio, n_tok in (("cmp4", 2, 4, 23), ("cmp128", 3, 128, 259)):
        tensors.clear()
        tensors.update(make_tensors(L, ratio))
        keep_weights(tag, L, only="compressor.")
        comp = ns_cmp["Compressor"](L, ratio)
        comp.kv_cache = torch.zeros(1, 512 // ratio + 8, GEOM["HEAD_DIM"])
        comp.freqs_cis = ns_cmp["precompute_freqs_cis"](64, 512, GEOM["ORIG_SEQ_LEN"], GEOM["COMPRESS_ROPE_THETA"],
                                                        GEOM["ROPE_FACTOR"], GEOM["BETA_FAST"], GEOM["BETA_SLOW"])
        x = torch.from_numpy(rng.standard_normal((1, n_tok, GEOM["DIM"])).astype(np.float32))
        rows = []
        for t in range(n_tok):
            r = comp.forward(x[:, t:t + 1], t)
            if r is not None:
                rows.append(r.reshape(-1).numpy().copy())
        store[f"{tag}_x"] = x[0].numpy()
        store[f"{tag}_rows"] = np.stack(rows)

    # ---- B. the whole layer without a compressor (layer 0: plain RoPE): prefill of 11 rows, two decode steps ----
    # ---- C. the whole layer WITH its compressor (layer 2: ratio 4, YaRN), decode steps from position 0 ----
    for tag, L, plan in (("layer0", 0, [(0, 11), (11, 1), (12, 1)]), ("layer2", 2, [(t, 1) for t in range(14)])):
        tensors.clear()
        tensors.update(make_tensors(L, GEOM["COMPRESS_RATIOS"][L]))
        keep_weights(tag, L)
        layer = ns_layer["LayerAttn"](L)
        n_tok = sum(n for _, n in plan)
        x = torch.from_numpy(rng.standard_normal((1, n_tok, GEOM["DIM"])).astype(np.float32))
        outs, t0 = [], 0
        for start, n in plan:
            assert start == t0
            outs.append(layer.forward(x[:, t0:t0 + n], start)[0].numpy().copy())
            t0 += n
        store[f"{tag}_x"] = x[0].numpy()
        store[f"{tag}_out"] = np.concatenate(outs)
        store[f"{tag}_plan"] = np.array(plan, np.int64)
        if layer.compressor is not None:
            store[f"{tag}_cmp_rows"] = layer.kv_cache[0, GEOM["WINDOW"]:GEOM["WINDOW"] + n_tok // 4].numpy().copy()

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_v4_layer.npz")
    np.savez_compressed(path, **store)
    print("wrote", path, os.path.getsize(path), "bytes,", len(store), "arrays")


if __name__ == "__main__":
    main()
