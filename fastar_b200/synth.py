"""Seeded synthetic inputs with the shapes and distributions of the benchmark configurations:
weights N(0, 0.02^2), RMSNorm weights 1, activations and cached rows N(0, 1).

Every tensor has its own generator keyed by (seed, tensor id, index), so a tensor is the same
whichever process or GPU builds it and however the batch is sharded.
"""
from __future__ import annotations

import numpy as np

from . import mla

_TENSOR_IDS = {"wq_a": 1, "wq_b": 2, "wkv_a": 3, "wkv_b": 4, "wo_a": 5, "wo_b": 6, "attn_sinks": 7, "attn_norm": 8,
               "x": 20, "cache": 21, "lens": 22, "perm": 23}


def rng_for(seed: int, tensor: str, *index: int) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(np.random.SeedSequence([seed, _TENSOR_IDS[tensor], *index])))


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """fp32 -> bf16 bit patterns, round-to-nearest-even."""
    b = np.ascontiguousarray(x, np.float32).view(np.uint32)
    r = ((b >> 16) & 1) + np.uint32(0x7FFF)
    return ((b + r) >> 16).astype(np.uint16)


def from_bf16_bits(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, np.uint16).astype(np.uint32) << 16).view(np.float32)


def normal_f32(seed: int, tensor: str, shape, std: float = 1.0, index=()) -> np.ndarray:
    g = rng_for(seed, tensor, *index)
    a = g.standard_normal(shape, dtype=np.float32)
    if std != 1.0:
        a *= np.float32(std)
    return a


def layer_weights_f32(cfg: mla.Config, seed: int = 0, lid: int = 0) -> dict:
    """fp32 weights of one layer: matrices N(0, 0.02^2), norm weights 1, sinks N(0, 1) (V4)."""
    out = {}
    for name, shape in mla.weight_shapes(cfg).items():
        if name in ("q_norm", "kv_norm"):
            out[name] = np.ones(shape, np.float32)
        elif name == "attn_sinks":
            out[name] = normal_f32(seed, name, shape, 1.0, (lid,))
        else:
            out[name] = normal_f32(seed, name, shape, 0.02, (lid,))
    return out


def weights_to_bits(w: dict) -> dict:
    return {k: (v if k == "attn_sinks" else to_bf16_bits(v)) for k, v in w.items()}


def weights_rounded(w: dict) -> dict:
    """The bf16-rounded values as fp32 (what the oracle consumes in the bf16 configurations)."""
    return {k: (v if k == "attn_sinks" else from_bf16_bits(to_bf16_bits(v))) for k, v in w.items()}


def hidden_f32(cfg: mla.Config, seed: int, n_tokens: int, index=()) -> np.ndarray:
    return normal_f32(seed, "x", (n_tokens, cfg.hidden), 1.0, index)


def cache_rows_f32(cfg: mla.Config, seed: int, seq_index: int, n_rows: int) -> np.ndarray:
    """Cached rows of one sequence: latent and k_pe values N(0, 1)."""
    return normal_f32(seed, "cache", (n_rows, mla.dims_of(cfg)["row"]), 1.0, (seq_index,))


def context_lengths(seed: int, batch: int, lo: int, hi: int, index=()) -> np.ndarray:
    """Context length of each sequence, uniform in [lo, hi]."""
    return rng_for(seed, "lens", *index).integers(lo, hi + 1, size=batch).astype(np.int64)
