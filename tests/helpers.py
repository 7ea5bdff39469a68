"""Shared test plumbing: seeded inputs, the oracle/GPU pair, the acceptance metrics."""
from __future__ import annotations

import numpy as np

from fastar_b200 import mla, synth
from oracle import oracle as O

# Acceptance bar for bf16 outputs against the CPU oracle on identical inputs.
COS_MIN = 0.9999
MAX_ABS = 2e-2


def cosine(a: np.ndarray, b: np.ndarray) -> float:
    a = np.asarray(a, np.float64).ravel()
    b = np.asarray(b, np.float64).ravel()
    na, nb = np.linalg.norm(a), np.linalg.norm(b)
    if na == 0 and nb == 0:
        return 1.0
    return float(a @ b / (na * nb + 1e-300))


def check_close(got_bits: np.ndarray, want_f32: np.ndarray, what: str, cos_min=COS_MIN, max_abs=MAX_ABS,
                ulps=0):
    """Cosine >= cos_min and max-abs <= max_abs.  The absolute bound is the acceptance figure for
    the benchmark distributions, whose outputs are small; for tensors whose values reach well above
    1 (stress inputs, the V4 preset, intermediate stages) pass `ulps`: the bound then is that many
    bf16 steps at the largest expected magnitude, if that is larger."""
    got = synth.from_bf16_bits(got_bits).reshape(want_f32.shape)
    assert np.all(np.isfinite(got)), f"{what}: non-finite output"
    c = cosine(got, want_f32)
    e = float(np.max(np.abs(got - want_f32))) if got.size else 0.0
    if ulps and want_f32.size:
        top = float(np.max(np.abs(want_f32)))
        if top > 0:
            max_abs = max(max_abs, ulps * 2.0 ** (np.floor(np.log2(top)) - 7))
    assert c >= cos_min and e <= max_abs, f"{what}: cosine {c:.6f} (>= {cos_min}), max-abs {e:.3e} (<= {max_abs})"
    return c, e


def oracle_cfg(cfg: mla.Config, round_bf16=True) -> O.OracleCfg:
    return O.make_cfg(cfg.preset, round_bf16=round_bf16, hidden=cfg.hidden, n_heads=cfg.n_heads,
                      q_lora=cfg.q_lora, kv_lora=cfg.kv_lora, qk_nope=cfg.qk_nope, qk_rope=cfg.qk_rope,
                      v_head=cfg.v_head, o_groups=cfg.o_groups, o_lora=cfg.o_lora,
                      rope_yarn=bool(cfg.rope_yarn))


def oracle_weights(w_rounded: dict) -> dict:
    return dict(w_rounded)


def xorshift_bf16(n: int, state: int = 0x123456789ABCDEF) -> tuple[np.ndarray, int]:
    """The generator of the reference's random-matrix probe (xorshift, uniform [-1, 1] rounded to
    bf16 by truncation; src/fst_engine.cpp:592-595).  Returns bf16 bits and the new state."""
    out = np.empty(n, np.uint16)
    mask = (1 << 64) - 1
    vals = np.empty(n, np.float32)
    for i in range(n):
        state ^= (state << 13) & mask
        state ^= state >> 7
        state ^= (state << 17) & mask
        vals[i] = np.float32((state >> 32) & 0xFFFF) / np.float32(65535.0) * np.float32(2.0) - np.float32(1.0)
    out[:] = (vals.view(np.uint32) >> 16).astype(np.uint16)
    return out, state
