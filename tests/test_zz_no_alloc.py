"""fst_cuda_mla_attention_noalloc: the decode-attention entry point for hosts that may not
allocate device memory (a fully pre-budgeted serving process, a no-malloc callback, a plugin that
only gets device pointers).  Its split-KV partials sit in a fixed array inside the library, so the
checks are: same answer as the regular entry point (fst_cuda_mla_attention_only over the paged
cache), twice in a row with different sizes so that what the first call left in the shared array
cannot leak into the second, and a clean refusal beyond the array's limits.

Collected last on purpose: a failure here must not hide the rest of a stop-at-first-failure run."""
import math

import numpy as np
import pytest
import torch

from fastar_b200 import mla, synth
from oracle import oracle as O
from tests.helpers import check_close

pytestmark = pytest.mark.gpu


def regular_path(rows_bits, q_bits):
    """The existing entry point on the same rows and query: paged cache, context-owned workspaces."""
    L = rows_bits.shape[0]
    cfg = mla.make_config(mla.PRESET_BASELINE, n_pages=L // 64 + 3, max_tokens=1, max_seqs=1)
    with mla.MlaContext(cfg) as ctx:
        w = {n: np.zeros(s, np.uint16) for n, s in mla.weight_shapes(cfg).items()}
        ctx.set_layer_weights(0, w)
        s = ctx.seq_alloc()
        ctx.cache_write(0, s, 0, rows_bits)
        ctx.plan([(s, L, 1, -1, 0)])
        return ctx.attention_only(0, q_bits)


def test_matches_the_regular_entry_point_twice_in_a_row():
    scale = 1.0 / math.sqrt(192.0)
    rng = np.random.default_rng(12)
    cfg = mla.make_config()
    # (the second, smaller call reuses the array's stale contents; the third is the largest size, all 32 splits
    # of the tcgen05 kernel with a ragged last page)
    for call, L in enumerate((5000, 777, 65536 - 37)):
        rows = synth.to_bf16_bits(synth.cache_rows_f32(cfg, 40 + call, 0, L))
        q = synth.to_bf16_bits(rng.standard_normal((64, 576)).astype(np.float32))
        d_rows = torch.from_numpy(rows.view(np.int16)).cuda()
        d_q = torch.from_numpy(q.view(np.int16)).cuda()
        d_out = torch.zeros((64, 512), dtype=torch.int16, device="cuda")
        torch.cuda.synchronize()
        rc = mla.attention_noalloc(d_q.data_ptr(), d_rows.data_ptr(), L, 64, 576, 512, scale, d_out.data_ptr(),
                                   torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        torch.cuda.synchronize()
        got = d_out.cpu().numpy().view(np.uint16)
        want = synth.from_bf16_bits(regular_path(rows, q))
        # same bar as the other attention tests: cosine >= 0.9999, max-abs <= 2e-2
        check_close(got, want, f"call {call} (L={L})")


@pytest.mark.parametrize("heads,d_qk,d_v,n_rows", [(64, 576, 512, 1), (64, 576, 512, 129), (5, 72, 64, 300),
                                                   (16, 512, 512, 1000), (3, 136, 128, 33)])
def test_small_and_odd_shapes_against_the_cpu_oracle(heads, d_qk, d_v, n_rows):
    """Fewer than 64 heads, narrow rows, one row, a ragged second split: each against the oracle's
    attention on the same bits (rows are d_qk wide with no padding; values are row[:d_v])."""
    rng = np.random.default_rng(heads * 1000 + n_rows)
    rows = synth.to_bf16_bits(rng.standard_normal((n_rows, d_qk)).astype(np.float32))
    q = synth.to_bf16_bits(rng.standard_normal((heads, d_qk)).astype(np.float32))
    scale = 1.0 / math.sqrt(d_qk)
    d_rows = torch.from_numpy(rows.view(np.int16)).cuda()
    d_q = torch.from_numpy(q.view(np.int16)).cuda()
    d_out = torch.zeros((heads, d_v), dtype=torch.int16, device="cuda")
    rc = mla.attention_noalloc(d_q.data_ptr(), d_rows.data_ptr(), n_rows, heads, d_qk, d_v, scale, d_out.data_ptr(),
                               torch.cuda.current_stream().cuda_stream)
    assert rc == 0, mla.load_library().fst_cuda_mla_last_error()
    torch.cuda.synchronize()
    # the oracle with this geometry: V4 form (row == d_qk, values = row[:kv_lora]) without a sink
    ocfg = O.make_cfg(O.PRESET_FASTAR_V4, n_heads=heads, kv_lora=d_qk, use_sink=False, softmax_scale=scale)
    want = O.attention(ocfg, synth.from_bf16_bits(q), synth.from_bf16_bits(rows), n_rows, 1)[:, :d_v]
    check_close(d_out.cpu().numpy().view(np.uint16), want, f"H={heads} d_qk={d_qk} d_v={d_v} rows={n_rows}", ulps=2)


def test_refusals_reach_the_last_error_string():
    d = torch.zeros(64 * 576, dtype=torch.int16, device="cuda")
    p = d.data_ptr()
    lib = mla.load_library()
    assert mla.attention_noalloc(p, p, 70000, 64, 576, 512, 0.07, p) == mla.ERR_CAPACITY
    assert b"65536 cached rows" in lib.fst_cuda_mla_last_error()
    assert mla.attention_noalloc(p, p, 64, 64, 576, 512, float("nan"), p) == mla.ERR_ARG
    assert b"softmax_scale" in lib.fst_cuda_mla_last_error()
    assert mla.attention_noalloc(p, p, 64, 64, 576, 512, float("inf"), p) == mla.ERR_ARG


def test_sizes_beyond_the_fixed_array_are_refused():
    d = torch.zeros(64 * 576, dtype=torch.int16, device="cuda")
    o = torch.zeros(64 * 512, dtype=torch.int16, device="cuda")
    p, q = d.data_ptr(), o.data_ptr()
    assert mla.attention_noalloc(p, p, 65537, 64, 576, 512, 0.07, q) == mla.ERR_CAPACITY
    assert mla.attention_noalloc(p, p, 64, 65, 576, 512, 0.07, q) == mla.ERR_CAPACITY
    assert mla.attention_noalloc(p, p, 64, 64, 584, 512, 0.07, q) == mla.ERR_CAPACITY
    assert mla.attention_noalloc(p, p, 64, 64, 576, 500, 0.07, q) == mla.ERR_ARG
    assert mla.attention_noalloc(0, p, 64, 64, 576, 512, 0.07, q) == mla.ERR_ARG
    assert mla.attention_noalloc(p, p, 0, 64, 576, 512, 0.07, q) == mla.ERR_ARG
