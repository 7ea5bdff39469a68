"""Failure paths that need no fault: a bounded device wait that runs out, the status word that
reports it, which kernel family ran, and two GPUs driven from one process."""
import numpy as np
import pytest

from fastar_b200 import mla, synth
from tests.helpers import check_close

pytestmark = pytest.mark.gpu


def small_ctx(**kw):
    cfg = mla.make_config(mla.PRESET_BASELINE, hidden=1024, q_lora=512, n_pages=16, max_tokens=2, max_seqs=2, **kw)
    ctx = mla.MlaContext(cfg)
    w = synth.layer_weights_f32(cfg, 0, 0)
    ctx.set_layer_weights(0, synth.weights_to_bits(w))
    return cfg, ctx


def one_step(cfg, ctx, seed=0):
    s = ctx.seq_alloc()
    ctx.cache_write(0, s, 0, synth.to_bf16_bits(synth.cache_rows_f32(cfg, seed, 0, 130)))
    h = synth.to_bf16_bits(synth.hidden_f32(cfg, seed, 1))
    out = ctx.forward(0, h, [s], [130], [1])
    ctx.seq_free(s)
    return out


def test_a_wait_that_runs_out_is_reported_and_the_context_stays_usable():
    """A tiny kernel waits on a barrier that nothing arrives at, with a limit of a few thousand
    polls; it gives up, records its status and returns.  The next sync reports
    FST_MLA_ERR_DEVICE_CHECK, clears the word, and the layer runs as before."""
    cfg, ctx = small_ctx()
    with ctx:
        before = one_step(cfg, ctx)
        ctx.selftest_wait_expiry(3000)
        with pytest.raises(mla.MlaError) as e:
            ctx.sync()
        assert e.value.code == mla.ERR_DEVICE_CHECK
        assert "status 5" in str(e.value)
        ctx.sync()  # the word was cleared
        after = one_step(cfg, ctx)
        assert np.array_equal(before, after)


def test_a_device_status_word_fails_the_next_call_once():
    cfg, ctx = small_ctx()
    with ctx:
        before = one_step(cfg, ctx)
        ctx.debug_set_status(3)
        s = ctx.seq_alloc()
        ctx.cache_write(0, s, 0, synth.to_bf16_bits(synth.cache_rows_f32(cfg, 0, 0, 130)))
        h = synth.to_bf16_bits(synth.hidden_f32(cfg, 0, 1))
        with pytest.raises(mla.MlaError) as e:
            ctx.forward(0, h, [s], [130], [1])
        assert e.value.code == mla.ERR_DEVICE_CHECK and "status 3" in str(e.value)
        ctx.seq_free(s)
        assert np.array_equal(one_step(cfg, ctx), before)


def test_auto_reports_which_kernel_family_ran():
    cfg, ctx = small_ctx()
    with ctx:
        one_step(cfg, ctx)
        fam = ctx.family_counts()
        assert fam["simt"] == 0 and fam["tensor"] >= 6  # five GEMMs and the attention
    cfg, ctx = small_ctx(attn_impl=mla.IMPL_SIMT, gemm_impl=mla.IMPL_SIMT)
    with ctx:
        one_step(cfg, ctx)
        fam = ctx.family_counts()
        assert fam["tensor"] == 0 and fam["simt"] >= 6
    # a head count the tcgen05 kernels do not cover: AUTO takes the CUDA-core attention, and says so
    cfg = mla.make_config(mla.PRESET_BASELINE, hidden=1024, q_lora=512, n_heads=16, n_pages=16, max_tokens=2, max_seqs=2)
    with mla.MlaContext(cfg) as ctx:
        ctx.set_layer_weights(0, synth.weights_to_bits(synth.layer_weights_f32(cfg, 0, 0)))
        one_step(cfg, ctx)
        assert ctx.family_counts()["simt"] >= 1


def test_two_devices_in_one_process():
    """One context per GPU, both in this process: the second device needs its own kernel
    attributes (more than 48 KB of dynamic shared memory) or its first launch fails."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    outs = []
    for dev in (0, 1):
        cfg, ctx = small_ctx(device=dev)
        with ctx:
            outs.append(one_step(cfg, ctx))
            assert ctx.family_counts()["simt"] == 0
    assert np.array_equal(outs[0], outs[1])
