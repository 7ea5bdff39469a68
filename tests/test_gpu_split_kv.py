"""Split-KV across ranks on ONE GPU: two contexts stand in for two ranks and run one after the
other (no kernel waits on another), their partials are concatenated as an all-gather would,
and the merge + output projections must reproduce the unsplit layer of the CPU oracle."""
import numpy as np
import pytest
import torch

from fastar_b200 import mla, parallel, synth
from oracle import oracle as O
from tests.helpers import check_close, oracle_cfg
from tests.test_gpu_layer import weights_for

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("preset,L,world", [(mla.PRESET_BASELINE, 1000, 2), (mla.PRESET_BASELINE, 333, 3),
                                            (mla.PRESET_FASTAR_V4, 500, 2)], ids=["bl-2", "bl-3", "v4-2"])
def test_partials_merge_to_the_unsplit_layer(preset, L, world):
    bits, rounded = weights_for(preset)
    cfg0 = mla.make_config(preset)
    d = mla.dims_of(cfg0)
    H = cfg0.n_heads
    rows = synth.to_bf16_bits(synth.cache_rows_f32(cfg0, 3, 0, L))
    h = synth.to_bf16_bits(synth.hidden_f32(cfg0, 3, 1))
    slices = parallel.kv_slices(L, world)
    owner = parallel.owner_of_row(L, L, world)
    assert owner == world - 1
    ctxs, seqs = [], []
    d_h = torch.from_numpy(h.view(np.int16)).cuda()
    d_out = torch.empty_like(d_h)
    gathered = torch.zeros((world, H, 2 + d["d_v"]), dtype=torch.float32, device="cuda")
    try:
        for r, (a, b) in enumerate(slices):
            cfg = mla.make_config(preset, n_pages=(b - a) // 64 + 3, max_tokens=1, max_seqs=1)
            c = mla.MlaContext(cfg)
            c.set_layer_weights(0, bits)
            s = c.seq_alloc()
            if b > a:
                c.cache_write(0, s, 0, rows[a:b])
            ctxs.append(c)
            seqs.append(s)
            # local row = global - slice begin; RoPE uses the global position
            if r == owner:
                c.plan([(s, L - a, 1, L, 1)])
            else:
                c.plan([(s, b - a, 1, L, 0)])
            c.run_partial_device(0, d_h.data_ptr(), gathered[r].data_ptr())
            c.sync()
        for c in ctxs:  # every rank merges; all must agree
            c.run_merge_device(0, gathered.data_ptr(), world, d_out.data_ptr())
            c.sync()
            got = d_out.cpu().numpy().view(np.uint16)
            cache = np.zeros((L + 1, d["row"]), np.float32)
            cache[:L] = synth.from_bf16_bits(rows)
            want = O.mla_forward(oracle_cfg(cfg0), rounded, synth.from_bf16_bits(h), L, cache, want_trace=True)
            check_close(got, want.out, "merged output", ulps=2 if preset == mla.PRESET_FASTAR_V4 else 0)
        # the owner appended the new row at its local position, bit for bit the kv stage row
        a, b = slices[owner]
        new_row = ctxs[owner].cache_read(0, seqs[owner], L - a, 1)
        assert np.array_equal(new_row, ctxs[owner].get_stage(mla.STAGE_KV))
        check_close(new_row, want.trace["kv"], "appended row", ulps=2)
        for r in range(world):
            if r != owner:
                assert ctxs[r].seq_len(seqs[r]) == slices[r][1] - slices[r][0]
    finally:
        for c in ctxs:
            c.close()


def test_split_layer_call_through_the_c_abi_with_a_host_gather():
    """fst_cuda_mla_run_split_device (local partial -> all-gather -> merge + projections in ONE call)
    with the host-supplied transport: two contexts on one GPU stand in for two ranks; each rank's
    gather function lays its own partial and the other rank's (computed beforehand, so nothing waits
    on anything) side by side.  Both ranks must reproduce the unsplit layer of the oracle, and the
    host-buffer form (fst_cuda_mla_forward_split) the same bits."""
    try:
        from cuda.bindings import runtime as cudart
    except ImportError:
        from cuda import cudart
    preset, L, world = mla.PRESET_BASELINE, 3000, 2
    bits, rounded = weights_for(preset)
    cfg0 = mla.make_config(preset)
    d = mla.dims_of(cfg0)
    H = cfg0.n_heads
    rows = synth.to_bf16_bits(synth.cache_rows_f32(cfg0, 13, 0, L))
    h = synth.to_bf16_bits(synth.hidden_f32(cfg0, 13, 1))
    slices = parallel.kv_slices(L, world)
    owner = parallel.owner_of_row(L, L, world)
    d_h = torch.from_numpy(h.view(np.int16)).cuda()
    d_out = torch.empty_like(d_h)
    stash = torch.zeros((world, H, 2 + d["d_v"]), dtype=torch.float32, device="cuda")
    ctxs, seqs, steps = [], [], []
    try:
        for r, (a, b) in enumerate(slices):
            cfg = mla.make_config(preset, n_pages=(b - a) // 64 + 3, max_tokens=1, max_seqs=1)
            c = mla.MlaContext(cfg)
            c.set_stream(torch.cuda.current_stream().cuda_stream)
            c.set_layer_weights(0, bits)
            s = c.seq_alloc()
            c.cache_write(0, s, 0, rows[a:b])
            ctxs.append(c)
            seqs.append(s)
            steps.append((s, L - a, 1, L, 1) if r == owner else (s, b - a, 1, L, 0))
            c.plan([steps[r]])
            c.run_partial_device(0, d_h.data_ptr(), stash[r].data_ptr())
            c.sync()
        cache = np.zeros((L + 1, d["row"]), np.float32)
        cache[:L] = synth.from_bf16_bits(rows)
        want = O.mla_forward(oracle_cfg(cfg0), rounded, synth.from_bf16_bits(h), L, cache, want_trace=False).out
        for r, c in enumerate(ctxs):
            def gather(send, recv, nbytes, stream, r=r):
                for q in range(world):
                    src = send if q == r else stash[q].data_ptr()
                    (err,) = cudart.cudaMemcpyAsync(recv + q * nbytes, src, nbytes,
                                                    cudart.cudaMemcpyKind.cudaMemcpyDeviceToDevice, stream)
                    if int(err) != 0:
                        return 1
                return 0
            c.comm_set_gather(gather, r, world)
            c.plan([steps[r]])
            c.run_split_device(0, d_h.data_ptr(), d_out.data_ptr())
            c.sync()
            got = d_out.cpu().numpy().view(np.uint16).copy()
            check_close(got, want, f"rank {r}: split layer call")
            assert np.array_equal(c.forward_split(0, h, [steps[r]]), got)
            t = c.kernel_times()
            c.comm_destroy()
            with pytest.raises(mla.MlaError) as e:
                c.run_split_device(0, d_h.data_ptr(), d_out.data_ptr())
            assert e.value.code == mla.ERR_STATE
    finally:
        for c in ctxs:
            c.close()
