"""One rank of the multi-GPU checks (launched by tests/test_gpu_multi.py under torch.distributed.run,
one process per GPU).  torch.distributed (gloo) is only the plumbing that hands the communicator id
and the results around; the data path is the library's own: sequence sharding has no collective,
split-KV exchanges its partials with the NCCL all-gather inside fst_cuda_mla_run_split_device."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from fastar_b200 import mla, parallel, synth, workloads  # noqa: E402
from oracle import oracle as O  # noqa: E402
from tests.helpers import check_close, oracle_cfg  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("gloo", rank=rank, world_size=world)

    # ---- one long sequence split along the KV axis, exchange through the C ABI (NCCL) ----
    L = 20000
    wl = workloads.build("longctx", rank=rank, world=world, device=local, ctx_lo=L, ctx_hi=L)
    ctx = wl.ctx
    uid = [mla.comm_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(uid, src=0)
    ctx.comm_init(uid[0], rank, world)
    owner = parallel.owner_of_row(L, L, world)
    s = wl.seqs[0]
    step = (s, L - wl.slice_begin, 1, L, 1) if rank == owner else (s, wl.rows[0], 1, L, 0)
    got = ctx.forward_split(0, wl.h_bits, [step])
    cache = np.zeros((L + 1, 576), np.float32)
    cache[:L] = synth.from_bf16_bits(synth.to_bf16_bits(synth.cache_rows_f32(wl.cfg, 0, 0, L)))
    w = synth.weights_rounded(synth.layer_weights_f32(wl.cfg, 0, 0))
    want = O.mla_forward(oracle_cfg(wl.cfg), w, synth.from_bf16_bits(wl.h_bits), L, cache)
    check_close(got, want.out, f"rank {rank}: split-KV layer over {world} GPUs")
    if rank == owner:
        check_close(ctx.cache_read(0, s, L - wl.slice_begin, 1), want.trace["kv"], "appended row", ulps=2)
    outs = [None] * world
    dist.all_gather_object(outs, got.tobytes())
    assert all(o == outs[0] for o in outs), "the ranks disagree on the merged output"
    ctx.comm_destroy()
    wl.close()

    # ---- one batch sharded by sequence (no collective): every rank its share, rank 0 checks all ----
    B = 16
    wl = workloads.build("batched", rank=rank, world=world, sharding="strong", device=local, batch=B, ctx_lo=100,
                         ctx_hi=3000)
    out = wl.ctx.forward(0, wl.h_bits, wl.seqs, wl.rows, [1] * len(wl.seqs))
    shards = [None] * world
    dist.all_gather_object(shards, (wl.global_index, out.tobytes()))
    if rank == 0:
        full = np.zeros((B, wl.cfg.hidden), np.uint16)
        seen = []
        for idx, raw in shards:
            full[idx] = np.frombuffer(raw, np.uint16).reshape(len(idx), -1)
            seen += list(idx)
        assert sorted(seen) == list(range(B)), "the shards do not cover the batch exactly once"
        lens = [int(x) for x in wl.all_lens]
        caches = []
        for b in range(B):
            c = np.zeros((lens[b] + 1, 576), np.float32)
            c[:lens[b]] = synth.from_bf16_bits(synth.to_bf16_bits(synth.cache_rows_f32(wl.cfg, 0, b, lens[b])))
            caches.append(c)
        hf = synth.from_bf16_bits(synth.to_bf16_bits(synth.hidden_f32(wl.cfg, 0, B, (0,))))
        r = O.mla_forward_batch(oracle_cfg(wl.cfg), w, hf, [1] * B, lens, caches)
        check_close(full, r.out, "batch sharded by sequence")
    wl.close()
    dist.barrier()
    print(f"MGPU_OK rank {rank}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
