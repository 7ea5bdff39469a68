"""The multi-GPU split-KV exchange on CPU ranks (gloo, world_size 2): page-aligned slices,
the [rows, 2 + d_v] partial layout, one all-gather, log-sum-exp merge == unsplit attention."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from fastar_b200 import parallel
from oracle import oracle as O


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, L, q_len, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        H = 4
        cfg = O.make_cfg(O.PRESET_BASELINE, n_heads=H, round_bf16=False, n_threads=1)
        rng = np.random.default_rng(7)  # every rank builds the same inputs, reads only its slice
        cache = rng.standard_normal((L + q_len, 576)).astype(np.float32)
        q = (rng.standard_normal((q_len * H, 576)) * 0.5).astype(np.float32)
        a, b = parallel.kv_slices(L + q_len, world)[rank]
        m, l, o = O.attention_partial(cfg, q, cache, a, b, q_len, pos0=L, causal=True)
        part = torch.from_numpy(parallel.pack_partial(m, l, o))
        gathered = torch.empty((world * part.shape[0], part.shape[1]), dtype=torch.float32)
        dist.all_gather_into_tensor(gathered, part)  # rank-major concatenation
        gm, gl, go = parallel.unpack_partials(gathered.numpy().reshape(world, *part.shape))
        merged = O.merge_partials(cfg, np.ascontiguousarray(gm), np.ascontiguousarray(gl),
                                  np.ascontiguousarray(go))
        want = O.attention(cfg, q, cache, L + q_len, q_len, pos0=L, causal=True)
        np.save(os.path.join(out_dir, f"err{rank}.npy"), np.array([np.max(np.abs(merged - want))]))
    finally:
        dist.destroy_process_group()


def test_split_kv_allgather_merge_matches_unsplit(tmp_path):
    for L, q_len in ((1000, 1), (130, 3), (10, 2)):
        mp.spawn(_worker, args=(2, _free_port(), L, q_len, str(tmp_path)), nprocs=2, join=True)
        for r in range(2):
            assert float(np.load(tmp_path / f"err{r}.npy")[0]) < 1e-5
