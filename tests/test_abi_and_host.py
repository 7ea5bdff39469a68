"""CPU-side checks: the C-ABI library loads and exports every symbol its header declares, and
refuses to run without a GPU (no CPU fallback); host-side sharding logic."""
import ctypes
import os
import re

import numpy as np
import pytest

from fastar_b200 import mla, parallel, synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = []
    for fn in sorted(os.listdir(os.path.join(ROOT, "include"))):
        text = open(os.path.join(ROOT, "include", fn)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names += re.findall(r"\b(fst_cuda_\w+)\s*\(", text)
    return sorted(set(names))


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(mla.LIB_PATH)
    names = declared_symbols()
    assert len(names) >= 30
    for n in names:
        assert hasattr(lib, n), n


def test_no_gpu_means_no_context():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(mla.MlaError) as e:
        mla.MlaContext(mla.make_config())
    assert e.value.code == mla.ERR_NO_DEVICE
    assert "no CPU fallback" in str(e.value)


def test_bad_config_is_rejected():
    lib = mla.load_library()
    h = ctypes.c_void_p()
    for kw in ({"n_pages": 0}, {"qk_rope": 63}, {"n_layers": 0}, {"preset": 5}):
        cfg = mla.make_config(**kw)
        assert lib.fst_cuda_mla_create(ctypes.byref(cfg), ctypes.byref(h)) == mla.ERR_ARG
        assert not h.value
    assert lib.fst_cuda_mla_create(None, ctypes.byref(h)) == mla.ERR_ARG
    assert lib.fst_cuda_mla_sync(None) == mla.ERR_ARG
    assert b"null" in lib.fst_cuda_mla_last_error()


def test_bf16_helpers_round_to_nearest_even():
    from oracle import oracle as O
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.standard_normal(1000).astype(np.float32),
                        np.array([1.00390625, 1.01171875, -1.00390625, 0.0, 65504.0], np.float32)])
    assert np.array_equal(synth.to_bf16_bits(x), O.to_bf16_bits(x))
    assert np.array_equal(synth.from_bf16_bits(synth.to_bf16_bits(x)), O.bf16_round(x))
    # ties go to the even mantissa
    assert synth.to_bf16_bits(np.array([1.00390625], np.float32))[0] == 0x3F80
    assert synth.to_bf16_bits(np.array([1.01171875], np.float32))[0] == 0x3F82


def test_synthetic_inputs_do_not_depend_on_sharding():
    cfg = mla.make_config()
    a = synth.cache_rows_f32(cfg, 0, 5, 100)
    b = synth.cache_rows_f32(cfg, 0, 5, 100)
    c = synth.cache_rows_f32(cfg, 0, 6, 100)
    assert np.array_equal(a, b) and not np.array_equal(a, c)
    assert abs(float(a.std()) - 1.0) < 0.02
    w = synth.normal_f32(0, "wq_a", (256, 256), 0.02, (0,))
    assert abs(float(w.std()) - 0.02) < 0.001


def test_shard_sequences_balances_rows():
    lens = synth.context_lengths(0, 64, 1024, 8192)
    assert lens.min() >= 1024 and lens.max() <= 8192
    for world in (1, 2, 4, 8):
        sh = parallel.shard_sequences(lens, world)
        assert sorted(i for s in sh for i in s) == list(range(64))
        loads = [int(sum(lens[i] for i in s)) for s in sh]
        assert max(loads) - min(loads) <= 8192


def test_kv_slices_are_page_aligned_and_cover():
    for n, world in ((131072, 8), (131072, 2), (1000, 4), (64, 8), (1, 2), (0, 4)):
        sl = parallel.kv_slices(n, world)
        assert sl[0][0] == 0 and sl[-1][1] == n
        for (a, b), (c, d) in zip(sl, sl[1:]):
            assert b == c and a <= b
        for a, b in sl[:-1]:
            assert a % 64 == 0 and b % 64 == 0
    assert parallel.owner_of_row(131072, 131072, 8) == 7
    assert parallel.owner_of_row(0, 131072, 8) == 0


def test_engine_library_loads_and_exports_its_entry_points():
    lib = ctypes.CDLL(os.path.join(os.path.dirname(mla.LIB_PATH), "libfst_engine.so"))
    for n in ("fst_engine_create", "fst_engine_destroy", "fst_engine_set_weight", "fst_engine_preload",
              "fst_engine_process_mla", "fst_engine_process_mla_batch", "fst_engine_reset_session",
              "fst_engine_rollback", "fst_engine_set_window", "fst_engine_randmat_test", "fst_engine_last_error",
              "fst_engine_load_shared_weights", "fst_engine_load_norm_override", "fst_file_read_tensor"):
        assert hasattr(lib, n), n
    import torch
    if not torch.cuda.is_available():
        lib.fst_engine_create.restype = ctypes.c_void_p
        lib.fst_engine_last_error.restype = ctypes.c_char_p
        assert not lib.fst_engine_create(1, 1, 128, 1, 16, 0, 0, 0)
        assert b"no CPU fallback" in lib.fst_engine_last_error()


def test_kernel_attributes_are_tracked_per_device():
    """Function attributes belong to the device that is current when they are set, so the library
    sets them once per (kernel, device): a second device must be told again, a larger request on
    the same device too, a repeat must not."""
    lib = mla.load_library()
    f = lib.fst_cuda_mla_debug_attr_first_use
    k1, k2 = 0x7E570001, 0x7E570002  # stand-ins for two kernel addresses
    assert f(k1, 0, 100_000) == 1
    assert f(k1, 0, 100_000) == 0      # same kernel, same device: nothing to do
    assert f(k1, 1, 100_000) == 1      # the second device has not been told yet
    assert f(k1, 1, 100_000) == 0
    assert f(k2, 0, 50_000) == 1       # another kernel
    assert f(k1, 0, 80_000) == 0       # a smaller request is covered
    assert f(k1, 0, 200_000) == 1      # a larger one is not
    assert f(k1, 1, 150_000) == 1


def test_strong_sharding_covers_the_batch_once():
    from fastar_b200 import workloads
    lens = synth.context_lengths(0, 64, 1024, 8192, (0,))
    for world in (2, 4, 8):
        shards = parallel.shard_sequences(lens, world)
        assert sorted(i for s in shards for i in s) == list(range(64))
    b, q, lo, hi, causal, _ = workloads.shape("verify")
    assert (b, q, lo, hi, causal) == (32, 16, 16384, 16384, True)
    assert workloads.shape("batched", batch=8)[0] == 8
