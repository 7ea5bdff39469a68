"""B200 (sm_100a) implementation of the FaStar engine's Multi-head Latent Attention layer.

Only what that path needs: `csrc/` (CUDA kernels and the C ABI of include/fst_cuda_mla.h),
`host/` (the FSTEngine-shaped C++ host class), `mla` (ctypes binding), `synth` (seeded
benchmark inputs), `parallel` (sequence sharding and split-KV across GPUs), `build`.
"""
from . import mla  # noqa: F401

__all__ = ["mla"]
