"""The GEMM tile engine through the C ABI, with the reference's own test patterns:
random-matrix cosine probe (randmat_test, src/fst_engine.cpp:586-685), ones @ identity
(tools/fst_gemm_probe.cpp:72-129), small-integer A @ B^T against the wrong-transpose
interpretation (scripts/fst_validate_gemms.py:42-87)."""
import numpy as np
import pytest

from fastar_b200 import mla, synth
from tests.helpers import cosine

pytestmark = pytest.mark.gpu

IMPLS = [("simt", mla.IMPL_SIMT), ("tensor", mla.IMPL_TENSOR)]


@pytest.fixture(scope="module", params=IMPLS, ids=[i[0] for i in IMPLS])
def ctx(request):
    c = mla.MlaContext(mla.make_config(n_pages=4, max_tokens=16, gemm_impl=request.param[1]))
    yield c
    c.close()


def ref_gemm(A_bits, B_bits, b_kn=False):
    A = synth.from_bf16_bits(A_bits).astype(np.float64)
    B = synth.from_bf16_bits(B_bits).astype(np.float64)
    return A @ (B if b_kn else B.T)


# the probe shapes of randmat_test: (K, N) for qc / wqb / ob / ffn-sized calls, M = 16
@pytest.mark.parametrize("K,N", [(4096, 1024), (1024, 2048), (8192, 2048), (4096, 2048), (2048, 2048)])
def test_random_matrix_probe(ctx, K, N):
    rng = np.random.default_rng(K * 7 + N)
    M = 16
    A = synth.to_bf16_bits(rng.uniform(-1, 1, (M, K)).astype(np.float32))
    B = synth.to_bf16_bits(rng.uniform(-1, 1, (N, K)).astype(np.float32))
    got = synth.from_bf16_bits(ctx.gemm(A, B))
    want = ref_gemm(A, B)
    c = cosine(got, want)
    ratio = np.linalg.norm(got) / np.linalg.norm(want)
    # the reference accepts cos >= 0.999 ("cos < 0.999 is a layout bug"); bf16 output rounding
    # alone keeps this path far above that
    assert c >= 0.99999, (K, N, c)
    assert abs(ratio - 1) < 1e-3
    assert np.max(np.abs(got - want)) <= 2.0 ** -8 * np.max(np.abs(want)) + 1e-6


def test_ones_at_identity(ctx):
    M, K = 16, 1024
    A = synth.to_bf16_bits(np.ones((M, K), np.float32))
    B = synth.to_bf16_bits(np.eye(K, dtype=np.float32))
    got = synth.from_bf16_bits(ctx.gemm(A, B))
    assert np.array_equal(got, np.ones((M, K), np.float32))


@pytest.mark.parametrize("M,K,N,seed", [(32, 4096, 2048, 1), (32, 2048, 4096, 2)])
def test_layout_discrimination(ctx, M, K, N, seed):
    rng = np.random.default_rng(seed)
    A = rng.integers(-2, 3, size=(M, K)).astype(np.float32)
    B = rng.integers(-2, 3, size=(N, K)).astype(np.float32)
    got = synth.from_bf16_bits(ctx.gemm(synth.to_bf16_bits(A), synth.to_bf16_bits(B)))
    correct = A @ B.T
    wrong = A @ B.reshape(K, N)
    err_c = np.max(np.abs(got - correct))
    err_w = np.max(np.abs(got - wrong))
    max_c = np.max(np.abs(correct)) + 1e-6
    assert err_c < 0.10 * max_c and err_c * 10 < err_w
    # small integers: fp32 accumulation is exact, only the bf16 store rounds
    assert err_c <= 2.0 ** -8 * max_c


@pytest.mark.parametrize("M,N,K", [(1, 1600, 4096), (3, 12288, 1024), (64, 1600, 4096), (64, 4096, 8192),
                                   (16, 100, 72), (130, 256, 320), (5, 128, 512)])
def test_shapes_with_tails(ctx, M, N, K):
    rng = np.random.default_rng(M * 131 + N)
    A = synth.to_bf16_bits(rng.standard_normal((M, K)).astype(np.float32))
    B = synth.to_bf16_bits((rng.standard_normal((N, K)) * 0.02).astype(np.float32))
    got = synth.from_bf16_bits(ctx.gemm(A, B))
    want = ref_gemm(A, B)
    assert cosine(got, want) >= 0.99999
    assert np.max(np.abs(got - want)) <= 2.0 ** -8 * np.max(np.abs(want)) + 1e-6


@pytest.mark.parametrize("M,K,N", [(9, 128, 512), (64, 128, 512), (3, 200, 136)])
def test_b_row_major_operand(ctx, M, K, N):
    # the qksv-style [K, N] operand (src/fst_engine.cpp:480)
    rng = np.random.default_rng(5 + M)
    A = synth.to_bf16_bits(rng.standard_normal((M, K)).astype(np.float32))
    B = synth.to_bf16_bits(rng.standard_normal((K, N)).astype(np.float32))
    got = synth.from_bf16_bits(ctx.gemm(A, B, b_kn=True))
    want = ref_gemm(A, B, b_kn=True)
    assert cosine(got, want) >= 0.99999
    assert np.max(np.abs(got - want)) <= 2.0 ** -8 * np.max(np.abs(want)) + 1e-6


def test_same_inputs_give_identical_bits(ctx):
    rng = np.random.default_rng(11)
    A = synth.to_bf16_bits(rng.standard_normal((64, 8192)).astype(np.float32))
    B = synth.to_bf16_bits((rng.standard_normal((4096, 8192)) * 0.02).astype(np.float32))
    a = ctx.gemm(A, B)
    b = ctx.gemm(A, B)
    assert np.array_equal(a, b)
