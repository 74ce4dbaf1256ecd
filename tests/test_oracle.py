"""CPU tests of the oracle itself: it must reproduce what the reference's own PyTorch model
(scripts/llm.py) computed for each linear layer — the fixtures under tests/golden/ — and agree
with an independent float64 matmul."""
import numpy as np
import pytest

from conftest import LAYERS, golden

FIXTURES = ["llm_tiny_aligned.npz", "llm_tiny_ragged.npz"]
# torch's CPU matmul sums in a different order than the reference kernels; fp32 rounding only
TOL_F32 = 2e-6
TOL_F64 = 1e-6  # float64 oracle vs the fp32 numbers torch stored


@pytest.mark.parametrize("fx", FIXTURES)
@pytest.mark.parametrize("layer", LAYERS)
def test_oracle_matches_reference_model(orc, fx, layer):
    z = golden(fx)
    x, w, y, dy, dx, dw = (z[f"{layer}.{k}"] for k in ("x", "w", "y", "dy", "dx", "dw"))
    b = z[f"{layer}.b"] if f"{layer}.b" in z else None
    for f64, tol in ((False, TOL_F32), (True, TOL_F64)):
        assert orc.max_rel_err(orc.forward(x, w, b, f64=f64), y) <= tol
        assert orc.max_rel_err(orc.backward_input(dy, w, f64=f64), dx) <= tol
        gw, gb = orc.backward_weight(dy, x, want_bias=b is not None, f64=f64)
        assert orc.max_rel_err(gw, dw) <= tol
        if b is not None:
            assert orc.max_rel_err(gb, z[f"{layer}.db"]) <= tol
        else:
            assert gb is None


@pytest.mark.parametrize("M,K,N", [(1, 1, 1), (3, 5, 7), (33, 31, 65), (128, 96, 40)])
def test_oracle_f64_is_exact_matmul(orc, M, K, N):
    rng = np.random.default_rng(M * 1000 + K * 10 + N)
    x = rng.standard_normal((M, K), dtype=np.float32)
    w = rng.standard_normal((K, N), dtype=np.float32)
    dy = rng.standard_normal((M, N), dtype=np.float32)
    b = rng.standard_normal(N, dtype=np.float32)
    x64, w64, dy64 = x.astype(np.float64), w.astype(np.float64), dy.astype(np.float64)
    assert np.allclose(orc.forward(x, w, b, f64=True), x64 @ w64 + b, rtol=1e-12, atol=1e-12)
    assert np.allclose(orc.backward_input(dy, w, f64=True), dy64 @ w64.T, rtol=1e-12, atol=1e-12)
    gw, gb = orc.backward_weight(dy, x, f64=True)
    assert np.allclose(gw, x64.T @ dy64, rtol=1e-12, atol=1e-12)
    assert np.allclose(gb, dy64.sum(0), rtol=1e-12, atol=1e-12)


def test_oracle_f32_is_sequential_fma(orc):
    """The fp32 flavour follows the reference's order: k ascending, one FMA per step."""
    rng = np.random.default_rng(5)
    x = rng.standard_normal((4, 37), dtype=np.float32)
    w = rng.standard_normal((37, 6), dtype=np.float32)
    got = orc.forward(x, w)
    want = np.zeros((4, 6), np.float32)
    for m in range(4):
        for n in range(6):
            acc = np.float32(0)
            for k in range(37):
                # fma in float64 then one rounding == fused multiply-add for fp32 inputs
                acc = np.float32(np.float64(x[m, k]) * np.float64(w[k, n]) + np.float64(acc))
            want[m, n] = acc
    assert np.array_equal(got, want)


def test_oracle_overwrites_and_null_bias(orc):
    x = np.ones((2, 3), np.float32)
    w = np.ones((3, 4), np.float32)
    assert np.array_equal(orc.forward(x, w, None), np.full((2, 4), 3, np.float32))
    gw, gb = orc.backward_weight(np.ones((2, 4), np.float32), x, want_bias=False)
    assert gb is None and np.array_equal(gw, np.full((3, 4), 2, np.float32))


def test_gelu_matches_formula(orc):
    x = np.linspace(-6, 6, 101, dtype=np.float32)
    want = 0.5 * x * (1 + np.tanh(np.sqrt(2 / np.pi) * (x + 0.044715 * x ** 3)))
    assert np.allclose(orc.gelu(x), want, atol=1e-6)


def test_gelu_gradient_matches_a_central_difference(orc):
    """the restated GELU backward (sech^2 form of the reference kernel) against d/dx of the forward"""
    x = np.linspace(-6, 6, 2001).astype(np.float32)
    g = np.full(x.shape, 1.5)
    h = 1e-4
    xd = x.astype(np.float64)
    k = np.sqrt(2 / np.pi)
    f = lambda v: 0.5 * v * (1 + np.tanh(k * (v + 0.044715 * v ** 3)))
    fd = (f(xd + h) - f(xd - h)) / (2 * h)
    assert np.allclose(orc.gelu_grad_mul(x, g), 1.5 * fd, atol=1e-7)
