"""Where direct mode (NumPy) and the traced graph may differ: half-precision contractions.

NumPy multiplies float16 matrices with float16 intermediate sums; the traced graph accumulates every
contraction in float32 and rounds once, which is what the tensor cores do.  With float32 inputs the two agree
to rounding; with float16 inputs that overflow or cancel (weights ~ N(0, 1) over a 2048-long contraction) single
elements differ by several percent -- rounding order, not a promotion difference: the result dtypes agree
and the graph equals the float32-accumulated product bit for bit."""
import numpy as np
import pytest

from nkipy_b200.core.compile import trace
from nkipy_b200.core.interp import evaluate


def mlp(x, w1, w2):
    h = np.matmul(x, w1)
    return np.matmul(h * (1.0 / (1.0 + np.exp(-h))), w2)


def test_float32_graph_matches_direct_mode():
    rng = np.random.default_rng(0)
    x, w1, w2 = (rng.standard_normal(s).astype(np.float32) for s in ((4, 512), (512, 1024), (1024, 256)))
    (got,) = evaluate(trace(mlp).specialize(x, w1, w2), [x, w1, w2])
    np.testing.assert_allclose(got, mlp(x, w1, w2), rtol=2e-4, atol=2e-3)


def test_float16_contractions_accumulate_in_float32():
    rng = np.random.default_rng(1)
    a = rng.standard_normal((8, 2048)).astype(np.float16)
    b = rng.standard_normal((2048, 64)).astype(np.float16)
    (got,) = evaluate(trace(lambda p, q: np.matmul(p, q)).specialize(a, b), [a, b])
    assert got.dtype == np.float16 == np.matmul(a, b).dtype                 # same promotion as NumPy
    exact = np.matmul(a.astype(np.float32), b.astype(np.float32)).astype(np.float16)
    assert np.array_equal(got, exact)                                       # one rounding, after the sum
    # NumPy's own float16 product of the same operands is the less accurate of the two
    ref = np.matmul(a.astype(np.float64), b.astype(np.float64))
    err_graph = np.abs(got.astype(np.float64) - ref).max()
    err_numpy = np.abs(np.matmul(a, b).astype(np.float64) - ref).max()
    assert err_graph <= err_numpy + 1e-6


@pytest.mark.parametrize("scale", [0.02, 0.05])
def test_float16_graph_stays_close_to_direct_mode_on_scaled_weights(scale):
    rng = np.random.default_rng(2)
    x = rng.standard_normal((4, 512)).astype(np.float16)
    w1 = (rng.standard_normal((512, 1024)) * scale).astype(np.float16)
    w2 = (rng.standard_normal((1024, 256)) * scale).astype(np.float16)
    (got,) = evaluate(trace(mlp).specialize(x, w1, w2), [x, w1, w2])
    want = mlp(x, w1, w2)
    assert got.dtype == want.dtype == np.float16
    np.testing.assert_allclose(got.astype(np.float32), want.astype(np.float32), rtol=2e-2, atol=2e-2)
