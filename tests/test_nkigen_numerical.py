"""Numerical checks of the nkigen front end and the native pass pipeline: each kernel is traced with
`nkigen.trace`, verified against NumPy as traced, run through the complete pipeline (21 native passes) and verified
again, so every pass is semantics-preserving on it.  Kernel families follow the reference's nkigen/tests/{unit,e2e}
(broadcast, elementwise, reductions, matrix products incl. batched, gather, multi-output, rmsnorm, rope, attention,
feed-forward, sigmoid variants, for-loops)."""
import numpy as np
import pytest

import nkipy_b200.nkigen as ng

R = np.random.default_rng(21)


def f32(*s, scale=1.0):
    return (R.standard_normal(s) * scale).astype(np.float32)


def _rmsnorm(x, w):
    return x * (1.0 / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + 1e-6)) * w


def _rope(x, cos, sin):
    h = x.shape[-1] // 2
    a, b = x[..., :h], x[..., h:]
    return np.concatenate([a * cos - b * sin, b * cos + a * sin], axis=-1)


def _attention(q, k, v):
    s = np.matmul(q, np.transpose(k, (0, 2, 1))) * np.float32(0.25)
    e = np.exp(s - np.max(s, axis=-1, keepdims=True))
    return np.matmul(e / np.sum(e, axis=-1, keepdims=True), v)


def _ffn(x, wgu, wd):
    gu = x @ wgu
    g, u = np.split(gu, 2, axis=-1)
    return (g * (1.0 / (1.0 + np.exp(-g))) * u) @ wd


def _loop(x, w):
    def body(i, acc):
        return np.tanh(acc @ w) + x
    return ng.fori_loop(0, 3, body, x)


KERNELS = {
    # broadcast
    "bcast_row": (lambda a, b: a + b, [f32(8, 16), f32(16)]),
    "bcast_col": (lambda a, b: a * b, [f32(8, 16), f32(8, 1)]),
    "bcast_scalar": (lambda a: a * 2.5 - 1.0, [f32(8, 16)]),
    "bcast_3d": (lambda a, b: a - b, [f32(2, 8, 16), f32(8, 1)]),
    "bcast_both": (lambda a, b: a + b, [f32(8, 1), f32(1, 16)]),
    # elementwise
    "chain": (lambda a, b: np.tanh(a) * np.exp(-np.abs(b)) + np.sqrt(np.abs(a) + 1.0), [f32(8, 16), f32(8, 16)]),
    "sigmoid": (lambda a: 1.0 / (1.0 + np.exp(-a)), [f32(8, 16)]),
    "sigmoid_times": (lambda a, b: a / (1.0 + np.exp(-a)) * b, [f32(8, 16), f32(8, 16)]),
    "max_min_where": (lambda a, b: np.where(a > b, np.maximum(a, 0.0), np.minimum(b, 0.0)), [f32(8, 16), f32(8, 16)]),
    "elementwise_3d": (lambda a, b: (a + b) * (a - b), [f32(2, 4, 8), f32(2, 4, 8)]),
    "divide_power": (lambda a, b: (np.abs(a) + 1.0) ** 1.5 / (np.abs(b) + 0.5), [f32(8, 16), f32(8, 16)]),
    # reductions
    "sum_last": (lambda a: np.sum(a, axis=-1), [f32(8, 16)]),
    "sum_first_keep": (lambda a: np.sum(a, axis=0, keepdims=True), [f32(8, 16)]),
    "mean_max": (lambda a: np.mean(a, axis=-1) + np.max(a, axis=-1), [f32(8, 16)]),
    "sum_two_axes": (lambda a: np.sum(a, axis=(0, 2)), [f32(2, 8, 4)]),
    "sum_all": (lambda a: np.sum(a), [f32(8, 16)]),
    "softmax": (lambda a: np.exp(a - np.max(a, -1, keepdims=True)) / np.sum(np.exp(a - np.max(a, -1, keepdims=True)), -1, keepdims=True),
                [f32(8, 16)]),
    # matrix products
    "matmul": (lambda a, b: a @ b, [f32(8, 16), f32(16, 12)]),
    "matmul_add": (lambda a, b, c: a @ b + c, [f32(8, 16), f32(16, 12), f32(12)]),
    "matmul_add_relu": (lambda a, b, c: np.maximum(a @ b + c, 0.0), [f32(8, 16), f32(16, 12), f32(8, 12)]),
    "matmul_batched": (lambda a, b: np.matmul(a, b), [f32(3, 8, 16), f32(3, 16, 4)]),
    "matmul_transposed": (lambda a, b: a @ b.T, [f32(8, 16), f32(12, 16)]),
    "matmul_chain": (lambda a, b, c: (a @ b) @ c, [f32(8, 16), f32(16, 16), f32(16, 4)]),
    # gather
    "gather_rows": (lambda t, i: np.take(t, i, axis=0), [f32(32, 8), np.array([3, 0, 31, 7], np.int32)]),
    "gather_then_scale": (lambda t, i, s: np.take(t, i, axis=0) * s, [f32(32, 8), np.array([1, 1, 5], np.int32), f32(8)]),
    # multi-output and shape ops
    "two_outputs": (lambda a, b: (a + b, a * b), [f32(8, 16), f32(8, 16)]),
    "three_outputs": (lambda a: (np.sum(a, -1), np.max(a, -1), a * 2.0), [f32(8, 16)]),
    "head_split": (lambda a: np.transpose(a.reshape(2, 8, 4, 4), (0, 2, 1, 3)), [f32(2, 8, 16)]),
    "head_merge": (lambda a: np.transpose(a, (0, 2, 1, 3)).reshape(2, 8, 16), [f32(2, 4, 8, 4)]),
    "concat_split": (lambda a, b: np.split(np.concatenate([a, b], axis=-1), 4, axis=-1)[2], [f32(8, 8), f32(8, 8)]),
    # model blocks
    "rmsnorm": (_rmsnorm, [f32(8, 32), f32(32)]),
    "rope": (_rope, [f32(2, 8, 16), f32(8, 8), f32(8, 8)]),
    "attention": (_attention, [f32(2, 8, 16), f32(2, 8, 16), f32(2, 8, 16)]),
    "feed_forward": (_ffn, [f32(8, 16), f32(16, 64, scale=0.3), f32(32, 16, scale=0.3)]),
    "layer": (lambda x, w, wgu, wd: x + _ffn(_rmsnorm(x, w), wgu, wd), [f32(8, 16), f32(16), f32(16, 64, scale=0.3),
                                                                       f32(32, 16, scale=0.3)]),
    # comparisons, selection, logic
    "equal": (lambda a, b: np.equal(a, b), [np.array([[1, 2], [3, 4]], np.float32), np.array([[1, 0], [3, 5]], np.float32)]),
    "greater": (lambda a, b: np.greater(a, b), [f32(8, 16), f32(8, 16)]),
    "less_scalar": (lambda a: np.less(a, 0.25), [f32(8, 16)]),
    "logical_not": (lambda a: np.logical_not(a > 0.0), [f32(8, 16)]),
    "bitwise_and": (lambda a, b: np.bitwise_and(a, b), [R.integers(0, 255, (8, 16)).astype(np.int32),
                                                        R.integers(0, 255, (8, 16)).astype(np.int32)]),
    "where_same_type": (lambda c, a, b: np.where(c > 0.0, a, b), [f32(8, 16), f32(8, 16), f32(8, 16)]),
    "where_scalar_branch": (lambda a: np.where(a > 0.5, a, 0.0), [f32(8, 16)]),
    "clip": (lambda a: np.clip(a, -0.5, 0.5), [f32(8, 16)]),
    # more shape ops
    "squeeze": (lambda a: np.squeeze(a, axis=1) * 2.0, [f32(8, 1, 16)]),
    "swapaxes": (lambda a: np.swapaxes(a, 0, 2) + 1.0, [f32(2, 8, 4)]),
    "stack": (lambda a, b: np.stack([a, b], axis=1), [f32(8, 16), f32(8, 16)]),
    "expand_then_broadcast": (lambda a, b: np.expand_dims(a, 1) * b, [f32(8, 16), f32(4, 16)]),
    # loops
    "fori_loop": (_loop, [f32(8, 8, scale=0.5), f32(8, 8, scale=0.5)]),
}


def _specs(inputs):
    names = {np.dtype(np.float32): "f32", np.dtype(np.int32): "i32"}
    return [(a.shape, names[a.dtype]) for a in inputs]


def _numpy_only(fn):
    """The same function with the loop construct replaced by a Python loop, as the NumPy oracle."""
    if fn is _loop:
        def plain(x, w):
            acc = x
            for _ in range(3):
                acc = np.tanh(acc @ w) + x
            return acc
        return plain
    return fn


@pytest.mark.parametrize("name", sorted(KERNELS))
def test_traced_and_fully_lowered_graphs_match_numpy(name):
    fn, inputs = KERNELS[name]
    traced = ng.trace(fn, input_specs=_specs(inputs))
    ir0 = traced.to_ir()
    oracle = _numpy_only(fn)
    assert ng.verify_against_numpy(oracle, ir0, inputs, rtol=2e-4, atol=2e-5), "traced graph differs from NumPy"
    ir1 = ng.apply_complete_knob_pipeline(ir0)
    assert ng.verify_against_numpy(oracle, ir1, inputs, rtol=2e-4, atol=2e-5), "graph after the pipeline differs from NumPy"
    assert "_mem" in ir1 or "_tiling" in ir1 or "_buffer" in ir1          # the passes left their decisions on the graph


def test_the_loop_stays_a_loop_until_it_is_expanded():
    fn, inputs = KERNELS["fori_loop"]
    ir0 = ng.trace(fn, input_specs=_specs(inputs)).to_ir()
    assert "loop" in ir0 and ir0.count("tanh") == 1                      # the body is traced once
