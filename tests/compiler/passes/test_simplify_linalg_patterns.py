"""simplify-linalg, pattern by pattern: transposes, slices, broadcasts and concatenations compose; data movement that
moves nothing (transposes of unit dimensions, reductions over unit dimensions, full slices) becomes a view; a view of
a broadcast scalar is a broadcast.  Results are compared bit for bit with direct mode."""
import numpy as np
import pytest

from nkipy_b200.nkigen import trace

from ..harness import filecheck, ir_after, run_kernel_test

R = np.random.default_rng(9)
X = R.standard_normal((8, 16)).astype(np.float32)
C = R.standard_normal((2, 4, 6)).astype(np.float32)
EXACT = dict(rtol=0, atol=0)


def run(fn, inputs, check):
    k = trace(input_specs=[(a.shape, "f32") for a in inputs])(fn)
    return run_kernel_test(k, inputs, passes=["simplify-linalg"], check=check, **EXACT)


def test_transposes_compose_and_cancel():
    g = run(lambda c: np.transpose(np.transpose(c, (1, 2, 0)), (2, 0, 1)) + 1.0, [C], "CHECK-NOT: transpose(\nCHECK: add(")
    assert len(g.nodes) == 3                                           # constant, broadcast, add
    g = run(lambda c: np.transpose(np.transpose(c, (1, 2, 0)), (1, 0, 2)), [C], "CHECK-COUNT-1: transpose(")
    (t,) = [n for n in g.nodes if n.opcode == "transpose"]
    assert t.attrs["perm"] == [2, 1, 0] and t.inputs[0] is g.params[0]


@pytest.mark.parametrize("shape,perm", [((8, 1, 16), (1, 0, 2)), ((1, 8, 16), (1, 2, 0)), ((8, 1, 1, 16), (2, 0, 3, 1)),
                                        ((1, 1, 8), (2, 0, 1))])
def test_a_transpose_of_unit_dimensions_is_a_reshape(shape, perm):
    x = R.standard_normal(shape).astype(np.float32)
    g = run(lambda a: np.transpose(a, perm) * 2.0, [x], "CHECK-NOT: transpose(\nCHECK: reshape(")
    assert tuple(g.results[0].shape) == tuple(shape[p] for p in perm)


def test_a_transpose_that_moves_data_stays():
    run(lambda a: np.transpose(a, (1, 0, 2)), [R.standard_normal((8, 2, 1)).astype(np.float32)], "CHECK: transpose(")


@pytest.mark.parametrize("fn", [lambda a: np.sum(a.reshape(8, 1, 16), axis=1), lambda a: np.max(a.reshape(1, 8, 16), axis=0),
                                lambda a: np.min(a.reshape(8, 16, 1, 1), axis=(2, 3)), lambda a: np.prod(a.reshape(8, 1, 16), axis=1)],
                         ids=["sum", "max", "min", "prod"])
def test_a_reduction_over_unit_dimensions_is_a_reshape(fn):
    g = run(lambda a: fn(a) + 1.0, [X], "CHECK-NOT: reduce(\nCHECK: add(")
    assert "reduce" not in [n.opcode for n in g.nodes]                 # the reshapes left over go in the next pass
    full = ir_after(trace(input_specs=[((8, 16), "f32")])(lambda a: fn(a) + 1.0), passes=["simplify-linalg", "canonicalize-reshape"])
    filecheck(full, "CHECK-NOT: reshape(\nCHECK-NOT: reduce(\nCHECK: add(")


def test_a_reduction_over_a_real_dimension_stays():
    run(lambda a: np.sum(a.reshape(8, 2, 8), axis=1), [X], "CHECK: reduce(")


def test_slices_compose():
    g = run(lambda a: a[1:7:2, 2:14][0:2, 1:9:3], [X], "CHECK-COUNT-1: slice(")
    (s,) = [n for n in g.nodes if n.opcode == "slice"]
    assert s.attrs["start"] == [1, 3] and s.attrs["stride"] == [2, 3] and s.inputs[0] is g.params[0]
    assert tuple(s.outputs[0].shape) == (2, 3)
    run(lambda a: a[::2][::2][1:], [X], "CHECK-COUNT-1: slice(")
    run(lambda a: a[:, 4:][:, :4][2:6], [X], "CHECK-COUNT-1: slice(")


def test_a_slice_of_a_slice_with_another_reader_keeps_both_values_right():
    def k(a):
        inner = a[2:8]
        return inner[1:3] * 2.0, inner + 1.0

    run(k, [X], "CHECK-COUNT-2: slice(")


def test_broadcasts_compose():
    v = R.standard_normal(16).astype(np.float32)
    g = run(lambda b: np.broadcast_to(np.broadcast_to(b, (4, 16)), (3, 4, 16)) * 1.5, [v], "CHECK-COUNT-2: broadcast(")
    wide = [n for n in g.nodes if n.opcode == "broadcast" and n.inputs[0] is g.params[0]]
    assert len(wide) == 1 and wide[0].attrs["dims"] == [2] and tuple(wide[0].outputs[0].shape) == (3, 4, 16)


def test_views_of_a_broadcast_scalar_are_broadcasts():
    from nkipy_b200.core.tensor_apis import constant

    def traced(a):
        s = constant(np.float32(3.0))
        wide = np.broadcast_to(s, (16, 8))
        return a + np.transpose(wide, (1, 0)) + np.broadcast_to(s, (4, 32)).reshape(8, 16) + np.broadcast_to(s, (9, 20))[1:, 4:]

    text = ir_after(trace(input_specs=[((8, 16), "f32")])(traced), passes=["simplify-linalg"])
    filecheck(text, "CHECK-NOT: transpose(\nCHECK-NOT: reshape(\nCHECK-NOT: slice(\nCHECK: add(")
    from nkipy_b200.core.interp import evaluate
    from nkipy_b200.core.ir import Graph

    np.testing.assert_array_equal(evaluate(Graph.from_text(text), [X])[0], ((X + np.float32(3)) + np.float32(3)) + np.float32(3))


def test_nested_concatenations_flatten():
    g = run(lambda a: np.concatenate([np.concatenate([a, a * 2.0], axis=0), a], axis=0), [X], "CHECK-COUNT-1: concat(")
    (c,) = [n for n in g.nodes if n.opcode == "concat"]
    assert len(c.inputs) == 3 and tuple(c.outputs[0].shape) == (24, 16)
    # different axes do not mix; an inner result that is read elsewhere stays
    run(lambda a: np.concatenate([np.concatenate([a, a], axis=1)[:, :16], a], axis=0), [X], "CHECK-COUNT-2: concat(")

    def shared(a):
        inner = np.concatenate([a, a], axis=0)
        return np.concatenate([inner, a], axis=0), inner * 2.0

    run(shared, [X], "CHECK-COUNT-2: concat(")


def test_rewrites_feed_one_another():
    # transpose of a unit dimension -> reshape; the sum over the unit dimension -> reshape: no data movement is left
    def k(a):
        t = np.transpose(a.reshape(8, 1, 16), (1, 0, 2))
        return np.sum(t, axis=0) * 2.0

    text = ir_after(trace(input_specs=[((8, 16), "f32")])(k), passes=["simplify-linalg", "canonicalize-reshape"])
    filecheck(text, "CHECK-NOT: transpose(\nCHECK-NOT: reduce(\nCHECK-NOT: reshape(\nCHECK: mul(")
