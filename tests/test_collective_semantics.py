"""Collective operations of the frontend on one process, under the convention that every rank of the group holds the
same data: direct mode (NumPy) and the interpreted trace agree, shapes follow the group size, reduction kinds are
recorded in the graph.  Cases follow the reference's tests/unit/test_collectives.py."""
import numpy as np
import pytest

import nkipy_b200.distributed.collectives as cc
from utils import check, trace_kernel

R = np.random.default_rng(5)
X = (R.random((16, 32)) + 0.5).astype(np.float32)
G2 = [[0, 1]]
G4 = [[0, 1, 2, 3]]


def _ops(g):
    return [n.opcode for n in g.nodes]


@pytest.mark.parametrize("groups,n", [(G2, 2), (G4, 4)])
def test_all_reduce_sums_the_copies(groups, n):
    k = lambda x: cc.all_reduce(x, replica_groups=groups, reduce_op=np.add)
    np.testing.assert_allclose(k(X), X * n, rtol=1e-6)
    g = check(k, X)
    assert "all_reduce" in _ops(g)


@pytest.mark.parametrize("op,expect", [(np.maximum, lambda x: x), (np.minimum, lambda x: x), (np.multiply, lambda x: x ** 2)])
def test_all_reduce_kinds(op, expect):
    k = lambda x: cc.all_reduce(x, replica_groups=G2, reduce_op=op)
    np.testing.assert_allclose(k(X), expect(X), rtol=1e-6)
    g = check(k, X)
    node = next(n for n in g.nodes if n.opcode == "all_reduce")
    assert node.attrs["op"] == {np.maximum: "maximum", np.minimum: "minimum", np.multiply: "multiply"}[op]
    assert node.attrs["replica_groups"] == G2


def test_all_reduce_with_an_unknown_kind_returns_a_copy_in_direct_mode():
    out = cc.all_reduce(X, replica_groups=G2, reduce_op=np.subtract)
    np.testing.assert_array_equal(out, X)
    assert out is not X


@pytest.mark.parametrize("dim", [0, 1, -1])
def test_all_gather_concatenates_along_the_dimension(dim):
    k = lambda x: cc.all_gather(x, all_gather_dim=dim, replica_groups=G2)
    out = k(X)
    np.testing.assert_array_equal(out, np.concatenate([X, X], axis=dim))
    g = check(k, X)
    assert tuple(g.outputs[0].shape) == out.shape


@pytest.mark.parametrize("dim", [0, 1])
@pytest.mark.parametrize("groups,n", [(G2, 2), (G4, 4)])
def test_reduce_scatter_keeps_the_first_part_reduced(dim, groups, n):
    k = lambda x: cc.reduce_scatter(x, reduce_scatter_dim=dim, replica_groups=groups, reduce_op=np.add)
    out = k(X)
    np.testing.assert_allclose(out, np.split(X, n, axis=dim)[0] * n, rtol=1e-6)
    check(k, X)


@pytest.mark.parametrize("op,expect", [(np.maximum, lambda p: p), (np.multiply, lambda p: p ** 2), (np.subtract, lambda p: p)])
def test_reduce_scatter_kinds(op, expect):
    k = lambda x: cc.reduce_scatter(x, reduce_scatter_dim=0, replica_groups=G2, reduce_op=op)
    out = k(X)
    assert out.shape == (8, 32)
    np.testing.assert_allclose(out, expect(X[:8]), rtol=1e-6)
    if op is not np.subtract:
        check(k, X)


def test_reduce_scatter_needs_a_divisible_dimension():
    with pytest.raises((ValueError, TypeError)):
        trace_kernel(lambda x: cc.reduce_scatter(x, reduce_scatter_dim=0, replica_groups=[[0, 1, 2]], reduce_op=np.add), X)


def test_all_to_all_moves_the_split_dimension_into_the_concat_dimension():
    k = lambda x: cc.all_to_all(x, split_dimension=1, concat_dimension=0, replica_groups=G2)
    out = k(X)
    assert out.shape == (32, 16)
    np.testing.assert_array_equal(out, np.concatenate([X[:, :16], X[:, :16]], axis=0))   # what rank 0 receives
    g = check(k, X)
    node = next(n for n in g.nodes if n.opcode == "all_to_all")
    assert (node.attrs["split_dim"], node.attrs["concat_dim"]) == (1, 0)


def test_all_to_all_on_one_dimension_keeps_the_shape():
    k = lambda x: cc.all_to_all(x, split_dimension=0, concat_dimension=0, replica_groups=G4)
    assert k(X).shape == X.shape
    check(k, X)


def test_collectives_compose_with_arithmetic():
    w = (R.random((16, 32)) + 0.5).astype(np.float32)

    def k(x, w):
        part = x * w
        full = cc.all_reduce(part, replica_groups=G2, reduce_op=np.add)
        rows = cc.all_gather(full + 1.0, all_gather_dim=0, replica_groups=G2)
        return cc.reduce_scatter(rows, reduce_scatter_dim=0, replica_groups=G2, reduce_op=np.add) * 0.5

    np.testing.assert_allclose(k(X, w), (X * w) * 2 + 1.0, rtol=1e-5)
    g = check(k, X, w)
    assert [o for o in _ops(g) if o in ("all_reduce", "all_gather", "reduce_scatter")] == ["all_reduce", "all_gather",
                                                                                            "reduce_scatter"]


def test_a_traced_collective_marks_the_graph_as_needing_a_group():
    g = trace_kernel(lambda x: cc.all_reduce(x, replica_groups=G2, reduce_op=np.add), X)
    text = g.to_text()
    assert "replica_groups" in text and "all_reduce" in text
