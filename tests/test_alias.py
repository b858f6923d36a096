"""Aliasing rules of traced kernels: a parameter that the kernel writes through becomes an output that shares its
buffer with the input (the reference's tests/unit/test_alias.py: single / multiple aliases, mutation without a
return value, mutated parameters mixed with fresh results, naming of inputs and outputs)."""
import numpy as np

from nkipy_b200.core.compile import trace
from nkipy_b200.core.interp import evaluate

A = np.arange(12, dtype=np.float32).reshape(3, 4)
B = np.ones((3, 4), np.float32)


def _graph(fn, *args):
    return trace(fn).specialize(*[a.copy() for a in args])


def test_mutation_without_return_yields_the_parameter_as_the_only_output():
    def kernel(a, b):
        a[0] = b[0] * 2.0

    g = _graph(kernel, A, B)
    assert [o.name for o in g.outputs] == ["a"]
    (al,) = g.aliases
    assert (al.output_index, al.param_index, al.param_name, al.is_user_returned) == (0, 0, "a", False)
    assert g.auto_aliased_indices == {0}                       # added by the tracer, not returned by the user
    assert [p.name for p in g.params] == ["a.must_alias_input", "b"]
    want = A.copy()
    want[0] = 2.0
    np.testing.assert_allclose(evaluate(g, [A.copy(), B.copy()])[0], want)


def test_several_parameters_can_be_aliased():
    def kernel(a, b):
        a[:, 0] = 5.0
        b[1] = a[1] + 1.0

    g = _graph(kernel, A, B)
    assert [o.name for o in g.outputs] == ["a", "b"]
    assert [(x.output_index, x.param_index) for x in g.aliases] == [(0, 0), (1, 1)]
    out_a, out_b = evaluate(g, [A.copy(), B.copy()])
    wa = A.copy()
    wa[:, 0] = 5.0
    wb = B.copy()
    wb[1] = wa[1] + 1.0
    np.testing.assert_allclose(out_a, wa)
    np.testing.assert_allclose(out_b, wb)


def test_fresh_results_come_first_and_are_numbered_mutated_parameters_follow_by_name():
    def kernel(a, b):
        a[0] = 1.0
        b[:, 1] = 2.0
        return a + b, a * 3.0

    g = _graph(kernel, A, B)
    assert [o.name for o in g.outputs] == ["output0", "output1", "a", "b"]
    assert g.auto_aliased_indices == {2, 3}


def test_a_returned_mutated_parameter_is_an_alias_the_user_asked_for():
    def kernel(a, b):
        a[2] = b[2]
        return a

    g = _graph(kernel, A, B)
    assert [o.name for o in g.outputs] == ["a"]
    (al,) = g.aliases
    assert al.is_user_returned and g.auto_aliased_indices == set()


def test_reading_a_parameter_does_not_alias_it():
    def kernel(a, b):
        c = a * 1.0
        c[0] = b[0]
        return c

    g = _graph(kernel, A, B)
    assert [o.name for o in g.outputs] == ["output0"] and not g.aliases
    assert [p.name for p in g.params] == ["a", "b"]


def test_later_reads_see_the_written_value():
    def kernel(a):
        a[1] = 0.0
        return a.sum(axis=0)

    g = _graph(kernel, A)
    out = evaluate(g, [A.copy()])
    want = A.copy()
    want[1] = 0.0
    np.testing.assert_allclose(out[[o.name for o in g.outputs].index("output0")], want.sum(0))
