"""What each tracing backend reports and how backend-dependent helpers behave: `get_backend()` inside and outside a
trace, `knob()` per backend, the parameter / result naming of the nkigen route, dtype narrowing of its inputs, and its
in-place update forms.  Cases follow the reference's tests/unit/test_nkigen_backend.py."""
import warnings

import numpy as np
import pytest

from nkipy_b200 import knob
from nkipy_b200.core.backend import get_backend, tracing
from nkipy_b200.core.backend.hlo import HLOModule, HLOTraceContext
from nkipy_b200.core.backend.nkigen import NkiGenIR, NkiGenTraceContext, get_nkigen_context
from nkipy_b200.core.interp import evaluate
from nkipy_b200.core.trace import NKIPyKernel

R = np.random.default_rng(17)
A = R.standard_normal((8, 16)).astype(np.float32)
B = R.standard_normal((8, 16)).astype(np.float32)


def test_knob_is_a_pass_through_outside_a_trace():
    assert knob(A, mem_space="Sbuf") is A
    assert knob(A) is A
    assert knob(A, mem_space="no such space") is A                  # nothing is validated in direct mode


def test_knob_warns_under_the_hlo_backend_and_returns_its_argument():
    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        with tracing(HLOTraceContext(HLOModule(name="t"))):
            assert knob(A, mem_space="Sbuf") is A
    assert len(w) == 1 and "only effective with backend='nkigen'" in str(w[0].message)


def test_knob_is_recorded_on_the_producing_node_under_nkigen():
    def k(a, b):
        c = a + b
        knob(c, mem_space="SharedHbm", tile_size=[8, 8])
        d = c * 2.0
        knob(d, partition_dim=1, reduction_tile=[4])
        return d

    with warnings.catch_warnings():
        warnings.simplefilter("error")                               # no warning on this backend
        g = NKIPyKernel(k, "nkigen").specialize(A, B)
    hints = {n.opcode: n.attrs["_knob"] for n in g.nodes if "_knob" in n.attrs}
    assert hints["add"] == {"mem_space": "Global", "tile_size": [8, 8]}
    assert hints["mul"] == {"partition_dim": 1, "reduction_tile": [4]}
    np.testing.assert_allclose(evaluate(g, [A, B])[0], (A + B) * 2, rtol=1e-6)


def test_knob_rejects_an_unknown_memory_space_while_tracing():
    with pytest.raises(ValueError, match="unknown mem_space"):
        NKIPyKernel(lambda a: knob(a * 1.0, mem_space="Nowhere"), "nkigen").specialize(A)


def test_active_backend_names():
    seen = {}

    def k(a):
        seen["name"] = get_backend()
        return a + 1.0

    assert get_backend() == "cpu"
    for backend in ("hlo", "nkigen"):
        NKIPyKernel(k, backend).specialize(A)
        assert seen["name"] == backend and get_backend() == "cpu"
    k(A)
    assert seen["name"] == "cpu"


def test_trace_context_objects():
    ctx = NkiGenTraceContext()
    assert ctx.backend_name == "nkigen" and ctx.honours_knobs and ctx.knobs == {}
    with pytest.raises(RuntimeError):
        get_nkigen_context()
    with tracing(ctx):
        assert get_backend() == "nkigen" and get_nkigen_context() is ctx
    assert get_backend() == "cpu"
    with tracing(HLOTraceContext()):
        assert get_backend() == "hlo"
        with pytest.raises(RuntimeError):
            get_nkigen_context()


def test_contexts_nest_and_unwind_on_errors():
    outer, inner = HLOTraceContext(), NkiGenTraceContext()
    with tracing(outer):
        with pytest.raises(KeyError):
            with tracing(inner):
                assert get_backend() == "nkigen"
                raise KeyError("x")
        assert get_backend() == "hlo"
    assert get_backend() == "cpu"


def test_nkigen_route_names_parameters_and_results():
    g = NKIPyKernel(lambda a, b: (a + b, a - b), "nkigen").specialize(A, B)
    assert [p.name for p in g.params] == ["in_tensor_0", "in_tensor_1"]
    text = g.to_text()
    assert "in_tensor_0" in text and "in_tensor_1" in text
    o0, o1 = evaluate(g, [A, B])
    np.testing.assert_allclose(o0, A + B)
    np.testing.assert_allclose(o1, A - B)
    view = NkiGenIR(g)
    assert len(view.inputs) == 2 and len(view.outputs) == 2 and view.content_hash("") == g.content_hash("")
    assert view.content_hash("-O1") != view.content_hash("")


def test_wide_inputs_are_narrowed():
    with warnings.catch_warnings(record=True):
        warnings.simplefilter("always")
        g = NKIPyKernel(lambda a, i: a[i], "nkigen").specialize(R.standard_normal((8, 4)), np.array([1, 3]))
    assert [np.dtype(p.dtype) for p in g.params] == [np.dtype(np.float32), np.dtype(np.int32)]


# ------------------------------------------------------------------ in-place updates of parameters on the nkigen route
def _run(fn, *arrays):
    g = NKIPyKernel(fn, "nkigen").specialize(*[a.copy() for a in arrays])
    return g, evaluate(g, [a.copy() for a in arrays])


def test_a_slice_update_of_a_parameter_returns_it_as_an_alias():
    def k(cache, new):
        cache[2:4] = new
        return cache

    new = R.standard_normal((2, 16)).astype(np.float32)
    g, (out,) = _run(k, A, new)
    want = A.copy(); want[2:4] = new
    np.testing.assert_array_equal(out, want)
    assert len(g.aliases) == 1 and g.aliases[0].param_index == 0 and g.aliases[0].output_index == 0


def test_several_slice_updates_of_one_parameter_are_one_alias():
    def k(cache, x, y):
        cache[0:1] = x
        cache[5:6] = y
        return cache

    x, y = A[:1] * 2, A[1:2] * 3
    g, (out,) = _run(k, A, x, y)
    want = A.copy(); want[0:1] = x; want[5:6] = y
    np.testing.assert_array_equal(out, want)
    assert len(g.aliases) == 1


def test_two_parameters_updated_and_returned():
    def k(kc, vc, kn, vn):
        kc[3:4] = kn
        vc[3:4] = vn
        return kc, vc

    kn, vn = B[:1], B[1:2]
    g, (o0, o1) = _run(k, A, A * 2, kn, vn)
    assert sorted((a.param_index, a.output_index) for a in g.aliases) == [(0, 0), (1, 1)]
    np.testing.assert_array_equal(o0[3], kn[0]); np.testing.assert_array_equal(o1[3], vn[0])


def test_an_update_without_a_return_still_reaches_the_caller():
    def k(cache, new):
        cache[0:2] = new

    new = B[:2]
    g, outs = _run(k, A, new)
    assert len(outs) == 1 and set(g.auto_aliased_indices) == {0}
    np.testing.assert_array_equal(outs[0][:2], new); np.testing.assert_array_equal(outs[0][2:], A[2:])


def test_an_updated_parameter_next_to_a_computed_result():
    def k(cache, new):
        cache[0:2] = new
        return np.sum(cache, axis=0)

    new = B[:2]
    g, outs = _run(k, A, new)
    want = A.copy(); want[:2] = new
    np.testing.assert_allclose(outs[0], want.sum(0), rtol=1e-5)
    assert len(outs) == 2 and set(g.auto_aliased_indices) == {1}
    np.testing.assert_array_equal(outs[1], want)


def test_an_update_computed_from_the_old_contents():
    def k(cache, new):
        cache[4:6] = cache[4:6] * 0.5 + new
        return cache

    new = B[:2]
    _, (out,) = _run(k, A, new)
    want = A.copy(); want[4:6] = want[4:6] * 0.5 + new
    np.testing.assert_allclose(out, want, rtol=1e-6)
