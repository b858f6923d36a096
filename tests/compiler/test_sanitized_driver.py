"""The native compiler under AddressSanitizer + UndefinedBehaviorSanitizer: the command-line driver is built with
both (any finding aborts the process) and runs the whole pipeline, single passes, the stop-after forms and its error
paths over a corpus of traced kernels.  Its output must equal the regular build's byte for byte."""
import shutil
import subprocess

import numpy as np
import pytest

from nkipy_b200 import nkigen
from nkipy_b200.compiler import native
from nkipy_b200.nkigen import transforms as T

pytestmark = pytest.mark.skipif(shutil.which("g++") is None, reason="no host compiler")


@pytest.fixture(scope="module")
def san():
    try:
        return native.build_sanitized()
    except RuntimeError as e:                                   # a toolchain without the sanitizer runtimes
        if "sanitize" in str(e) or "asan" in str(e):
            pytest.skip("sanitizer runtime not installed")
        raise


def _loop(x, w):
    return nkigen.fori_loop(0, 4, lambda i, h: np.tanh(h @ w + x[i]), np.zeros(16, np.float32))


def _attention(q, k, v):
    s = np.matmul(q, np.transpose(k, (0, 2, 1))) * np.float32(0.25)
    e = np.exp(s - np.max(s, axis=-1, keepdims=True))
    return np.matmul(e / np.sum(e, axis=-1, keepdims=True), v)


def _knobbed(a, b):
    y = a @ b.T
    nkigen.knob(y).tile_op(tile_size=[128, 64])
    z = np.maximum(y, 0.0)
    nkigen.knob.fuse(y, z)
    return z


def _views(a, v):
    s = a[1:7:2, 2:14][0:2, 1:9:3]
    b = np.broadcast_to(np.broadcast_to(v, (4, 16)).reshape(4, 1, 16), (4, 3, 16))
    c = np.concatenate([np.concatenate([a, a], axis=0), a], axis=0)
    t = np.transpose(np.transpose(a.reshape(8, 1, 16), (1, 0, 2)), (0, 2, 1))
    return s, b, c, t, np.sum(a.reshape(8, 1, 16), axis=1) / 4.0, (-(-a)).astype(np.float16).astype(np.float32)


def _update(cache, new):
    cache[2:4] = new * 1.0 + 0.0
    return np.sum(cache, axis=0)


CORPUS = {
    "loop": (_loop, [((4, 16), "f32"), ((16, 16), "f32")]),
    "attention": (_attention, [((2, 8, 16), "f32")] * 3),
    "knobbed": (_knobbed, [((256, 128), "bf16"), ((192, 128), "bf16")]),
    "views": (_views, [((8, 16), "f32"), ((16,), "f32")]),
    "update": (_update, [((8, 16), "f32"), ((2, 16), "f32")]),
    "gather": (lambda t, i: np.take(t, i, axis=0) * 2.0, [((32, 8), "f32"), ((4,), "i32")]),
    "big_constant": (lambda x: x + np.full((64, 64), 3.0, np.float32) + np.arange(64, dtype=np.float32), [((64, 64), "f32")]),
}


def _run(exe, text, *args):
    return subprocess.run([str(exe), *args, "-"], input=text, capture_output=True, text=True, timeout=120)


@pytest.mark.parametrize("name", sorted(CORPUS))
def test_pipeline_is_clean_and_matches_the_regular_build(san, name):
    fn, specs = CORPUS[name]
    text = nkigen.trace(fn, input_specs=specs).to_ir()
    res = _run(san, text, "--pipeline")
    assert res.returncode == 0, res.stderr[-3000:]
    assert "Sanitizer" not in res.stderr and "runtime error" not in res.stderr, res.stderr[-3000:]
    assert res.stdout == T.apply_complete_knob_pipeline(text)


@pytest.mark.parametrize("name", ["views", "knobbed", "loop"])
def test_every_pass_alone_and_every_stop_point(san, name):
    fn, specs = CORPUS[name]
    text = nkigen.trace(fn, input_specs=specs).to_ir()
    native_passes = [p for p in T.pass_list() if not p.startswith("py:")]
    for p in native_passes:
        res = _run(san, text, "--pass", p)
        assert res.returncode == 0 and "runtime error" not in res.stderr, (p, res.stderr[-2000:])
    for stop in ("1", str(len(native_passes)), "cse", "canonicalize", "layout", "memory", "canonicalize:1"):
        res = _run(san, text, "--pipeline", "--stop-after", stop)
        assert res.returncode == 0 and "runtime error" not in res.stderr, (stop, res.stderr[-2000:])


def test_small_shared_memory_budget_and_fast_math(san):
    fn, specs = CORPUS["knobbed"]
    text = nkigen.trace(fn, input_specs=specs).to_ir()
    for extra in (["--smem-capacity", "49152"], ["--fast-math"], ["--sm-count", "4", "--tmem-columns", "128"]):
        res = _run(san, text, "--pipeline", *extra)
        assert res.returncode == 0 and "runtime error" not in res.stderr, (extra, res.stderr[-2000:])


@pytest.mark.parametrize("text", ["", "graph @k {", "graph @k {\n  %0 = param() {\"name\": \"x\"} : f32[4]\n  %1 = nosuch(%0) {} : f32[4]\n  return %1 {\"name\": \"o\"}\n}\n",
                                  "graph @k {\n  %0 = param() {\"name\": \"x\"} : f32[4]\n  %1 = add(%0, %7) {} : f32[4]\n  return %1 {\"name\": \"o\"}\n}\n",
                                  "graph @k {\n  %0 = param() {\"name\": \"x\"} : f32[4\n}\n", "\x00\x01garbage"],
                         ids=["empty", "truncated", "unknown_opcode", "undefined_value", "bad_type", "binary"])
def test_malformed_input_is_an_error_message_not_a_crash(san, text):
    res = _run(san, text, "--pipeline")
    assert res.returncode in (0, 1), res.stderr[-2000:]          # a clean exit either way; a sanitizer abort is neither
    assert "Sanitizer" not in res.stderr and "runtime error" not in res.stderr, res.stderr[-3000:]
    if res.returncode == 1:
        assert "nkipy-b200-opt: error:" in res.stderr


def test_bad_options_are_reported(san):
    fn, specs = CORPUS["gather"]
    text = nkigen.trace(fn, input_specs=specs).to_ir()
    for args in (["--pass", "no-such-pass"], ["--stop-after", "no-such-pass", "--pipeline"], ["--no-such-option"],
                 ["--pass"], ["--smem-capacity", "many"]):
        res = _run(san, text, *args) if args != ["--pass"] else subprocess.run([str(san), "--pass"], input=text,
                                                                                capture_output=True, text=True)
        assert res.returncode == 1 and "Sanitizer" not in res.stderr, (args, res.stderr[-1500:])


def test_the_numerical_suite_kernels_are_clean_too(san):
    import test_nkigen_numerical as N

    for name in sorted(N.KERNELS):
        fn, inputs = N.KERNELS[name]
        text = nkigen.trace(fn, input_specs=N._specs(inputs)).to_ir()
        res = _run(san, text, "--pipeline")
        assert res.returncode == 0 and "Sanitizer" not in res.stderr and "runtime error" not in res.stderr, \
            (name, res.stderr[-3000:])


def test_the_spec_kernels_are_clean_and_keep_their_results(san):
    """Every specification kernel under tests/kernels, traced on its default inputs, goes through the sanitized
    pipeline; the lowered graph still evaluates to what direct mode gives."""
    import copy
    import glob
    import importlib
    import os

    from utils import trace_kernel

    from nkipy_b200.core.interp import evaluate
    from nkipy_b200.core.ir import Graph

    here = os.path.dirname(os.path.abspath(__file__))
    n = 0
    for path in sorted(glob.glob(os.path.join(here, "..", "kernels", "*.py"))):
        stem = os.path.splitext(os.path.basename(path))[0]
        if stem == "__init__":
            continue
        specs = getattr(importlib.import_module(f"kernels.{stem}"), "kernel_specs", None) or []
        for spec in specs if isinstance(specs, list) else [specs]:
            if not spec.is_pure_numpy:
                continue
            inputs = spec.default_inputs(np.random.default_rng(0))
            g = trace_kernel(spec.function, *copy.deepcopy(inputs))
            res = _run(san, g.to_text(), "--pipeline")
            assert res.returncode == 0 and "Sanitizer" not in res.stderr and "runtime error" not in res.stderr, \
                (stem, spec.function.__name__, res.stderr[-3000:])
            arrays = [np.asarray(a) for a in inputs if isinstance(a, np.ndarray)]
            got = evaluate(Graph.from_text(res.stdout), [a.astype(p.dtype) for a, p in zip(arrays, g.params)])
            want = spec.function(*copy.deepcopy(inputs))
            want = list(want) if isinstance(want, (tuple, list)) else [want]
            for o, e in zip(got, want):
                np.testing.assert_allclose(np.asarray(o, np.float64), np.asarray(e, np.float64), rtol=2e-3, atol=2e-3)
            n += 1
    assert n >= 12
