"""The raw surface of the C++ device runtime (`_spike.Spike`, tensors, loaded modules, trace session) used
directly, without the Python convenience layer: the counterpart of the reference's
tests/unit/test_spike_cpp_api.py.  The kernels are an add and a multiply compiled on the spot."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
N = 1024


def _run_child(code: str):
    res = subprocess.run([sys.executable, "-W", "ignore", "-c", f"import sys; sys.path.insert(0, {ROOT!r})\n" + code],
                         capture_output=True, text=True, timeout=180)
    assert res.returncode == 0, f"child exited with {res.returncode}\n{res.stdout}\n{res.stderr}"
    return res.stdout


@pytest.fixture(scope="module")
def rt():
    from nkipy_b200.spike import get_spike_singleton

    return get_spike_singleton()


def _compile(fn, tmp, name):
    from nkipy_b200.core.compile import compile_to_neff, trace

    k = trace(fn)
    k.specialize(np.zeros(N, np.float32), np.zeros(N, np.float32))
    return compile_to_neff(k, str(tmp / name), f"{name}.cubin")


@pytest.fixture(scope="module")
def add_cubin(tmp_path_factory):
    return _compile(lambda x, y: x + y, tmp_path_factory.mktemp("add"), "add")


@pytest.fixture(scope="module")
def mul_cubin(tmp_path_factory):
    return _compile(lambda x, y: x * y, tmp_path_factory.mktemp("mul"), "mul")


def _f32(rt, t):
    return np.frombuffer(rt.tensor_read(t, 0, t.size), dtype=np.float32)


def test_tensor_and_runtime_may_be_dropped_in_either_order():
    _run_child("""
from nkipy_b200.spike.spike_singleton import _native
S = _native()
s = S.Spike()
t = s.allocate_tensor(100)
del s            # the runtime goes first; the tensor's destructor must still be harmless
del t
s = S.Spike()
t = s.allocate_tensor(100)
del t
assert s.close() == 0
""")


def test_interpreter_shutdown_with_live_tensors():
    _run_child("""
from nkipy_b200.spike import get_spike_singleton
rt = get_spike_singleton()
tensors = [rt.allocate_tensor(4) for _ in range(128)]
""")


def test_open_close_reopen_and_static_queries():
    out = _run_child("""
from nkipy_b200.spike.spike_singleton import _native
S = _native()
assert S.Spike.get_visible_neuron_core_count() > 0
s = S.Spike()
assert not s.is_closed and s.sm_count > 0 and s.total_memory > 0
assert s.close() == 0 and s.is_closed
assert s.close() == 0                       # closing twice is not an error
try:
    s.allocate_tensor(16)
    raise SystemExit("allocation on a closed runtime")
except S.SpikeError:
    pass
s2 = S.Spike()                              # a new runtime after the first one closed
assert s2.close() == 0
print("REOPEN_OK")
""")
    assert "REOPEN_OK" in out


def test_tensor_operations(rt):
    t = rt.allocate_tensor(size=16, name="t")
    assert t.size == 16 and t.name == "t" and not t.is_freed and t.va != 0
    rt.tensor_write(t, np.arange(4, dtype=np.float32).tobytes(), 0)
    assert len(rt.tensor_read(t, 0, 16)) == 16
    assert _f32(rt, t).tolist() == [0, 1, 2, 3]
    rt.tensor_write(t, np.array([9.0], np.float32), 8)                # any buffer object, at a byte offset
    assert _f32(rt, t).tolist() == [0, 1, 9, 3]
    dest = np.zeros(2, np.float32)
    rt.tensor_read_to_buffer(t, dest, 8)
    assert dest.tolist() == [9, 3]
    s = rt.slice_from_tensor(t, 4, 8, "part")
    assert s.size == 8 and s.name == "part" and s.va == t.va + 4
    assert _f32(rt, s).tolist() == [1, 9]
    rt.tensor_write(s, np.array([5.0], np.float32), 0)                # a slice aliases its source
    assert _f32(rt, t).tolist() == [0, 5, 9, 3]
    from nkipy_b200.spike.spike_singleton import _native

    err = _native().SpikeError
    with pytest.raises(err):
        rt.tensor_read(t, 8, 16)                                      # past the end
    with pytest.raises(err):
        rt.slice_from_tensor(t, 12, 8, "bad")
    rt.free_tensor(s)
    assert s.is_freed and not t.is_freed
    rt.free_tensor(t)
    assert t.is_freed
    with pytest.raises(err):
        rt.tensor_read(t, 0, 4)


def _xyz(rt, *values):
    out = []
    for i, v in enumerate(values):
        t = rt.allocate_tensor(size=4 * N, name=f"t{i}")
        rt.tensor_write(t, np.full(N, v, np.float32), 0)
        out.append(t)
    return out


def test_model_load_execute_unload(rt, add_cubin):
    model = rt.load_model(add_cubin)
    assert model.neff_path == add_cubin and not model.unloaded and model.num_launches >= 1
    assert not model.is_collective and model.world_size == 1
    x, y, out = _xyz(rt, 1.0, 1.0, 0.0)
    assert rt.execute(model, {"x": x, "y": y}, {"output0": out}) is None
    assert np.all(_f32(rt, out) == 2.0)
    from nkipy_b200.spike.spike_singleton import _native

    err = _native().SpikeError
    with pytest.raises(err):
        rt.execute(model, {"x": x}, {"output0": out})                 # a missing input is named, not read
    small = rt.allocate_tensor(size=4, name="small")
    with pytest.raises(err):
        rt.execute(model, {"x": x, "y": small}, {"output0": out})     # wrong size
    rt.unload_model(model)
    assert model.unloaded
    with pytest.raises(err):
        rt.execute(model, {"x": x, "y": y}, {"output0": out})
    for t in (x, y, out, small):
        rt.free_tensor(t)


def test_trace_session_sees_the_launches(rt, add_cubin):
    from nkipy_b200.spike.spike_singleton import _native

    model = rt.load_model(add_cubin)
    x, y, out = _xyz(rt, 1.0, 2.0, 0.0)
    with _native().SystemTraceSession(model.core_id) as sess:
        assert sess.active
        rt.execute(model, {"x": x, "y": y}, {"output0": out})
        events = json.loads(sess.fetch_events_json())["events"]
    assert not sess.active
    runs = [e for e in events if e["event_type"] == "kernel_exec"]
    assert {e["phase"] for e in runs} == {"start", "stop"} and len(runs) == 2 * model.num_launches
    by_id = {}
    for e in runs:
        by_id.setdefault(e["tracking_id"], {})[e["phase"]] = e["device_timestamp_ns"]
    assert all(v["stop"] >= v["start"] for v in by_id.values())
    assert all(e["core_id"] == model.core_id and e["model"] == model.name for e in runs)
    rt.unload_model(model)
    for t in (x, y, out):
        rt.free_tensor(t)


def test_two_models_chained_through_a_device_tensor(rt, add_cubin, mul_cubin):
    add, mul = rt.load_model(add_cubin), rt.load_model(mul_cubin)
    x, y, z, s, p = _xyz(rt, 2.0, 3.0, 4.0, 0.0, 0.0)
    rt.execute(add, {"x": x, "y": y}, {"output0": s})
    rt.execute(mul, {"x": s, "y": z}, {"output0": p})                  # (2 + 3) * 4
    assert np.all(_f32(rt, p) == 20.0)
    rt.unload_model(add)
    rt.unload_model(mul)
    for t in (x, y, z, s, p):
        rt.free_tensor(t)


def test_get_tensor_info(rt, add_cubin):
    model = rt.load_model(add_cubin)
    info = rt.get_tensor_info(model)
    assert set(info.inputs) == {"x", "y"} and set(info.outputs) == {"output0"}
    assert list(info.input_order) == ["x", "y"] and list(info.output_order) == ["output0"]
    for meta in list(info.inputs.values()) + list(info.outputs.values()):
        assert meta.size == 4 * N and meta.dtype in ("f32", "float32") and list(meta.shape) == [N]
        assert "TensorMetadata(" in repr(meta)
    rt.unload_model(model)
