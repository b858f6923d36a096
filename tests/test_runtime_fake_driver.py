"""The C++ device runtime on a machine without a GPU: `tests/fake_cuda/fake_libcuda.cpp` (device memory = host memory,
launches and copies written to a log, error codes injected by name) is built as libcuda.so.1 and put first on the
library path of a child process that drives the runtime through its Python bindings.

Covers what the reference checks through its bindings in tests/unit/test_spike_cpp_api.py (tensor life cycle, slices,
bounds, use after free, models and executes, error types with preserved driver codes, close) plus the launch list a
loaded module issues and host-side failure injection: the failing driver call is a fake that returns an error code."""
import json
import os
import shutil
import subprocess
import sys
import textwrap

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.skipif(shutil.which("g++") is None, reason="no host compiler")


@pytest.fixture(scope="module")
def fake_lib(tmp_path_factory):
    d = tmp_path_factory.mktemp("fake_cuda")
    cuda_inc = os.environ.get("CUDA_HOME", "/usr/local/cuda") + "/include"
    if not os.path.exists(os.path.join(cuda_inc, "cuda.h")):
        pytest.skip("CUDA headers not installed")
    cmd = ["g++", "-O1", "-g", "-std=c++17", "-shared", "-fPIC", "-Wall", f"-I{cuda_inc}",
           os.path.join(ROOT, "tests", "fake_cuda", "fake_libcuda.cpp"), "-o", str(d / "libcuda.so.1")]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    return d


@pytest.fixture(scope="module")
def compiled(tmp_path_factory):
    """A real compiled module (cubin + plan) of a small kernel: the fake driver ignores the code, the runtime reads the plan."""
    if shutil.which("nvcc") is None and not os.path.exists("/usr/local/cuda/bin/nvcc"):
        pytest.skip("nvcc not installed")
    from nkipy_b200.core.compile import compile_to_neff, trace

    def kernel(a, b):
        return np.tanh(a @ b) + 1.0, np.sum(a, axis=0)

    out = tmp_path_factory.mktemp("module")
    k = trace(kernel)
    k.specialize(np.zeros((8, 16), np.float32), np.zeros((16, 4), np.float32))
    path = compile_to_neff(k, str(out), "k.cubin")
    plan = json.loads(open(os.path.splitext(path)[0] + ".json").read())
    return path, plan


@pytest.fixture(scope="module")
def sanitized_module(tmp_path_factory):
    from nkipy_b200.runtime import native

    preload = native.sanitizer_preload()
    if not preload or not all(os.path.exists(p) for p in preload.split()):
        pytest.skip("no shared AddressSanitizer runtime")
    return native.build_sanitized(), preload


@pytest.fixture(params=["plain", "sanitized"])
def fake_dir(request, fake_lib):
    """The directory of the fake driver; in the `sanitized` variant the child process also loads the runtime module
    built with AddressSanitizer + UndefinedBehaviorSanitizer (any finding aborts the child, which fails the test)."""
    if request.param == "plain":
        return FakeEnv(fake_lib, None, None)
    so, preload = request.getfixturevalue("sanitized_module")
    return FakeEnv(fake_lib, so, preload)


class FakeEnv:
    def __init__(self, lib_dir, san_module, preload):
        self.lib_dir, self.san_module, self.preload = lib_dir, san_module, preload


_SAN_PREAMBLE = """
import importlib.util
_spec = importlib.util.spec_from_file_location("nkipy_b200.spike._spike", %r)
_mod = importlib.util.module_from_spec(_spec); _spec.loader.exec_module(_mod)
sys.modules["nkipy_b200.spike._spike"] = _mod
import os as _os
_os.environ.pop("LD_PRELOAD", None)          # it has done its work here; compilers started from this process must not inherit it
"""


def run_child(fake, body, env=None, log=None):
    code = "import sys\nsys.path.insert(0, %r)\nimport numpy as np\n" % ROOT
    e = dict(os.environ)
    if fake.san_module is not None:
        code += _SAN_PREAMBLE % str(fake.san_module)
        e["LD_PRELOAD"] = fake.preload
        e["ASAN_OPTIONS"] = "detect_leaks=0:abort_on_error=0:exitcode=99"      # the interpreter's own leaks are not ours
    code += textwrap.dedent(body)
    fake_dir = fake.lib_dir
    e["LD_LIBRARY_PATH"] = str(fake_dir) + os.pathsep + e.get("LD_LIBRARY_PATH", "")
    e.pop("CUDA_VISIBLE_DEVICES", None)
    if log is not None:
        e["FAKE_CUDA_LOG"] = str(log)
    e.update(env or {})
    res = subprocess.run([sys.executable, "-W", "ignore", "-c", code], capture_output=True, text=True, timeout=300, env=e)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    return res.stdout


def test_device_discovery_and_properties(fake_dir):
    out = run_child(fake_dir, """
        from nkipy_b200 import spike
        from nkipy_b200.spike import get_spike_singleton
        assert "torch" not in sys.modules
        print(spike.visible_device_count())
        rt = get_spike_singleton()
        print(rt.device_name, rt.sm_count, rt.total_memory >> 30, rt.device_ordinal, rt.is_closed)
    """, env={"FAKE_CUDA_DEVICES": "4"})
    assert out.split() == ["4", "Fake", "B200", "#0", "148", "180", "0", "False"]


def test_no_devices_is_reported_not_raised(fake_dir):
    out = run_child(fake_dir, """
        from nkipy_b200 import spike
        print(spike.visible_device_count())
        try:
            spike.get_spike_singleton()
        except spike.SpikeError as e:
            print("error:", e)
    """, env={"FAKE_CUDA_DEVICES": "0"})
    assert out.startswith("0\n") and "out of range" in out


def test_tensor_life_cycle(fake_dir, tmp_path):
    log = tmp_path / "log.txt"
    run_child(fake_dir, """
        from nkipy_b200 import spike
        from nkipy_b200.spike import SpikeTensor, get_spike_singleton
        rt = get_spike_singleton()
        a = np.arange(64, dtype=np.float32).reshape(8, 8)
        t = SpikeTensor.from_numpy(a, "whole")
        assert t.tensor_ref.size == 256 and t.tensor_ref.name == "whole" and t.va != 0 and not t.tensor_ref.is_freed
        np.testing.assert_array_equal(t.numpy(), a)
        # a byte-range view shares the allocation
        rows = t.slice_bytes(2 * 32, (2, 8), name="rows")
        np.testing.assert_array_equal(rows.numpy(), a[2:4])
        rows.write_from_numpy(np.zeros((2, 8), np.float32))
        want = a.copy(); want[2:4] = 0
        np.testing.assert_array_equal(t.numpy(), want)
        assert rows.va == t.va + 64
        # bounds
        for bad in (lambda: t.slice_bytes(250, (4,), np.float32), lambda: rt.tensor_write(t.tensor_ref, np.zeros(8, np.uint8), 252),
                    lambda: rt.tensor_read_to_buffer(t.tensor_ref, np.zeros(300, np.uint8), 0)):
            try:
                bad()
            except spike.SpikeError as e:
                assert "exceeds" in str(e)
            else:
                raise AssertionError("no error")
        # free: the view dies with its parent, later use is an error, a second free is not
        t.free()
        assert t.tensor_ref.is_freed and rows.tensor_ref.is_freed
        for bad in (t.numpy, rows.numpy, lambda: t.slice_bytes(0, (1,), np.float32)):
            try:
                bad()
            except spike.SpikeError as e:
                assert "freed" in str(e)
            else:
                raise AssertionError("no error")
        t.free()
        # zero-size tensors
        z = SpikeTensor.from_numpy(np.zeros((0, 4), np.float32))
        assert z.numpy().shape == (0, 4)
    """, log=log)
    text = log.read_text()
    assert "bad_free" not in text and "out_of_bounds" not in text          # the runtime's own checks came first


def test_module_load_execute_and_launch_list(fake_dir, compiled, tmp_path):
    path, plan = compiled
    log = tmp_path / "log.txt"
    out = run_child(fake_dir, f"""
        from nkipy_b200 import spike
        from nkipy_b200.spike import SpikeModel, SpikeTensor, get_spike_singleton
        m = SpikeModel.load_from_neff({path!r}, name="k")
        ref = m.model_ref
        print(ref.num_launches, ref.is_collective, ref.rank_id, ref.world_size, ref.unloaded)
        print(sorted((n, tuple(t.shape), t.dtype) for n, t in m.input_info.items()), m.input_order)
        print(sorted((n, tuple(t.shape), t.dtype) for n, t in m.output_info.items()), m.output_order)
        a = SpikeTensor.from_numpy(np.ones((8, 16), np.float32), "a")
        b = SpikeTensor.from_numpy(np.ones((16, 4), np.float32), "b")
        outs = m({{"a": a, "b": b}})
        print(sorted((k, v.shape) for k, v in outs.items()))
        # missing, extra and wrongly sized tensors are rejected before anything is launched
        for bad in ({{"a": a}}, {{"a": a, "b": b, "c": b}}, {{"a": b, "b": a}}):
            try:
                m(bad)
            except (ValueError, spike.SpikeError) as e:
                print("rejected")
        a.free()
        try:
            m({{"a": a, "b": b}})
        except (ValueError, spike.SpikeError) as e:
            print("freed input rejected")
        m.unload()
        print(ref.unloaded)
    """, log=log)
    lines = out.strip().splitlines()
    assert lines[0] == f"{len(plan['launches'])} False 0 1 False"
    assert "('a', (8, 16), 'f32')" in lines[1] and "('b', (16, 4), 'f32')" in lines[1]
    assert "(8, 4)" in lines[3] and "(16,)" in lines[3]
    assert lines.count("rejected") == 3 and "freed input rejected" in lines and lines[-1] == "True"
    launches = [ln for ln in log.read_text().splitlines() if ln.startswith("launch ")]
    assert len(launches) == len(plan["launches"])                            # one execute went through; the rejected ones launched nothing
    for ln, want in zip(launches, plan["launches"]):
        assert ln.split()[1] == want["kernel"]
        assert f"grid={','.join(map(str, want['grid']))}" in ln and f"block={','.join(map(str, want['block']))}" in ln
    assert "module_load id=1" in log.read_text() and "module_unload id=1" in log.read_text()


def test_benchmark_uses_device_events(fake_dir, compiled):
    path, plan = compiled
    out = run_child(fake_dir, f"""
        from nkipy_b200.spike import SpikeModel, SpikeTensor
        m = SpikeModel.load_from_neff({path!r}, name="k")
        a = SpikeTensor.from_numpy(np.ones((8, 16), np.float32), "a")
        b = SpikeTensor.from_numpy(np.ones((16, 4), np.float32), "b")
        r = m.benchmark({{"a": a, "b": b}}, warmup_iterations=2, benchmark_iterations=5, mode="device")
        print(r.iterations, r.warmup_iterations, round(r.mean_ms, 3), round(r.min_ms, 3), round(r.max_ms, 3))
    """, env={"FAKE_CUDA_EVENT_MS": "0.5"})
    per_execute = f"{0.5 * len(plan['launches']):.1f}"            # one event pair per launch, 0.5 ms each from the fake
    assert out.split() == ["5", "2", per_execute, per_execute, per_execute]


@pytest.mark.parametrize("call,code,name", [("cuLaunchKernel", 719, "CUDA_ERROR_LAUNCH_FAILED"),
                                            ("cuLaunchKernel", 702, "CUDA_ERROR_LAUNCH_TIMEOUT"),
                                            ("cuStreamSynchronize", 700, "CUDA_ERROR_ILLEGAL_ADDRESS"),
                                            ("cuModuleLoadData", 2, "CUDA_ERROR_OUT_OF_MEMORY")])
def test_a_failing_driver_call_surfaces_with_its_code_and_leaves_the_runtime_usable(fake_dir, compiled, call, code, name):
    path, _ = compiled
    out = run_child(fake_dir, f"""
        import os
        from nkipy_b200 import spike
        from nkipy_b200.spike import SpikeModel, SpikeTensor
        a = SpikeTensor.from_numpy(np.ones((8, 16), np.float32), "a")
        b = SpikeTensor.from_numpy(np.ones((16, 4), np.float32), "b")
        os.environ["FAKE_CUDA_FAIL"] = "{call}:{code}:1"            # the first call of that function fails
        try:
            m = SpikeModel.load_from_neff({path!r}, name="k")
            m({{"a": a, "b": b}})
            print("no error")
        except spike.NrtError as e:
            print("code", e.code, "|", e)
            assert isinstance(e, spike.SpikeRuntimeError)
        os.environ.pop("FAKE_CUDA_FAIL")
        m = SpikeModel.load_from_neff({path!r}, name="k2")                 # the runtime still works afterwards
        outs = m({{"a": a, "b": b}})
        print("recovered", len(outs))
    """)
    assert "no error" not in out
    assert f"code {code} |" in out and name in out and f"({code})" in out
    assert "recovered 2" in out


def test_allocation_failure_is_a_typed_error(fake_dir):
    out = run_child(fake_dir, """
        import os
        from nkipy_b200 import spike
        from nkipy_b200.spike import SpikeTensor, get_spike_singleton
        get_spike_singleton()
        os.environ["FAKE_CUDA_FAIL"] = "cuMemAlloc_v2:2"
        try:
            SpikeTensor.empty((1024,), np.float32)
        except spike.CudaError as e:
            print("oom:", e.code, e)
        os.environ.pop("FAKE_CUDA_FAIL")
        print(SpikeTensor.empty((1024,), np.float32).nbytes)
    """)
    assert "CUDA_ERROR_OUT_OF_MEMORY (2)" in out and out.strip().endswith("4096")


def test_close_and_reset(fake_dir, tmp_path):
    log = tmp_path / "log.txt"
    out = run_child(fake_dir, """
        import warnings
        from nkipy_b200 import spike
        from nkipy_b200.spike import SpikeTensor, get_spike_singleton
        rt = get_spike_singleton()
        t = SpikeTensor.from_numpy(np.ones(4, np.float32))
        try:
            spike.configure(visible_cores=[0])
        except RuntimeError as e:
            print("configure refused")
        with warnings.catch_warnings(record=True):
            warnings.simplefilter("always")
            spike.reset()
        print(rt.is_closed, t.tensor_ref.is_freed)
        try:
            t.numpy()
        except spike.SpikeError:
            print("stale tensor rejected")
        rt2 = get_spike_singleton()
        print(rt2 is not rt, rt2.is_closed)
        print(SpikeTensor.from_numpy(np.full(4, 3.0, np.float32)).numpy().sum())
    """, log=log)
    assert out.split("\n")[:5] == ["configure refused", "True True", "stale tensor rejected", "True False", "12.0"]
    assert log.read_text().count("ctx_release") == 2                         # once at reset, once at exit


def test_system_trace_session(fake_dir, compiled):
    path, _ = compiled
    out = run_child(fake_dir, f"""
        import json
        from nkipy_b200 import spike
        from nkipy_b200.spike import SpikeModel, SpikeTensor
        m = SpikeModel.load_from_neff({path!r}, name="k")
        a = SpikeTensor.from_numpy(np.ones((8, 16), np.float32), "a")
        b = SpikeTensor.from_numpy(np.ones((16, 4), np.float32), "b")
        with spike.SystemTraceSession() as s:
            for _ in range(3):
                m({{"a": a, "b": b}})
            ev = json.loads(s.fetch_events_json())["events"]
        kinds = [(e["event_type"], e["phase"]) for e in ev]
        print(kinds.count(("kernel_exec", "start")), kinds.count(("kernel_exec", "stop")))
        print(len(json.loads(s.fetch_events_json())["events"]))                # the ring was consumed
    """)
    assert out.split() == ["3", "3", "0"]


# ------------------------------------------------------------------ symmetric memory on the fake driver's VMM emulation
def test_symmetric_buffers_alias_across_ranks_and_release_everything(fake_dir, tmp_path):
    log = tmp_path / "log.txt"
    out = run_child(fake_dir, """
        import ctypes, os
        from nkipy_b200.spike.spike_singleton import _native
        S = _native()
        assert S.SymmetricBuffer.supported(0) and S.SymmetricBuffer.multicast_supported(1)
        bufs = [S.SymmetricBuffer(r, 1000) for r in range(3)]
        print(sorted({b.size for b in bufs}), [b.device_ordinal for b in bufs])
        fds = [b.export_fd() for b in bufs]
        for r, b in enumerate(bufs):
            for p, fd in enumerate(fds):
                if p != r:
                    b.import_peer(p, fd)
            b.zero()
        for fd in fds:
            os.close(fd)
        # what rank r writes through its mapping of rank p's memory, rank p reads in its own
        for r, b in enumerate(bufs):
            for p in range(3):
                if p != r:
                    ctypes.memmove(b.peer_ptr(p) + 64 * r, b"from%d" % r, 5)
        for p, b in enumerate(bufs):
            got = [ctypes.string_at(b.local_ptr + 64 * r, 5) for r in range(3) if r != p]
            assert got == [b"from%d" % r for r in range(3) if r != p], got
            assert b.peer_ptr(p) == 0 and len({b.peer_ptr(q) for q in range(3) if q != p} | {b.local_ptr}) == 3
        # multicast object: created by rank 0, imported by the others, every device added before anyone binds
        m = bufs[0].multicast_create(3)
        for b in bufs[1:]:
            b.multicast_import(m)
        os.close(m)
        for b in bufs:
            b.multicast_add_device()
        for b in bufs:
            b.multicast_bind()
        print([b.has_multicast for b in bufs], all(b.multicast_ptr for b in bufs))
        for b in bufs:
            b.close()
            b.close()                                   # idempotent
        print([b.closed for b in bufs])
    """, env={"FAKE_CUDA_DEVICES": "3"}, log=log)
    assert out.splitlines() == ["[2097152] [0, 1, 2]", "[True, True, True] True", "[True, True, True]"]
    text = log.read_text()
    assert text.count("mem_create") == 3 and text.count("multicast_bind") == 3 and text.count("multicast_unbind") == 3
    assert text.strip().splitlines()[-1] == "mem_release live_handles=0"
    for bad in ("bad_release", "bad_unmap", "bad_unbind", "bad_address_free", "address_free_while_mapped"):
        assert bad not in text


def test_symmetric_buffer_misuse_and_driver_failures(fake_dir, tmp_path):
    log = tmp_path / "log.txt"
    out = run_child(fake_dir, """
        import os
        from nkipy_b200 import spike
        from nkipy_b200.spike.spike_singleton import _native
        S = _native()
        a = S.SymmetricBuffer(0, 4096)
        def expect(fn, *types):
            try:
                fn()
            except types as e:
                return type(e).__name__
            return "no error"
        r, w = os.pipe()
        print(expect(lambda: a.import_peer(1, w), spike.SpikeRuntimeError))       # not an allocation handle
        os.close(r); os.close(w)
        print(expect(lambda: a.import_peer(0, a.export_fd()), spike.SpikeRuntimeError, ValueError))   # mapping one's own allocation a second time is allowed
        print(expect(lambda: S.SymmetricBuffer(7, 4096), spike.SpikeRuntimeError))  # no such device
        os.environ["FAKE_CUDA_FAIL"] = "cuMemMap:2"
        print(expect(lambda: S.SymmetricBuffer(1, 4096), spike.CudaError))
        os.environ["FAKE_CUDA_FAIL"] = "cuMemSetAccess:1"
        print(expect(lambda: S.SymmetricBuffer(1, 4096), spike.CudaError))
        os.environ.pop("FAKE_CUDA_FAIL")
        b = S.SymmetricBuffer(1, 4096)                                            # and afterwards it works
        a.close(); b.close()
        print(expect(lambda: a.export_fd(), spike.SpikeRuntimeError))             # closed
    """, env={"FAKE_CUDA_DEVICES": "2"}, log=log)
    lines = out.splitlines()
    assert lines == ["CudaError", "no error", "CudaError", "CudaError", "CudaError", "SpikeError"]
    text = log.read_text()
    # the constructors that failed half way gave back what they had taken
    assert "address_free_while_mapped" not in text and "bad_unmap" not in text and "bad_release" not in text
    assert text.strip().splitlines()[-1] == "mem_release live_handles=0"


def test_descriptors_cross_processes(fake_lib, tmp_path):
    """Two processes, one buffer each; the descriptors travel over a Unix socket pair with SCM_RIGHTS, and a write by
    one process through its mapping of the other's memory is read by the owner."""
    body = """
        import ctypes, os, socket, sys, time
        from nkipy_b200.spike.spike_singleton import _native
        S = _native()
        rank = int(sys.argv[1]); sock = socket.socket(fileno=int(sys.argv[2]))
        buf = S.SymmetricBuffer(rank, 8192); buf.zero()
        fd = buf.export_fd()
        socket.send_fds(sock, [b"fd"], [fd]); os.close(fd)
        _, fds, _, _ = socket.recv_fds(sock, 16, 1)
        buf.import_peer(1 - rank, fds[0]); os.close(fds[0])
        ctypes.memmove(buf.peer_ptr(1 - rank) + 128, b"written by rank %d" % rank, 17)
        sock.sendall(b"done"); assert sock.recv(4) == b"done"                  # both have written
        print(ctypes.string_at(buf.local_ptr + 128, 17).decode())
        sock.sendall(b"read"); assert sock.recv(4) == b"read"                  # both have read: safe to unmap
        buf.close()
    """
    import socket

    a, b = socket.socketpair(socket.AF_UNIX, socket.SOCK_STREAM)
    code = "import sys\nsys.path.insert(0, %r)\n" % ROOT + textwrap.dedent(body)
    env = dict(os.environ, LD_LIBRARY_PATH=str(fake_lib), FAKE_CUDA_DEVICES="2")
    env.pop("CUDA_VISIBLE_DEVICES", None)
    procs = [subprocess.Popen([sys.executable, "-W", "ignore", "-c", code, str(r), str(s.fileno())], env=env, pass_fds=[s.fileno()],
                              stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True) for r, s in ((0, a), (1, b))]
    outs = [p.communicate(timeout=120) for p in procs]
    a.close(); b.close()
    assert [p.returncode for p in procs] == [0, 0], outs
    assert outs[0][0].strip() == "written by rank 1" and outs[1][0].strip() == "written by rank 0"


# ------------------------------------------------------------------ modules with collectives
@pytest.fixture(scope="module")
def compiled_cc(tmp_path_factory):
    if shutil.which("nvcc") is None and not os.path.exists("/usr/local/cuda/bin/nvcc"):
        pytest.skip("nvcc not installed")
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from test_segmented_cc import _data, make_kernel

    from nkipy_b200.core.compile import compile_to_neff, trace

    paths = {}
    for world in (1, 2):
        x, w = _data(0)
        k = trace(make_kernel(world))
        k.specialize(x, w)
        out = tmp_path_factory.mktemp(f"cc{world}")
        paths[world] = compile_to_neff(k, str(out), "k.cubin")
    return paths


def test_collective_module_load_rules(fake_dir, compiled_cc, tmp_path):
    log = tmp_path / "log.txt"
    out = run_child(fake_dir, f"""
        from nkipy_b200 import spike
        from nkipy_b200.spike import get_spike_singleton, SpikeTensor
        rt = get_spike_singleton()
        def expect(fn):
            try:
                fn()
            except spike.SpikeRuntimeError as e:
                return str(e)
            return "no error"
        one, two = {compiled_cc[1]!r}, {compiled_cc[2]!r}
        # traced for one rank: the module brings its own workspace and runs alone
        m1 = rt.load_model(one, 0, False, 0, 1)
        print(m1.has_collectives, m1.collective_world, m1.workspace_bytes > 0)
        print(expect(lambda: m1.set_collective_workspace([1])))                   # already set at load
        # traced for two ranks: needs a collective load of the same world
        print(expect(lambda: rt.load_model(two, 0, False, 0, 1)))
        print(expect(lambda: rt.load_model(two, 0, True, 0, 4)))
        print(expect(lambda: rt.load_model(two, 0, True, 2, 2)))
        m2 = rt.load_model(two, 0, True, 1, 2)
        print(m2.is_collective, m2.rank_id, m2.world_size, m2.collective_world)
        info = rt.get_tensor_info(m2)
        ins = {{n: SpikeTensor.empty(tuple(t.shape), np.float32, n).tensor_ref for n, t in dict(info.inputs).items()}}
        outs = {{n: SpikeTensor.empty(tuple(t.shape), np.float32, n).tensor_ref for n, t in dict(info.outputs).items()}}
        print(expect(lambda: rt.execute(m2, ins, outs, "", False)))               # no peer table yet
        print(expect(lambda: m2.set_collective_workspace([4096])))                # one entry for two ranks
        ws = [SpikeTensor.empty((m2.workspace_bytes,), np.uint8, f"ws{{r}}") for r in range(2)]
        m2.set_collective_workspace([w.va for w in ws])
        print(expect(lambda: m2.set_collective_workspace([w.va for w in ws])))    # only once
        rt.execute(m2, ins, outs, "", False)
        print("executed", m2.num_launches)
    """, log=log)
    lines = out.splitlines()
    assert lines[0] == "True 1 True" and "already set" in lines[1]
    assert "load it with cc_enabled and world_size 2" in lines[2] and "world_size 2" in lines[3]
    assert "rank_id < world_size" in lines[4]
    assert lines[5] == "True 1 2 2"
    assert "set_collective_workspace" in lines[6] and "needs 2 entries" in lines[7] and "already set" in lines[8]
    assert lines[9].startswith("executed ")
    launched = [ln.split()[1] for ln in log.read_text().splitlines() if ln.startswith("launch ")]
    assert len(launched) == int(lines[9].split()[1])
    kinds = {k.split("_", 1)[1] for k in launched}
    assert {"cc_push", "cc_all_reduce", "cc_all_gather", "cc_reduce_scatter", "cc_all_to_all"} <= kinds


# ------------------------------------------------------------------ the spike-run command line, end to end
def _cli(fake_lib, args, env=None, cwd=None):
    e = dict(os.environ, LD_LIBRARY_PATH=str(fake_lib), PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    e.pop("CUDA_VISIBLE_DEVICES", None)
    e.update(env or {})
    return subprocess.run([sys.executable, "-W", "ignore", "-m", "nkipy_b200.spike.cli", *args], capture_output=True,
                          text=True, timeout=300, env=e, cwd=cwd)


def test_cli_single_core_run_benchmark_and_trace(fake_lib, compiled, tmp_path):
    path, plan = compiled
    a = np.ones((8, 16), np.float32)
    np.save(tmp_path / "a.npy", a)
    log = tmp_path / "log.txt"
    res = _cli(fake_lib, [path, "-i", f"a={tmp_path / 'a.npy'}", "--output-dir", str(tmp_path / "out")],
               env={"FAKE_CUDA_LOG": str(log)})
    assert res.returncode == 0, res.stderr[-2000:]
    produced = sorted(os.listdir(tmp_path / "out"))
    assert len(produced) == 2 and all(p.endswith(".npy") for p in produced)        # b was not given: zeros
    shapes = sorted(np.load(tmp_path / "out" / p).shape for p in produced)
    assert shapes == [(8, 4), (16,)]
    assert sum(ln.startswith("launch ") for ln in log.read_text().splitlines()) == len(plan["launches"])
    # without an output directory the results are summarised on stdout
    res = _cli(fake_lib, [path])
    assert res.returncode == 0 and res.stdout.count("[core 0]") == 2 and "shape=(8, 4)" in res.stdout
    # benchmark: warm-up + iterations executes, the statistics come from device events
    log.write_text("")
    res = _cli(fake_lib, [path, "--benchmark", "--warmup", "2", "--iterations", "3"],
               env={"FAKE_CUDA_LOG": str(log), "FAKE_CUDA_EVENT_MS": "0.125"})
    assert res.returncode == 0, res.stderr[-2000:]
    assert "over 3 iterations (2 warm-up)" in res.stdout and f"mean {0.125 * len(plan['launches']):.4f} ms" in res.stdout
    assert sum(ln.startswith("launch ") for ln in log.read_text().splitlines()) == 5 * len(plan["launches"])
    # trace file
    res = _cli(fake_lib, [path, "--save-trace", "--ntff-name", str(tmp_path / "trace.json")])
    assert res.returncode == 0, res.stderr[-2000:]
    trace_doc = json.loads((tmp_path / "trace.json").read_text())
    assert trace_doc and json.dumps(trace_doc).count(plan["launches"][0]["kernel"]) >= 1


def test_cli_rejects_bad_inputs(fake_lib, compiled, tmp_path):
    path, _ = compiled
    np.save(tmp_path / "wrong.npy", np.ones((3, 3), np.float32))
    res = _cli(fake_lib, [path, "-i", f"a={tmp_path / 'wrong.npy'}"])
    assert res.returncode != 0 and "expected shape (8, 16)" in res.stderr
    res = _cli(fake_lib, [path, "-i", "a"])
    assert res.returncode != 0 and "expected name=path.npy" in res.stderr
    res = _cli(fake_lib, [str(tmp_path / "missing.cubin")])
    assert res.returncode != 0
    res = _cli(fake_lib, [path, "--cc-enabled", "--rank-id", "3", "--world-size", "2"])
    assert res.returncode != 0 and "--rank-id" in res.stderr


def test_cli_multi_core_expands_rank_in_input_names(fake_lib, compiled, tmp_path):
    path, _ = compiled
    for r in range(2):
        np.save(tmp_path / f"a_{r}.npy", np.full((8, 16), float(r + 1), np.float32))
    log = tmp_path / "log.txt"
    res = _cli(fake_lib, [path, "--num-cores", "2", "-i", f"a={tmp_path}/a_{{rank}}.npy", "--output-dir", str(tmp_path / "out")],
               env={"FAKE_CUDA_DEVICES": "2", "FAKE_CUDA_LOG": str(log)})
    assert res.returncode == 0, res.stderr[-2000:]
    assert sorted(os.listdir(tmp_path / "out")) == ["core_0", "core_1"]
    assert all(len(os.listdir(tmp_path / "out" / f"core_{r}")) == 2 for r in range(2))
    # more cores than devices
    res = _cli(fake_lib, [path, "--num-cores", "2"], env={"FAKE_CUDA_DEVICES": "1"})
    assert res.returncode != 0


# ------------------------------------------------------------------ one-shot execution and the kernel cache
def test_jit_and_one_shot_execution_flow(fake_dir, tmp_path):
    """Trace -> compile -> load -> run -> read back, as the reference's tests/integration/test_execute.py does on a
    device.  The stand-in driver computes nothing, so the checks are on shapes, dtypes, names, write-back and files."""
    out = run_child(fake_dir, f"""
        import os
        from nkipy_b200.runtime import baremetal_jit, baremetal_run_traced_kernel, BaremetalExecutor, CompiledKernel
        from nkipy_b200.core.compile import trace, compile_to_neff

        def kernel(a, b):
            return np.tanh(a @ b), a.sum(axis=0)

        a, b = np.ones((8, 16), np.float32), np.ones((16, 4), np.float32)
        assert [x.shape for x in kernel(a, b)] == [(8, 4), (16,)]                  # direct mode needs no device
        o = baremetal_jit(kernel)(a, b)
        print([x.shape for x in o], [str(x.dtype) for x in o])
        o = baremetal_jit(kernel)(a.astype(np.float64), b.astype(np.float64))      # wide inputs are narrowed
        print([str(x.dtype) for x in o])
        print(baremetal_jit(lambda x: x[:, :0] * 2.0)(a).shape)                    # an empty result never reaches the device

        def update(cache, v):
            cache[2:4] = v
            return np.sum(cache, axis=0)

        cache = np.arange(128, dtype=np.float32).reshape(8, 16)
        r = baremetal_run_traced_kernel(update, cache, np.ones((2, 16), np.float32), artifacts_dir={str(tmp_path)!r},
                                        save_trace=True)
        print(r.shape, cache.shape, str(cache.dtype))                               # the mutated input is read back from the device
        print(sorted(f for f in os.listdir({str(tmp_path)!r}) if f.endswith(".json"))[:3])

        k = trace(kernel); k.specialize(a, b)
        ck = CompiledKernel(k, compile_to_neff(k, {str(tmp_path / 'ck')!r}, "k.cubin"))
        with BaremetalExecutor() as ex:
            r = ex.run(ck, a, b)
            st = ex.benchmark(ck, a, b, warmup_iterations=1, benchmark_iterations=4)
        print([x.shape for x in r], st.iterations, st.warmup_iterations)
    """)
    lines = out.splitlines()
    assert lines[0] == "[(8, 4), (16,)] ['float32', 'float32']" and lines[1] == "['float32', 'float32']"
    assert lines[2] == "(8, 0)"
    assert lines[3] == "(16,) (8, 16) float32"
    assert any("trace" in f for f in eval(lines[4]))
    assert lines[5] == "[(8, 4), (16,)] 4 1"


def test_kernel_cache_in_memory_and_on_disk(fake_dir, tmp_path):
    build = str(tmp_path / "build")
    body = f"""
        from nkipy_b200.runtime import DeviceKernel, device_kernel as DK
        def mm(a, b):
            return a @ b
        a, b = np.ones((8, 16), np.float32), np.ones((16, 4), np.float32)
        if sys.argv[-1] == "second":
            def refuse(*args, **kw):
                raise AssertionError("compiled again although the artifact is on disk")
            DK.compile_to_neff = refuse
        k1 = DeviceKernel.compile_and_load(mm, a, b, name="mm", build_dir={build!r})
        k2 = DeviceKernel.compile_and_load(mm, a, b, name="mm", build_dir={build!r})
        k3 = DeviceKernel.compile_and_load(mm, a[:4], b, name="mm", build_dir={build!r}) if sys.argv[-1] != "second" else None
        print(k1 is k2, k3 is not k1 if k3 is not None else "-", k1.neff_path.startswith({build!r}))
    """
    log = tmp_path / "log.txt"
    out = run_child(fake_dir, body, log=log)
    assert out.split() == ["True", "True", "True"]
    assert log.read_text().count("module_load") == 2                               # two shapes, each loaded once
    # a new process finds the artifact on disk
    code_env = {"FAKE_CUDA_LOG": str(log)}
    log.write_text("")
    out = run_child(fake_dir, body.replace('sys.argv[-1]', '"second"'), env=code_env)
    assert out.split() == ["True", "-", "True"] and log.read_text().count("module_load") == 1


def test_symmetric_memory_bootstrap_over_gloo_ranks(fake_lib, tmp_path):
    """`parallel.symm.SymmetricMemory` end to end on two host processes: gloo for the barriers, Unix sockets for the
    descriptors, the C++ `SymmetricBuffer` on the stand-in driver for the mappings, a multicast object on top; then the
    collective close, and on a second buffer the one-sided `abandon()` of the recovery path."""
    body = """
        import ctypes, datetime, os, sys
        import torch, torch.distributed as dist
        rank, world, port = int(sys.argv[1]), 2, sys.argv[2]
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=60))
        from nkipy_b200.parallel.comm import TPGroup
        from nkipy_b200.parallel.symm import SymmetricMemory
        tp = TPGroup(rank, world, dist.group.WORLD, torch.device("cpu"))
        mem = SymmetricMemory(tp, 1 << 16, multicast=True)
        assert mem.backend == "vmm" and len(mem.ptrs) == 2 and mem.ptrs[rank] == mem.local_ptr and mem.mc_ptr != 0
        ctypes.memmove(mem.ptrs[1 - rank] + 256, b"rank %d was here" % rank, 15)
        tp.barrier()
        print(ctypes.string_at(mem.local_ptr + 256, 15).decode())
        mem.close(); mem.close()
        second = SymmetricMemory(tp, 4096, multicast=False)
        assert second.mc_ptr == 0
        tp.barrier()
        second.abandon()                       # no barrier inside: either rank may go first
        print("closed")
        dist.destroy_process_group()
    """
    import socket

    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    code = "import sys\nsys.path.insert(0, %r)\n" % ROOT + textwrap.dedent(body)
    logs = [tmp_path / f"log{r}.txt" for r in range(2)]
    procs = []
    for r in range(2):
        env = dict(os.environ, LD_LIBRARY_PATH=str(fake_lib), FAKE_CUDA_DEVICES="2", FAKE_CUDA_LOG=str(logs[r]),
                   NKIPY_B200_NVLS="1")
        env.pop("CUDA_VISIBLE_DEVICES", None)
        procs.append(subprocess.Popen([sys.executable, "-W", "ignore", "-c", code, str(r), str(port)], env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    outs = [p.communicate(timeout=240) for p in procs]
    assert [p.returncode for p in procs] == [0, 0], outs
    assert outs[0][0].split("\n")[:2] == ["rank 1 was here", "closed"] and outs[1][0].split("\n")[:2] == ["rank 0 was here", "closed"]
    for log in logs:
        text = log.read_text()
        assert text.count("multicast_bind") == 1 and text.count("multicast_unbind") == 1
        assert "mem_release live_handles=0" in text.splitlines()[-1]
        assert not any(bad in text for bad in ("bad_release", "bad_unmap", "bad_unbind", "address_free_while_mapped"))


def test_profiler_adapter_logs_each_execute_on_rank_zero_only(fake_lib, compiled, tmp_path):
    path, _ = compiled
    fake = FakeEnv(fake_lib, None, None)
    out = run_child(fake, f"""
        import os
        from nkipy_b200.spike import SpikeProfiler, SpikeTensor, get_spike_singleton
        rt = get_spike_singleton()
        m = rt.load_model({path!r}, 0, False, 0, 1)
        info = rt.get_tensor_info(m)
        ins = {{n: SpikeTensor.empty(tuple(t.shape), np.float32, n).tensor_ref for n, t in dict(info.inputs).items()}}
        outs = {{n: SpikeTensor.empty(tuple(t.shape), np.float32, n).tensor_ref for n, t in dict(info.outputs).items()}}
        for rank in (0, 1):
            prof = SpikeProfiler(rt, log_dir={str(tmp_path)!r}, rank=rank)
            prof.execute(m, ins, outs)
            prof.execute(m, ins, outs)
            assert prof.sm_count == rt.sm_count                    # everything else is passed through
        print(sorted(os.listdir({str(tmp_path)!r})), os.getpid())
    """)
    files, pid = out.strip().rsplit(" ", 1)
    assert "debug_rank_0.txt" in files and "debug_rank_1.txt" not in files
    text = (tmp_path / "debug_rank_0.txt").read_text()
    assert text.count(f"PID {pid}\n") == 2 and text.count("SOURCE ") == 2 and text.count(f"({path})") == 2
