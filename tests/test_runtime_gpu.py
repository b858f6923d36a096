"""Traced kernels compiled to cubins and run through the C++ device runtime on a B200."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

R = np.random.default_rng(0)


def f32(*s):
    return R.standard_normal(s).astype(np.float32)


def run(fn, *args, **kw):
    from nkipy_b200.runtime import baremetal_run_traced_kernel

    return baremetal_run_traced_kernel(fn, *args, **kw)


def check(fn, *args, rtol=1e-4, atol=1e-4):
    import copy

    exp = fn(*copy.deepcopy(args))
    got = run(fn, *args)
    exp = exp if isinstance(exp, tuple) else (exp,)
    got = got if isinstance(got, tuple) else (got,)
    for e, g in zip(exp, got):
        e = np.asarray(e)
        assert g.shape == e.shape
        np.testing.assert_allclose(g.astype(np.float64), e.astype(np.float64), rtol=rtol, atol=atol)


def test_softmax_and_mlp_jit():
    def softmax(x):
        e = np.exp(x - np.max(x, axis=-1, keepdims=True))
        return e / np.sum(e, axis=-1, keepdims=True)

    check(softmax, f32(128, 512), atol=1e-5)

    def mlp(x, w1, w2):
        h = x @ w1
        h = 0.5 * h * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (h + 0.044715 * h ** 3)))
        return h @ w2

    check(mlp, f32(64, 256), f32(256, 1024) * 0.02, f32(1024, 256) * 0.02, atol=1e-4)


def test_elementwise_views_reductions():
    x, y = f32(6, 8, 10), f32(8, 10)
    check(lambda a, b: np.tanh(a * 2 + b) / (1 + np.abs(b)), x, y)
    check(lambda a: a.transpose(2, 0, 1)[::2, 1:, ::3] * 1.5, x)
    check(lambda a: np.sum(a, axis=(0, 2)) + np.max(a, axis=(0, 2)), x, rtol=1e-3)
    check(lambda a: (a.reshape(48, 10).T @ a.reshape(48, 10)), x, rtol=1e-3, atol=1e-3)
    check(lambda a: np.where(a > 0, a, 0.1 * a).mean(axis=-1), x)
    check(lambda a: np.concatenate([a[:2], a[4:]], axis=0), x)
    check(lambda a: np.pad(a[0], ((1, 2), (0, 3)), constant_values=-1.0), x)
    check(lambda a: np.argmax(a, axis=1) + np.argmin(a, axis=1), x)
    check(lambda a: np.cumsum(a[0], axis=0), x, rtol=1e-3)


def test_indexing_scatter_topk_conv():
    from nkipy_b200.core import tensor_apis

    x = f32(6, 8, 10)
    idx = np.array([4, 0, 3], dtype=np.int32)
    check(lambda a, i: a[:, i] * 2, x, idx)
    check(lambda a: a[[0, 1], :, [2, 3]], x)
    check(lambda a, i: np.take_along_axis(a, i, axis=2), x, R.integers(0, 10, (6, 8, 2)).astype(np.int32))

    def assign(a, v):
        a[1:3, ::2] = v
        return a

    check(assign, x.copy(), f32(2, 4, 10))

    def scatter(a, i, v):
        a[:, i] = v
        return a * 1.0

    check(scatter, x.copy(), idx, f32(6, 3, 10))
    check(lambda a: tensor_apis.topk(a, 3)[0], f32(5, 40))
    got = run(lambda a: tensor_apis.topk(a, 3)[1], x[0])
    assert got.dtype == np.uint32 and np.array_equal(got, np.argsort(-x[0], axis=-1, kind="stable")[:, :3])
    check(lambda i, k, b: tensor_apis.conv2d(i, k, b, stride=2, padding=1), f32(2, 4, 9, 9), f32(6, 4, 3, 3), f32(6),
          rtol=1e-3, atol=1e-3)


def test_bf16_matmul_uses_tcgen05_template():
    import ml_dtypes

    from nkipy_b200.core.compile import lower_to_cuda, trace

    a = f32(256, 512).astype(ml_dtypes.bfloat16)
    b = (f32(512, 384) * 0.05).astype(ml_dtypes.bfloat16)

    def mm(x, w):
        return x @ w

    k = trace(mm)
    k.specialize(a, b)
    assert "gemm_bf16_body" in lower_to_cuda(k)
    got = run(mm, a, b)
    ref = a.astype(np.float32) @ b.astype(np.float32)
    err = np.linalg.norm(got.astype(np.float32) - ref) / np.linalg.norm(ref)
    assert err < 1e-2, err


def test_alias_writes_back_and_device_kernel_cache(tmp_path):
    from nkipy_b200.runtime import DeviceKernel, DeviceTensor

    def upd(cache, v):
        cache[2:4] = v
        return cache.sum(axis=0)

    cache, v = f32(8, 16), f32(2, 16)
    before = cache.copy()
    out = run(upd, cache, v)
    before[2:4] = v
    np.testing.assert_allclose(cache, before)          # mutated input written back
    np.testing.assert_allclose(out, before.sum(0), rtol=1e-4, atol=1e-4)

    def mm(a, b):
        return a @ b

    a, b = f32(64, 32), f32(32, 16)
    k1 = DeviceKernel.compile_and_load(mm, a, b, name="mm", build_dir=str(tmp_path))
    k2 = DeviceKernel.compile_and_load(mm, a, b, name="mm", build_dir=str(tmp_path))
    assert k1 is k2
    ta, tb = DeviceTensor.from_numpy(a, "a"), DeviceTensor.from_numpy(b, "b")
    res = k1(inputs={"a": ta, "b": tb})
    np.testing.assert_allclose(res["output0"].numpy(), a @ b, rtol=1e-3, atol=1e-3)
    bench = k1.benchmark({"a": ta, "b": tb}, warmup_iterations=2, benchmark_iterations=5, mode="device")
    assert bench.iterations == 5 and bench.mean_ms > 0
    with pytest.raises(ValueError):
        k1(inputs={"a": ta})
    ta.write_from_numpy(a * 2)
    np.testing.assert_allclose(ta.numpy(), a * 2)
    with pytest.raises(ValueError):
        ta.write_from_numpy(np.zeros(3, np.float32))
    import torch

    tt = DeviceTensor.from_torch(torch.arange(6, dtype=torch.bfloat16).reshape(2, 3))
    assert torch.equal(tt.torch(), torch.arange(6, dtype=torch.bfloat16).reshape(2, 3))


def test_runtime_lifecycle_in_subprocess():
    code = """
import numpy as np, sys
sys.path.insert(0, %r)
from nkipy_b200 import spike
from nkipy_b200.spike import SpikeTensor, get_spike_singleton
from nkipy_b200.spike.spike_singleton import _native
_spike = _native()
rt = get_spike_singleton()
assert rt.sm_count > 0 and 'B200' in rt.device_name or rt.sm_count > 0
t = SpikeTensor.from_numpy(np.arange(16, dtype=np.float32))
s = t.slice_bytes(16, (4,), np.float32)
assert s.numpy().tolist() == [4, 5, 6, 7]
try:
    rt.tensor_read(t.tensor_ref, 0, 1000)
    raise SystemExit('no bounds error')
except _spike.SpikeError:
    pass
try:
    _spike.Spike()
    raise SystemExit('second runtime allowed')
except _spike.SpikeError:
    pass
t.free()
try:
    t.numpy()
    raise SystemExit('read after free allowed')
except _spike.SpikeError:
    pass
with _spike.SystemTraceSession(0) as sess:
    assert 'events' in sess.fetch_events_json()
keep = SpikeTensor.from_numpy(np.ones(4, np.float32))
spike.reset()           # tensors outlive the runtime: their destructors must be harmless
print('LIFECYCLE_OK')
""" % os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    res = subprocess.run([sys.executable, "-W", "ignore", "-c", code], capture_output=True, text=True, timeout=120)
    assert "LIFECYCLE_OK" in res.stdout, res.stdout + res.stderr


def test_custom_cuda_op_and_native_backend_on_device(tmp_path):
    from nkipy_b200 import nkigen
    from nkipy_b200.core.cuda_op import cuda_custom_op
    from nkipy_b200.nkigen.compile import compile_to_neff
    from nkipy_b200.runtime import DeviceKernel, DeviceTensor

    src = ('extern "C" __global__ void scale_add_kernel(const float* a, const float* b, float* out) {'
           ' int i = blockIdx.x * blockDim.x + threadIdx.x; if (i < 4096) out[i] = 2.f * a[i] + b[i]; }')
    op = cuda_custom_op("scale_add", src, "scale_add_kernel", [((4096,), "f32")], grid=(16,), block=(256,),
                        reference=lambda a, b: 2 * a + b)
    a, b = f32(4096), f32(4096)
    check(lambda x, y: op(x, y) * 0.5 + 1, a, b)

    @nkigen.trace(input_specs=[((64, 128), "f32"), ((96, 128), "f32")])
    def k(x, w):
        h = x @ np.transpose(w, (1, 0))
        return np.tanh(h + np.zeros_like(h)) ** 2

    path = compile_to_neff(k, str(tmp_path), "k.cubin", dump_dir=str(tmp_path / "dump"))
    model = DeviceKernel.load_from_neff(path)
    x, w = f32(64, 128), f32(96, 128)
    out = model({"in_tensor_0": DeviceTensor.from_numpy(x), "in_tensor_1": DeviceTensor.from_numpy(w)})
    np.testing.assert_allclose(out["output"].numpy(), np.tanh(x @ w.T) ** 2, rtol=1e-3, atol=1e-4)


def _run_nkigen(kernel, tmp, inputs, name="k"):
    """Compile a nkigen-traced kernel through the native pass pipeline and run it on the device."""
    from nkipy_b200.nkigen.compile import compile_to_neff
    from nkipy_b200.runtime import DeviceKernel, DeviceTensor

    path = compile_to_neff(kernel, str(tmp), f"{name}.cubin")
    plan = json.loads(open(os.path.splitext(path)[0] + ".json").read())
    model = DeviceKernel.load_from_neff(path)
    out = model({f"in_tensor_{i}": DeviceTensor.from_numpy(a) for i, a in enumerate(inputs)})
    return out, plan


def test_knobs_change_the_emitted_gemm_and_not_its_result(tmp_path):
    import ml_dtypes

    from nkipy_b200 import nkigen

    bf = ml_dtypes.bfloat16
    x, w = f32(512, 1024).astype(bf), (f32(768, 1024) * 0.05).astype(bf)
    ref = x.astype(np.float32) @ w.astype(np.float32).T
    results, shapes = [], []
    for i, tile in enumerate((None, [128, 64], [128, 128])):
        @nkigen.trace(input_specs=[((512, 1024), "bf16"), ((768, 1024), "bf16")])
        def mm(a, b):
            y = a @ b.T
            if tile:
                nkigen.knob(y).tile_op(tile_size=tile)
            return y

        out, plan = _run_nkigen(mm, tmp_path / f"t{i}", [x, w])
        ga = plan["launches"][0]["args"][2]["gemm_args"]
        shapes.append((ga["block_n"], ga["stages"]))
        results.append(out["output"].numpy().astype(np.float32))
    assert [s[0] for s in shapes] == [256, 64, 128] and len({s[1] for s in shapes}) >= 2
    for r in results:
        assert np.linalg.norm(r - ref) / np.linalg.norm(ref) < 1e-2
    for r in results[1:]:
        # the same k-order and fp32 accumulation whatever the tile: identical bf16 results
        np.testing.assert_array_equal(r, results[0])


def test_fused_gemm_epilogue_on_device(tmp_path):
    import ml_dtypes

    from nkipy_b200 import nkigen

    bf = ml_dtypes.bfloat16

    @nkigen.trace(input_specs=[((256, 512), "bf16"), ((384, 512), "bf16"), ((384,), "bf16"), ((256, 384), "bf16")])
    def k(x, w, b, r):
        z = x @ w.T + b
        return z / (1.0 + np.exp(-z)) + r

    x, w = f32(256, 512).astype(bf), (f32(384, 512) * 0.05).astype(bf)
    b, r = f32(384).astype(bf), f32(256, 384).astype(bf)
    out, plan = _run_nkigen(k, tmp_path, [x, w, b, r])
    assert len(plan["launches"]) == 1 and plan["launches"][0]["args"][2]["gemm_args"]["fused_epilogue"]
    z = x.astype(np.float32) @ w.astype(np.float32).T + b.astype(np.float32)
    ref = z / (1.0 + np.exp(-z)) + r.astype(np.float32)
    got = out["output"].numpy().astype(np.float32)
    assert np.linalg.norm(got - ref) / np.linalg.norm(ref) < 1e-2
    # per 128-column block, so that a wrong tile cannot hide in the norm
    for c in range(0, 384, 128):
        e = np.linalg.norm(got[:, c:c + 128] - ref[:, c:c + 128]) / np.linalg.norm(ref[:, c:c + 128])
        assert e < 1.5e-2, (c, e)


def test_loop_kernel_on_device(tmp_path):
    from nkipy_b200 import nkigen

    @nkigen.trace(input_specs=[((6, 32), "f32"), ((32, 32), "f32")])
    def k(x, w):
        def body(i, h):
            return np.tanh(h @ w + x[i])

        return nkigen.fori_loop(0, 6, body, np.zeros(32, np.float32))

    x, w = f32(6, 32), f32(32, 32) * 0.3
    out, plan = _run_nkigen(k, tmp_path, [x, w])
    np.testing.assert_allclose(out["output"].numpy(), k(x, w), rtol=1e-4, atol=1e-5)


def test_softmax_and_rms_norm_ops_are_single_launches(tmp_path):
    """`tensor_apis.softmax` / `rms_norm` over the last axis are one node and one row kernel each."""
    from nkipy_b200.core import tensor_apis as T
    from nkipy_b200.core.compile import compile_to_neff, trace

    def k(x, w):
        return T.softmax(x), T.rms_norm(x, w, 1e-5), T.rms_norm(x * 2.0)

    x, w = f32(33, 1000), f32(1000)
    check(k, x, w, rtol=1e-4, atol=1e-5)
    kern = trace(k)
    kern.specialize(x, w)
    compile_to_neff(kern, str(tmp_path), "rows.cubin")
    plan = json.load(open(tmp_path / "rows.json"))
    names = [l["kernel"].split("_", 1)[1] for l in plan["launches"]]
    assert names.count("softmax") == 1 and names.count("rms_norm") == 2 and "reduce" not in names
    import ml_dtypes

    xb, wb = x.astype(ml_dtypes.bfloat16), w.astype(ml_dtypes.bfloat16)
    check(lambda a, b: (T.softmax(a), T.rms_norm(a, b)), xb, wb, rtol=2e-2, atol=2e-2)
