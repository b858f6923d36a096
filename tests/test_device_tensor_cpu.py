"""`SpikeTensor` / `DeviceTensor` against a host-memory stand-in for the runtime: construction, round trips through
NumPy and torch, in-place overwrites (same allocation, same metadata), size checks, non-contiguous sources, byte-range
views and extended dtypes.  Cases follow the reference's tests/integration/test_write_from.py and
test_device_kernel_tensor.py (round-trip part); the same calls run against the real runtime in tests/test_runtime_gpu.py."""
import numpy as np
import pytest
import torch

from nkipy_b200.core.dtypes import bfloat16
from nkipy_b200.runtime.device_tensor import DeviceTensor
from nkipy_b200.spike import spike_tensor as ST
from nkipy_b200.spike.spike_tensor import SpikeTensor


class _Ref:
    def __init__(self, buf, core_id, name, offset=0, nbytes=None):
        self.buf, self.core_id, self.name, self.offset = buf, core_id, name, offset
        self.nbytes = len(buf) if nbytes is None else nbytes
        self.va = 0x7000_0000_0000 + id(buf) % (1 << 20) * 256 + offset
        self.freed = False


class FakeRuntime:
    """Just enough of the runtime's tensor calls, on bytearrays."""

    def __init__(self):
        self.allocations = 0
        self.writes = 0

    def allocate_tensor(self, nbytes, core_id, name):
        self.allocations += 1
        return _Ref(bytearray(nbytes), core_id, name)

    def tensor_write(self, ref, data, offset):
        assert not ref.freed and data.dtype == np.uint8 and data.ndim == 1 and data.flags.c_contiguous
        assert offset + data.size <= ref.nbytes
        self.writes += 1
        ref.buf[ref.offset + offset: ref.offset + offset + data.size] = data.tobytes()

    def tensor_read_to_buffer(self, ref, out, offset):
        assert not ref.freed and out.dtype == np.uint8 and out.ndim == 1
        out[:] = np.frombuffer(ref.buf, np.uint8, out.size, ref.offset + offset)

    def slice_from_tensor(self, ref, offset, nbytes, name):
        if offset + nbytes > ref.nbytes:
            raise ValueError("slice outside the allocation")
        return _Ref(ref.buf, ref.core_id, name, ref.offset + offset, nbytes)

    def free_tensor(self, ref):
        ref.freed = True


@pytest.fixture
def rt(monkeypatch):
    fake = FakeRuntime()
    monkeypatch.setattr(ST, "get_spike_singleton", lambda: fake)
    import nkipy_b200.spike.spike_singleton as SS

    monkeypatch.setattr(SS, "get_spike_singleton", lambda: fake)          # DeviceTensor looks it up there at call time
    return fake


R = np.random.default_rng(2)


@pytest.mark.parametrize("cls", [SpikeTensor, DeviceTensor])
@pytest.mark.parametrize("dtype", [np.float32, np.float16, np.int32, np.int8, np.uint8, bfloat16])
@pytest.mark.parametrize("shape", [(32,), (4, 8), (2, 3, 4), ()])
def test_numpy_round_trip(rt, cls, dtype, shape):
    src = (R.random(shape) * 100).astype(dtype)
    t = cls.from_numpy(src, name="x")
    assert isinstance(t, cls) and t.shape == tuple(shape) and t.dtype == np.dtype(dtype) and t.name == "x"
    assert t.nbytes == src.nbytes
    back = t.numpy()
    assert back.shape == src.shape and back.dtype == src.dtype
    assert back.tobytes() == src.tobytes()


def test_empty_tensor_and_zero_size(rt):
    t = SpikeTensor.empty((4, 4), np.float32, name="e", core_id=0)
    assert t.shape == (4, 4) and t.nbytes == 64 and t.numpy().shape == (4, 4)
    z = SpikeTensor.from_numpy(np.zeros((0, 8), np.float32))
    assert z.nbytes == 0 and z.numpy().shape == (0, 8) and rt.writes == 0


def test_write_from_numpy_overwrites_in_place(rt):
    a = R.standard_normal(128).astype(np.float32)
    t = DeviceTensor.from_numpy(a, name="w")
    ref, n_alloc = t.tensor_ref, rt.allocations
    for k in range(3):
        new = R.standard_normal(128).astype(np.float32)
        t.write_from_numpy(new)
        np.testing.assert_array_equal(t.numpy(), new)
    assert t.tensor_ref is ref and rt.allocations == n_alloc           # no reallocation
    assert (t.shape, t.dtype, t.name) == ((128,), np.dtype(np.float32), "w")


def test_write_from_numpy_two_dimensional_and_metadata(rt):
    t = DeviceTensor.from_numpy(np.zeros((8, 16), np.float32), name="m")
    new = R.standard_normal((8, 16)).astype(np.float32)
    t.write_from_numpy(new)
    assert t.shape == (8, 16) and t.name == "m"
    np.testing.assert_array_equal(t.numpy(), new)


def test_write_from_numpy_size_mismatch(rt):
    t = DeviceTensor.from_numpy(np.zeros(16, np.float32))
    with pytest.raises(ValueError, match="size mismatch"):
        t.write_from_numpy(np.zeros(8, np.float32))
    with pytest.raises(ValueError, match="size mismatch"):
        t.write_from_numpy(np.zeros(16, np.float16))
    t.write_from_numpy(np.ones((4, 4), np.float32))                     # same bytes, other shape: allowed
    np.testing.assert_array_equal(t.numpy(), np.ones(16, np.float32))


def test_non_contiguous_sources_are_packed(rt):
    base = R.standard_normal((8, 8)).astype(np.float32)
    t = DeviceTensor.from_numpy(base.T)
    np.testing.assert_array_equal(t.numpy(), base.T)
    t.write_from_numpy(base[:, ::-1])
    np.testing.assert_array_equal(t.numpy(), base[:, ::-1])
    strided = np.arange(32, dtype=np.float32)[::2]
    np.testing.assert_array_equal(DeviceTensor.from_numpy(strided).numpy(), strided)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16, torch.int32, torch.int8, torch.uint8,
                                   torch.float8_e4m3fn, torch.float8_e5m2, torch.bool])
def test_torch_round_trip(rt, dtype):
    src = (torch.rand(4, 8) * 10).to(dtype)
    t = DeviceTensor.from_torch(src, name="t")
    assert t.shape == (4, 8) and t.nbytes == src.numel() * src.element_size()
    back = t.torch()
    assert back.dtype == dtype and back.shape == src.shape
    assert torch.equal(back.view(torch.uint8), src.view(torch.uint8))


def test_write_from_torch(rt):
    t = DeviceTensor.from_torch(torch.zeros(8, 16))
    ref = t.tensor_ref
    for _ in range(2):
        new = torch.randn(8, 16)
        t.write_from_torch(new)
        assert torch.equal(t.torch(), new)
    assert t.tensor_ref is ref and t.shape == (8, 16)
    t.write_from_torch(torch.randn(16, 8).t())                           # non-contiguous source
    with pytest.raises(ValueError, match="size mismatch"):
        t.write_from_torch(torch.zeros(4, 16))
    with pytest.raises(ValueError, match="size mismatch"):
        t.write_from_torch(torch.zeros(8, 16, dtype=torch.bfloat16))


def test_numpy_and_torch_views_of_one_tensor_agree(rt):
    a = R.standard_normal((4, 4)).astype(np.float32)
    t = DeviceTensor.from_numpy(a)
    assert torch.equal(t.torch(), torch.from_numpy(a))
    t.write_from_torch(torch.full((4, 4), 7.0))
    np.testing.assert_array_equal(t.numpy(), np.full((4, 4), 7.0, np.float32))
    bf = DeviceTensor.from_torch(torch.arange(6, dtype=torch.bfloat16).reshape(2, 3))
    assert bf.dtype == bfloat16
    np.testing.assert_array_equal(bf.numpy().astype(np.float32), np.arange(6, dtype=np.float32).reshape(2, 3))


def test_unsupported_torch_dtype(rt):
    with pytest.raises(TypeError, match="unsupported torch dtype"):
        DeviceTensor.from_torch(torch.zeros(4, dtype=torch.complex64))


def test_byte_range_views_share_the_allocation(rt):
    a = np.arange(64, dtype=np.float32).reshape(8, 8)
    t = SpikeTensor.from_numpy(a, name="whole")
    rows = t.slice_bytes(2 * 8 * 4, (2, 8), name="rows")
    np.testing.assert_array_equal(rows.numpy(), a[2:4])
    rows.write_from_numpy(np.zeros((2, 8), np.float32))
    want = a.copy(); want[2:4] = 0
    np.testing.assert_array_equal(t.numpy(), want)
    as_bytes = t.slice_bytes(0, (16,), np.uint8)
    assert as_bytes.dtype == np.uint8 and as_bytes.nbytes == 16
    with pytest.raises(ValueError):
        t.slice_bytes(60 * 4, (8,), np.float32)
    assert rt.allocations == 1


def test_free_and_repr(rt):
    t = SpikeTensor.from_numpy(np.zeros(4, np.float32), name="gone", core_id=0)
    assert "gone" in repr(t) and "(4,)" in repr(t) and t.core_id == 0 and t.va > 0
    t.free()
    assert t.tensor_ref.freed
