"""`DeviceKernel.compile_and_load` under a (mocked) process group: rank 0 traces and compiles, the path is
broadcast, every rank loads with its rank / world size; MPMD mode compiles per rank
(mirrors the reference's tests/unit/test_device_kernel_cc.py, which mocks torch.distributed the same way)."""
import os

import numpy as np
import pytest

from nkipy_b200.runtime import device_kernel as DK


class FakeDist:
    def __init__(self, rank, world, payload_box):
        self.rank, self.world, self.box = rank, world, payload_box
        self.barriers = 0

    def is_available(self):
        return True

    def is_initialized(self):
        return True

    def get_world_size(self):
        return self.world

    def get_rank(self):
        return self.rank

    def broadcast_object_list(self, payload, src=0):
        if self.rank == src:
            self.box[:] = list(payload)
        else:
            payload[:] = list(self.box)

    def barrier(self):
        self.barriers += 1


@pytest.fixture
def patched(monkeypatch, tmp_path):
    calls = {"compile": [], "load": []}
    box = []

    def fake_compile(ir, out_dir, name, **kw):
        os.makedirs(out_dir, exist_ok=True)
        path = os.path.join(out_dir, name)
        open(path, "w").write("cubin")
        open(os.path.splitext(path)[0] + ".json", "w").write("{}")
        calls["compile"].append(path)
        return path

    def fake_load(cls, neff_path, name=None, core_id=0, cc_enabled=False, rank_id=0, world_size=1):
        calls["load"].append(dict(path=neff_path, cc=cc_enabled, rank=rank_id, world=world_size))
        obj = object.__new__(cls)
        obj.neff_path = neff_path
        return obj

    monkeypatch.setattr(DK, "compile_to_neff", fake_compile)
    monkeypatch.setattr(DK.DeviceKernel, "load_from_neff", classmethod(fake_load))
    DK._LOADED_KERNELS.clear()

    def use(rank, world):
        fd = FakeDist(rank, world, box)
        monkeypatch.setattr(DK, "_dist", lambda: fd)
        return fd

    return calls, use, str(tmp_path)


def kern(a, b):
    return a @ b + 1.0


def test_spmd_rank0_compiles_and_everyone_loads_with_its_rank(patched):
    calls, use, build = patched
    a, b = np.ones((4, 8), np.float32), np.ones((8, 4), np.float32)
    fd0 = use(0, 2)
    k0 = DK.DeviceKernel.compile_and_load(kern, a, b, name="mm", build_dir=build)
    assert len(calls["compile"]) == 1 and fd0.barriers == 1
    DK._LOADED_KERNELS.clear()
    fd1 = use(1, 2)
    k1 = DK.DeviceKernel.compile_and_load(kern, a, b, name="mm", build_dir=build)
    assert len(calls["compile"]) == 1                       # rank 1 did not compile
    assert k0.neff_path == k1.neff_path and fd1.barriers == 1
    assert [c["rank"] for c in calls["load"]] == [0, 1]
    assert all(c["cc"] and c["world"] == 2 for c in calls["load"])


def test_mpmd_compiles_per_rank_and_cache_hits(patched):
    calls, use, build = patched
    a, b = np.ones((4, 8), np.float32), np.ones((8, 4), np.float32)
    use(1, 2)
    k = DK.DeviceKernel.compile_and_load(kern, a, b, name="mm", build_dir=build, is_spmd=False)
    assert "rank_1" in k.neff_path and len(calls["compile"]) == 1
    again = DK.DeviceKernel.compile_and_load(kern, a, b, name="mm", build_dir=build, is_spmd=False)
    assert again is k and len(calls["compile"]) == 1         # in-memory cache
    DK._LOADED_KERNELS.clear()
    DK.DeviceKernel.compile_and_load(kern, a, b, name="mm", build_dir=build, is_spmd=False)
    assert len(calls["compile"]) == 1                       # on-disk cache
    DK.DeviceKernel.compile_and_load(kern, a, b, name="mm", build_dir=build, is_spmd=False,
                                     use_cached_if_exists=False, additional_compiler_args="-O2")
    assert len(calls["compile"]) == 2                       # different compiler arguments: new key


def test_explicit_rank_and_validation(patched):
    calls, use, build = patched
    a, b = np.ones((4, 8), np.float32), np.ones((8, 4), np.float32)
    use(0, 1)
    DK.DeviceKernel.compile_and_load(kern, a, b, name="mm", build_dir=build, cc_enabled=True, rank_id=3, world_size=4)
    assert calls["load"][-1] == dict(path=calls["load"][-1]["path"], cc=True, rank=3, world=4)
    DK._LOADED_KERNELS.clear()
    with pytest.raises(ValueError):
        DK.DeviceKernel.compile_and_load(kern, a, b, name="mm", build_dir=build, cc_enabled=True, rank_id=4,
                                         world_size=4)
    DK._LOADED_KERNELS.clear()
    DK.DeviceKernel.compile_and_load(kern, a, b, name="mm", build_dir=build)        # single process: no collectives
    assert calls["load"][-1]["cc"] is False and calls["load"][-1]["world"] == 1
