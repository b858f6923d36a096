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
        self.broadcasts = 0

    def is_available(self):
        return True

    def is_initialized(self):
        return True

    def get_world_size(self):
        return self.world

    def get_rank(self):
        return self.rank

    def broadcast_object_list(self, payload, src=0):
        self.broadcasts += 1
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
        """Pretend to be `rank` of `world`; world 0 means torch.distributed is not initialised."""
        if world == 0:
            monkeypatch.setattr(DK, "_dist", lambda: None)
            return None
        fd = FakeDist(rank, world, box)
        monkeypatch.setattr(DK, "_dist", lambda: fd)
        return fd

    return calls, use, str(tmp_path)


def kern(a, b):
    return a @ b + 1.0


A = np.ones((4, 8), np.float32)
B = np.ones((8, 4), np.float32)


def load(build, **kw):
    return DK.DeviceKernel.compile_and_load(kern, A, B, name="mm", build_dir=build, **kw)


# ----------------------------------------------------------------------------- SPMD (the default)
def test_spmd_rank0_compiles_and_everyone_loads_with_its_rank(patched):
    calls, use, build = patched
    fd0 = use(0, 2)
    k0 = load(build)
    assert len(calls["compile"]) == 1 and fd0.barriers == 1 and fd0.broadcasts == 1
    DK._LOADED_KERNELS.clear()
    fd1 = use(1, 2)
    k1 = load(build)
    assert len(calls["compile"]) == 1                       # rank 1 did not compile
    assert k0.neff_path == k1.neff_path and fd1.barriers == 1 and fd1.broadcasts == 1
    assert [c["rank"] for c in calls["load"]] == [0, 1]
    assert all(c["cc"] and c["world"] == 2 for c in calls["load"])


def test_spmd_barrier_fires_also_with_explicit_cc(patched):
    calls, use, build = patched
    fd = use(0, 2)
    load(build, cc_enabled=True)
    assert fd.barriers == 1 and calls["load"][-1]["cc"] is True


def test_spmd_cc_false_keeps_broadcast_and_barrier_but_loads_without_collectives(patched):
    calls, use, build = patched
    fd = use(0, 2)
    load(build, cc_enabled=False)
    assert fd.broadcasts == 1 and fd.barriers == 1
    assert calls["load"][-1]["cc"] is False and calls["load"][-1]["world"] == 1


def test_spmd_explicit_rank_and_world_win_over_the_group(patched):
    calls, use, build = patched
    use(0, 2)
    load(build, cc_enabled=True, rank_id=5, world_size=16)
    assert (calls["load"][-1]["rank"], calls["load"][-1]["world"]) == (5, 16)


# ----------------------------------------------------------------------------- MPMD
def test_mpmd_compiles_per_rank_without_broadcast_or_barrier(patched):
    calls, use, build = patched
    fd = use(1, 2)
    k = load(build, is_spmd=False)
    assert f"{os.sep}rank_1{os.sep}" in k.neff_path and len(calls["compile"]) == 1
    assert fd.broadcasts == 0 and fd.barriers == 0
    assert calls["load"][-1] == dict(path=k.neff_path, cc=True, rank=1, world=2)     # collectives auto-detected


def test_mpmd_namespace_follows_the_explicit_rank(patched):
    calls, use, build = patched
    use(0, 2)
    k = load(build, is_spmd=False, cc_enabled=True, rank_id=3, world_size=8)
    assert f"{os.sep}rank_3{os.sep}" in k.neff_path
    assert (calls["load"][-1]["rank"], calls["load"][-1]["world"]) == (3, 8)


def test_mpmd_cc_false(patched):
    calls, use, build = patched
    use(0, 2)
    load(build, is_spmd=False, cc_enabled=False)
    assert calls["load"][-1]["cc"] is False


def test_mpmd_without_a_process_group(patched):
    calls, use, build = patched
    use(0, 0)
    k = load(build, is_spmd=False, cc_enabled=True, rank_id=1, world_size=4)
    assert f"{os.sep}rank_1{os.sep}" in k.neff_path
    assert calls["load"][-1] == dict(path=k.neff_path, cc=True, rank=1, world=4)
    DK._LOADED_KERNELS.clear()
    k = load(build, is_spmd=False)                          # no rank known at all: plain build directory
    assert "rank_" not in k.neff_path and calls["load"][-1]["cc"] is False


# ----------------------------------------------------------------------------- no process group
def test_single_process_defaults_to_no_collectives(patched):
    calls, use, build = patched
    use(0, 0)
    load(build)
    assert calls["load"][-1]["cc"] is False and calls["load"][-1]["world"] == 1
    use(0, 1)                                               # a one-rank group counts as not distributed
    DK._LOADED_KERNELS.clear()
    load(build)
    assert calls["load"][-1]["cc"] is False


def test_single_process_explicit_collectives(patched):
    calls, use, build = patched
    use(0, 0)
    load(build, cc_enabled=True, rank_id=0, world_size=2)
    assert calls["load"][-1]["cc"] is True and calls["load"][-1]["world"] == 2


# ----------------------------------------------------------------------------- validation
@pytest.mark.parametrize("kw", [dict(cc_enabled=True), dict(cc_enabled=True, rank_id=0),
                                dict(cc_enabled=True, world_size=2)])
def test_collectives_without_rank_or_world_need_a_group(patched, kw):
    calls, use, build = patched
    use(0, 0)
    with pytest.raises(ValueError, match="rank_id and world_size are required"):
        load(build, **kw)
    assert not calls["load"]


@pytest.mark.parametrize("rank,world", [(4, 4), (-1, 2)])
def test_rank_outside_the_world_is_rejected(patched, rank, world):
    calls, use, build = patched
    use(0, 0)
    with pytest.raises(ValueError, match="outside world"):
        load(build, cc_enabled=True, rank_id=rank, world_size=world)


# ----------------------------------------------------------------------------- caches
def test_in_memory_cache_hit_skips_the_load(patched):
    calls, use, build = patched
    use(0, 2)
    k = load(build)
    again = load(build)
    assert again is k and len(calls["load"]) == 1 and len(calls["compile"]) == 1
    assert list(DK._LOADED_KERNELS.values()) == [k]


def test_on_disk_cache_hit_skips_the_compile(patched):
    calls, use, build = patched
    use(0, 0)
    load(build)
    DK._LOADED_KERNELS.clear()
    load(build)
    assert len(calls["compile"]) == 1 and len(calls["load"]) == 2


def test_cache_disabled_recompiles_reloads_and_stores_nothing(patched):
    calls, use, build = patched
    use(0, 0)
    a = load(build, use_cached_if_exists=False)
    b = load(build, use_cached_if_exists=False)
    assert a is not b and len(calls["compile"]) == 2 and len(calls["load"]) == 2
    assert not DK._LOADED_KERNELS


def test_compiler_arguments_are_part_of_the_key(patched):
    calls, use, build = patched
    use(0, 0)
    a = load(build)
    b = load(build, additional_compiler_args="-O2")
    assert a is not b and len(calls["compile"]) == 2 and len(DK._LOADED_KERNELS) == 2


def test_shapes_are_part_of_the_key(patched):
    calls, use, build = patched
    use(0, 0)
    load(build)
    DK.DeviceKernel.compile_and_load(kern, np.ones((2, 8), np.float32), B, name="mm", build_dir=build)
    assert len(calls["compile"]) == 2


def test_mpmd_ranks_do_not_share_artifacts(patched):
    calls, use, build = patched
    use(0, 2)
    k0 = load(build, is_spmd=False)
    DK._LOADED_KERNELS.clear()
    use(1, 2)
    k1 = load(build, is_spmd=False)
    assert k0.neff_path != k1.neff_path and len(calls["compile"]) == 2


def test_device_tensor_arguments_are_traced_by_shape_and_dtype(patched):
    calls, use, build = patched
    use(0, 0)

    class Ref:                      # what a device tensor looks like to the tracer: shape, dtype, a handle
        def __init__(self, shape, dtype):
            self.shape, self.dtype, self.tensor_ref = shape, np.dtype(dtype), object()

    k_np = load(build)
    DK._LOADED_KERNELS.clear()
    k_dev = DK.DeviceKernel.compile_and_load(kern, Ref((4, 8), np.float32), Ref((8, 4), np.float32), name="mm",
                                             build_dir=build)
    assert k_dev.neff_path == k_np.neff_path and len(calls["compile"]) == 1
