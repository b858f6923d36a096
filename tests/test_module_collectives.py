"""Collectives inside ONE loaded module: the code generator lowers all_reduce / all_gather / reduce_scatter /
all_to_all to kernels of the module that exchange over a symmetric workspace (peer stores, arrival counters,
bounded waits); the C++ runtime hands them the peer table.  The kernel and the expected values are the ones
of tests/test_segmented_cc.py, which runs the same graph cut into pieces with torch.distributed between them."""
import json
import os
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "tests"))

from test_segmented_cc import _data, _free_port, expected, make_kernel  # noqa: E402


def test_codegen_emits_collective_kernels_and_a_workspace_plan():
    from nkipy_b200.compiler.codegen import generate
    from nkipy_b200.core.compile import trace

    x, w = _data(0)
    prog = generate(trace(make_kernel(2)).specialize(x, w))
    plan = json.loads(prog.plan_json())
    kinds = [l["kernel"].split("_", 1)[1] for l in plan["launches"]]
    assert kinds.count("cc_push") == 4
    for op in ("cc_all_reduce", "cc_all_gather", "cc_reduce_scatter", "cc_all_to_all"):
        assert op in kinds
    c = plan["collective"]
    # the largest operand is z / the matmul result [8, 12] fp32: two ranks' slots per half
    assert c["world"] == 2 and c["half_bytes"] >= 2 * 8 * 12 * 4 and c["workspace_bytes"] == 256 + 2 * c["half_bytes"]
    assert all(any("cc" in a for a in l["args"]) for l in plan["launches"] if "_cc_" in l["kernel"])
    assert "struct CcTable" in prog.source and "red.release.sys" in prog.source
    # a module without collectives carries no workspace
    plain = json.loads(generate(trace(lambda a, b: a @ b).specialize(x, w)).plan_json())
    assert "collective" not in plain


def test_more_than_eight_ranks_is_rejected():
    from nkipy_b200.compiler.codegen import CodegenError, generate
    from nkipy_b200.core.compile import trace
    from nkipy_b200.distributed import collectives as cc

    k = trace(lambda a: cc.all_reduce(a, [list(range(16))]))
    with pytest.raises(CodegenError, match="up to 8 ranks"):
        generate(k.specialize(np.ones((4, 4), np.float32)))


@pytest.mark.gpu
def test_single_rank_module_runs_its_collectives_locally(tmp_path):
    from nkipy_b200.runtime import DeviceKernel, DeviceTensor

    x, w = _data(0)
    k = DeviceKernel.compile_and_load(make_kernel(1), x, w, name="cc1", build_dir=str(tmp_path))
    assert k.model_ref.has_collectives and k.model_ref.collective_world == 1
    for _ in range(3):                                   # the module's use counter and buffer halves advance
        out = k(inputs={"x": DeviceTensor.from_numpy(x, "x"), "w": DeviceTensor.from_numpy(w, "w")})
        got = [out[n].numpy() for n in k.output_order]
        for a, b in zip(got, expected([x], [w], 0)):
            np.testing.assert_allclose(a, b, rtol=1e-3, atol=1e-3)


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0", NKIPY_B200_NVLS="0")
    import torch.distributed as dist

    from nkipy_b200.parallel.comm import TPGroup
    from nkipy_b200.runtime import DeviceKernel, DeviceTensor
    from nkipy_b200.spike import spike_singleton

    tp = TPGroup.from_env()
    spike_singleton.configure(device_ordinal=rank)
    x, w = _data(rank)
    # SPMD: rank 0 compiles, everyone loads with its rank; the module gets its symmetric workspace at load time
    k = DeviceKernel.compile_and_load(make_kernel(world), x, w, name="ccN", build_dir=f"/tmp/module_cc_{port}")
    assert k.model_ref.is_collective and k.model_ref.collective_world == world
    xs, ws = zip(*[_data(r) for r in range(world)])
    want = expected(xs, ws, rank)
    errs = []
    for _ in range(4):
        out = k(inputs={"x": DeviceTensor.from_numpy(x, "x"), "w": DeviceTensor.from_numpy(w, "w")})
        got = [out[n].numpy() for n in k.output_order]
        errs.append(max(float(np.abs(np.asarray(a, dtype=np.float64) - b).max()) for a, b in zip(got, want)))
    tp.barrier()
    k.unload()
    q.put((rank, errs))
    dist.destroy_process_group()


def _worlds():
    n = torch.cuda.device_count()
    return [w for w in (2, 4) if w <= n] or [2]


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("world", _worlds())
def test_ranks_exchange_inside_the_module(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, errs in res:
        assert max(errs) < 1e-3, (rank, errs)
