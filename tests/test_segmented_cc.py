"""Traced kernels with collectives: the graph is cut at the collectives, compute pieces run through the
interpreter (CPU ranks, gloo) or as device modules (GPU ranks, NCCL), collectives through torch.distributed."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def make_kernel(world):
    from nkipy_b200.distributed import collectives as cc

    groups = [list(range(world))]

    def kernel(x, w):
        y = cc.all_reduce(x @ w, groups)                         # row-parallel matmul
        z = np.tanh(y) * 0.5
        g = cc.all_gather(z[:, :4], 1, groups)                    # gather a slice along columns
        r = cc.reduce_scatter(z, 0, groups)                       # rows scattered, summed
        t = cc.all_to_all(z, 0, 1, groups)
        return g, r + 1.0, t

    return kernel


def expected(xs, ws, rank):
    world = len(xs)
    y = sum(x @ w for x, w in zip(xs, ws))
    z = np.tanh(y) * 0.5
    g = np.concatenate([z[:, :4]] * world, axis=1)
    rows = z.shape[0] // world
    r = world * z[rank * rows:(rank + 1) * rows] + 1.0
    parts = np.split(z, world, axis=0)
    t = np.concatenate([parts[rank]] * world, axis=1)
    return g, r, t


def _data(rank):
    rng = np.random.default_rng(10 + rank)
    return rng.standard_normal((8, 16)).astype(np.float32), (rng.standard_normal((16, 12)) * 0.2).astype(np.float32)


def test_split_structure_and_single_rank():
    from nkipy_b200.runtime.segmented import Segment, SegmentedKernel

    k = SegmentedKernel.compile(make_kernel(1), *_data(0), backend="interp")
    assert k.num_collectives == 4 and k.num_segments >= 3
    assert isinstance(k.steps[0], Segment)
    got = k(*_data(0))
    for a, b in zip(got, expected([_data(0)[0]], [_data(0)[1]], 0)):
        np.testing.assert_allclose(a, b, rtol=1e-5, atol=1e-5)


def _worker(rank, world, port, q, backend):
    sys.path.insert(0, ROOT)
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    from nkipy_b200.runtime.segmented import SegmentedKernel

    if backend == "device":
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(f"cuda:{rank}"))
        from nkipy_b200.spike import spike_singleton

        spike_singleton.configure(device_ordinal=rank)
    else:
        dist.init_process_group("gloo", rank=rank, world_size=world)
    x, w = _data(rank)
    k = SegmentedKernel.compile(make_kernel(world), x, w, backend=backend,
                                build_dir=None if backend == "interp" else f"/tmp/seg_cc_rank{rank}")
    got = k(x, w)
    xs, ws = zip(*[_data(r) for r in range(world)])
    errs = [float(np.abs(np.asarray(a, dtype=np.float64) - b).max()) for a, b in zip(got, expected(xs, ws, rank))]
    q.put((rank, errs))
    dist.barrier()
    dist.destroy_process_group()


def _launch(backend, tol):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q, backend)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=240) for _ in range(2)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, errs in res:
        assert max(errs) < tol, (rank, errs)


def test_two_cpu_ranks_gloo():
    _launch("interp", 1e-5)


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_two_gpu_ranks_nccl():
    _launch("device", 1e-3)


@pytest.mark.gpu
def test_single_gpu_segments():
    from nkipy_b200.runtime.segmented import SegmentedKernel

    x, w = _data(0)
    k = SegmentedKernel.compile(make_kernel(1), x, w, backend="device")
    got = k(x, w)
    for a, b in zip(got, expected([x], [w], 0)):
        np.testing.assert_allclose(a, b, rtol=1e-3, atol=1e-3)
