"""Data-parallel replica groups and the pipeline-stage wrapper on CPU ranks (gloo)."""
import os
import socket
import sys

import torch
import torch.multiprocessing as mp

from nkipy_b200.parallel.groups import PipelineStage, replica_groups

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def test_replica_groups_and_partition():
    assert replica_groups(8, 2) == [[0, 1], [2, 3], [4, 5], [6, 7]]
    assert PipelineStage.partition(10, 4) == [(0, 3), (3, 6), (6, 8), (8, 10)]


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    import torch.distributed as dist

    from nkipy_b200.parallel.groups import PipelineStage, make_replica_group

    tp, replica, n_rep = make_replica_group(2, backend="gloo")
    # each replica sums only over its own two ranks
    t = torch.full((3,), float(rank))
    tp.all_reduce(t)
    expect = float(sum(range(replica * 2, replica * 2 + 2)))
    ok_dp = (t == expect).all().item() and n_rep == 2 and tp.world_size == 2 and tp.rank == rank % 2
    # pipeline of 4 stages over the world: stage s applies x -> 2 x + s to three micro-batches
    weights = [(2.0, float(s)) for s in range(world)]
    stage = PipelineStage([lambda x, a=weights[rank][0], b=weights[rank][1]: a * x + b], rank, world)
    outs = []
    for mb in range(3):
        x0 = torch.full((4,), float(mb)) if rank == 0 else None
        y = stage.forward(x0, shape=(4,), dtype=torch.float32, device="cpu")
        if y is not None:
            outs.append(y[0].item())
    stage.drain()
    q.put((rank, ok_dp, outs))
    dist.barrier()
    dist.destroy_process_group()


def test_dp_groups_and_pipeline_over_gloo():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 4, port, q)) for r in range(4)]
    for p in procs:
        p.start()
    res = {r[0]: r for r in (q.get(timeout=120) for _ in range(4))}
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0

    def ref(x):
        for s in range(4):
            x = 2.0 * x + s
        return x

    assert all(res[r][1] for r in range(4))
    assert res[3][2] == [ref(0.0), ref(1.0), ref(2.0)]
    assert res[0][2] == []
