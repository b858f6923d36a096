"""Host side of the symmetric-memory bootstrap, without a GPU: file descriptors travel between rank
processes over Unix sockets (gloo ranks on CPU), in the all-to-all form used for the per-rank allocation
handles and in the one-to-all form used for the multicast object's handle."""
import os
import socket
import sys

import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    import torch.distributed as dist

    from nkipy_b200.parallel.comm import TPGroup
    from nkipy_b200.parallel.symm import exchange_fds

    tp = TPGroup.from_env(backend="gloo")
    # every rank owns a pipe; the write ends are exchanged, each peer writes its rank into every pipe it got
    r_end, w_end = os.pipe()
    got = exchange_fds(tp, w_end)
    assert got[rank] is None and all(g is not None for i, g in enumerate(got) if i != rank)
    for i, fd in enumerate(got):
        if fd is not None:
            os.write(fd, bytes([rank]))
            os.close(fd)
    tp.barrier()
    os.close(w_end)
    seen = sorted(os.read(r_end, 64))
    os.close(r_end)
    # one-to-all: rank 1 shares one descriptor, everybody else reads what rank 1 wrote through its own end
    r2, w2 = os.pipe()
    got2 = exchange_fds(tp, r2 if rank == 1 else -1, only_from=1)
    text = None
    if rank == 1:
        for _ in range(world - 1):
            os.write(w2, b"x")
        assert all(g is None for g in got2)
    else:
        assert got2[1] is not None and sum(g is not None for g in got2) == 1
        text = os.read(got2[1], 1)
        os.close(got2[1])
    tp.barrier()
    os.close(r2)
    os.close(w2)
    q.put((rank, seen, text))
    dist.destroy_process_group()


def test_descriptor_exchange_three_ranks():
    world = 3
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, seen, text in res:
        assert seen == [r for r in range(world) if r != rank]
        assert text == (None if rank == 1 else b"x")
