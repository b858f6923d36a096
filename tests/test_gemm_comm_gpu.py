"""GEMM fused with reduce-scatter / all-gather over peer memory (csrc/kernels/gemm_comm.cu).

One-rank cases run in this process (staging, counters and the reducer are exercised with tp = 1);
the two-rank cases run as child processes on 2 GPUs and compare against NCCL + fp32 matmul."""
import os
import socket
import sys

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-6)).item()


@pytest.mark.parametrize("m,n,k", [(256, 512, 256), (384, 256, 192), (100, 136, 64), (1024, 1024, 512)])
def test_gemm_rs_single_rank(m, n, k):
    from nkipy_b200 import ops
    from nkipy_b200.parallel.comm import TPGroup
    from nkipy_b200.parallel.symm import GemmReduceScatter

    dev = torch.device("cuda:0")
    tp = TPGroup.single(dev)
    op = GemmReduceScatter(tp, m, n)
    torch.manual_seed(0)
    for it in range(3):       # three calls: both buffers and the growing counters
        x = torch.randn(m, k, device=dev).to(torch.bfloat16)
        w = (torch.randn(n, k, device=dev) * 0.1).to(torch.bfloat16)
        out = op(x, w)
        ref = x.float() @ w.float().T
        assert _rel(out, ref) < 1e-2, (it, _rel(out, ref))
    assert ops.device_status() == 0
    op.close()


@pytest.mark.parametrize("m,n,k", [(256, 512, 256), (100, 136, 64), (1024, 768, 512)])
def test_ag_gemm_single_rank(m, n, k):
    from nkipy_b200 import ops
    from nkipy_b200.parallel.comm import TPGroup
    from nkipy_b200.parallel.symm import AllGatherGemm

    dev = torch.device("cuda:0")
    tp = TPGroup.single(dev)
    op = AllGatherGemm(tp, m, k)
    torch.manual_seed(1)
    for it in range(3):
        x = torch.randn(m, k, device=dev).to(torch.bfloat16)
        w = (torch.randn(n, k, device=dev) * 0.1).to(torch.bfloat16)
        out = op(x, w)
        ref = x.float() @ w.float().T
        assert _rel(out, ref) < 1e-2, (it, _rel(out, ref))
    assert ops.device_status() == 0
    op.close()


@pytest.mark.parametrize("m,i,k", [(1024, 384, 512), (512, 200, 256)])
def test_ag_gemm_gated_single_rank(m, i, k):
    from nkipy_b200 import ops
    from nkipy_b200.parallel.comm import TPGroup
    from nkipy_b200.parallel.symm import AllGatherGemm

    dev = torch.device("cuda:0")
    op = AllGatherGemm(TPGroup.single(dev), m, k)
    torch.manual_seed(2)
    x = torch.randn(m, k, device=dev).to(torch.bfloat16)
    w = (torch.randn(2 * i, k, device=dev) * 0.1).to(torch.bfloat16)
    out = op(x, w, gated=True)
    ref = torch.nn.functional.silu(x.float() @ w[:i].float().T) * (x.float() @ w[i:].float().T)
    assert out.shape == (m, i) and _rel(out, ref) < 1e-2
    assert ops.device_status() == 0
    op.close()


def _worker(rank, world, port, q):
    try:
        _worker_body(rank, world, port, q)
    except BaseException:       # make a failing rank visible instead of letting its peer wait for it
        import traceback

        q.put((rank, float("inf"), -1, {"exception": traceback.format_exc()[-1500:]}))
        raise


def _worker_body(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    from nkipy_b200 import ops
    from nkipy_b200.parallel.comm import TPGroup
    from nkipy_b200.parallel.symm import AllGatherGemm, GemmReduceScatter

    tp = TPGroup.from_env()
    dev = tp.device
    g = torch.Generator(device=dev).manual_seed(7 + rank)
    errs = {}
    for (m, n, k) in [(512, 512, 256), (192, 264, 128), (2048, 1024, 512)]:
        # row-parallel: x, w hold this rank's K shard
        rs = GemmReduceScatter(tp, m, n)
        for it in range(3):
            x = torch.randn(m, k, device=dev, generator=g).to(torch.bfloat16)
            w = (torch.randn(n, k, device=dev, generator=g) * 0.1).to(torch.bfloat16)
            out = rs(x, w)
            full = x.float() @ w.float().T
            dist.all_reduce(full)
            ref = full[rank * (m // world):(rank + 1) * (m // world)]
            errs[("rs", m, n, k, it)] = _rel(out, ref)
        torch.cuda.synchronize()
        tp.barrier()
        rs.close()
        # column-parallel: x_local is this rank's row slab, w this rank's column shard
        ag = AllGatherGemm(tp, m, k, comm_ctas=8)
        for it in range(3):
            xl = torch.randn(m // world, k, device=dev, generator=g).to(torch.bfloat16)
            w = (torch.randn(n, k, device=dev, generator=g) * 0.1).to(torch.bfloat16)
            out = ag(xl, w)
            xs = [torch.empty_like(xl) for _ in range(world)]
            dist.all_gather(xs, xl)
            ref = torch.cat(xs).float() @ w.float().T
            errs[("ag", m, n, k, it)] = _rel(out, ref)
            if n // 2 >= 128:
                out = ag(xl, w, gated=True)                  # w read as [gate; up]
                full = torch.cat(xs).float()
                h = n // 2
                ref = torch.nn.functional.silu(full @ w[:h].float().T) * (full @ w[h:].float().T)
                errs[("ag-gated", m, n, k, it)] = _rel(out, ref)
        torch.cuda.synchronize()
        tp.barrier()
        ag.close()
    status = ops.device_status()
    tp.barrier()
    q.put((rank, max(errs.values()), status, {str(k): v for k, v in errs.items() if v > 1e-2}))
    dist.destroy_process_group()


def _worlds():
    n = torch.cuda.device_count()
    return [w for w in (2, 4, 8) if w <= n] or [2]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("world", _worlds())
def test_gemm_comm_ranks(world):
    """Every rank count the box offers: the peer rotation, the per-rank counter stride and the slab ownership
    all depend on it."""
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
    for rank, err, status, bad in res:
        assert status == 0, (rank, status)
        assert err < 1e-2, (rank, err, bad)
