"""Fused GEMM + all-reduce + RMSNorm over peer memory, 2 ranks on 2 GPUs (child processes)."""
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


# how the symmetric buffers are made: CUDA IPC, virtual memory management with file-descriptor handles, and
# the latter bound to an NVLink multicast object (multimem stores in the push epilogue)
MODES = {"ipc": dict(NKIPY_B200_SYMM="ipc", NKIPY_B200_NVLS="0", NKIPY_B200_PRESUM_MIN_SPLITS="2", NKIPY_B200_PRESUM_MIN_WORLD="1"),
         "vmm": dict(NKIPY_B200_SYMM="vmm", NKIPY_B200_NVLS="0", NKIPY_B200_PRESUM_MIN_SPLITS="2", NKIPY_B200_PRESUM_MIN_WORLD="1"),
         "nvls": dict(NKIPY_B200_SYMM="vmm", NKIPY_B200_NVLS="1", NKIPY_B200_PRESUM_MIN_SPLITS="2", NKIPY_B200_PRESUM_MIN_WORLD="1"),
         # the older exchange: the GEMM epilogue pushes one partial per split (default is the pre-summing kernel)
         "vmm-push": dict(NKIPY_B200_SYMM="vmm", NKIPY_B200_NVLS="0", NKIPY_B200_TP_EXCHANGE="push"),
         "nvls-push": dict(NKIPY_B200_SYMM="vmm", NKIPY_B200_NVLS="1", NKIPY_B200_TP_EXCHANGE="push")}


def _worker(rank, world, port, q, mode="ipc"):
    sys.path.insert(0, ROOT)
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0", **MODES[mode])
    import torch.distributed as dist

    from nkipy_b200 import ops
    from nkipy_b200.parallel.comm import TPGroup
    from nkipy_b200.parallel.symm import FusedTP

    tp = TPGroup.from_env()
    dev = tp.device
    M, N, K = 64, 1024, 1536
    fused = FusedTP(tp, M, N)
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    errs = []
    resid = torch.randn(M, N, device=dev, generator=g).to(torch.bfloat16)
    dist.broadcast(resid, 0)
    wn = torch.randn(N, device=dev, generator=g).to(torch.bfloat16)
    dist.broadcast(wn, 0)

    def reference(x, w, r):
        y = x.float() @ w.float().T
        dist.all_reduce(y)
        h = (y + r.float()).to(torch.bfloat16).float()
        n = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + 1e-5) * wn.float()
        return h, n

    xs = [torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16) for _ in range(6)]
    ws = [(torch.randn(N, K, device=dev, generator=g) * 0.05).to(torch.bfloat16) for _ in range(6)]
    fused.begin_step()
    for i in range(6):
        h, n = fused.gemm_allreduce_add_rmsnorm(xs[i], ws[i], resid, wn, None, 1e-5, splits=1 + (i % 3))
        rh, rn = reference(xs[i], ws[i], resid)
        errs.append(((h.float() - rh).norm() / rh.norm()).item())
        errs.append(((n.float() - rn).norm() / rn.norm()).item())
    # the same sequence captured in a CUDA graph and replayed: counters must keep working
    torch.cuda.synchronize()
    tp.barrier()
    outs = []

    def body():
        fused.begin_step()
        outs.clear()
        for i in range(6):
            outs.append(fused.gemm_allreduce_add_rmsnorm(xs[i], ws[i], resid, wn, None, 1e-5, splits=2))

    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        body()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        body()
    for _ in range(5):
        graph.replay()
    torch.cuda.synchronize()
    for i in range(6):
        rh, rn = reference(xs[i], ws[i], resid)
        errs.append(((outs[i][0].float() - rh).norm() / rh.norm()).item())
    status = ops.device_status()
    tp.barrier()
    used = (fused.mem.backend, bool(fused.mem.mc_ptr))
    fused.close()
    q.put((rank, max(errs), status, used))
    dist.destroy_process_group()


def _worlds():
    n = torch.cuda.device_count()
    return [w for w in (2, 4, 8) if w <= n] or [2]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("mode", ["ipc", "vmm", "nvls", "vmm-push", "nvls-push"])
@pytest.mark.parametrize("world", _worlds())
def test_fused_gemm_allreduce_ranks(world, mode):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q, mode)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=240) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err, status, used in res:
        assert status == 0, (rank, status)
        assert err < 2e-2, (rank, err)
        if mode == "ipc":
            assert used == ("ipc", False)
        elif mode == "vmm":
            assert used[1] is False


def test_fused_gemm_allreduce_single_rank():
    """The push epilogue, the arrival counters and the consumer with this GPU as the only peer (eager calls and
    graph replays), including the argmax exchange used by the vocabulary-parallel head."""
    from nkipy_b200 import ops
    from nkipy_b200.parallel.comm import TPGroup
    from nkipy_b200.parallel.symm import FusedTP

    dev = torch.device("cuda:0")
    M, N, K = 48, 1024, 1536
    fused = FusedTP(TPGroup.single(dev), 64, N)
    g = torch.Generator(device=dev).manual_seed(5)
    resid = torch.randn(M, N, device=dev, generator=g).to(torch.bfloat16)
    wn = torch.randn(N, device=dev, generator=g).to(torch.bfloat16)
    xs = [torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16) for _ in range(4)]
    ws = [(torch.randn(N, K, device=dev, generator=g) * 0.05).to(torch.bfloat16) for _ in range(4)]

    def reference(x, w):
        h = (x.float() @ w.float().T + resid.float()).to(torch.bfloat16).float()
        return h, h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + 1e-5) * wn.float()

    outs = []

    def body():
        fused.begin_step()
        outs.clear()
        for i in range(4):
            outs.append(fused.gemm_allreduce_add_rmsnorm(xs[i], ws[i], resid, wn, None, 1e-5, splits=1 + i % 3))

    body()
    torch.cuda.synchronize()
    for i in range(4):
        rh, rn = reference(xs[i], ws[i])
        assert ((outs[i][0].float() - rh).norm() / rh.norm()).item() < 2e-2
        assert ((outs[i][1].float() - rn).norm() / rn.norm()).item() < 2e-2
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        body()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        body()
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    for i in range(4):
        rh, _ = reference(xs[i], ws[i])
        assert ((outs[i][0].float() - rh).norm() / rh.norm()).item() < 2e-2
    vals = torch.randn(M, device=dev, generator=g)
    ids = torch.randint(0, 1000, (M,), device=dev, generator=g, dtype=torch.int32)
    got = fused.argmax_exchange(vals, ids, 7)
    torch.cuda.synchronize()
    assert torch.equal(got, ids + 7)
    assert ops.device_status() == 0
    fused.close()


@pytest.mark.parametrize("N", [1024, 8192])
def test_presum_exchange_single_rank_matches_fp32(N):
    """The pre-summing exchange on one rank (the only peer is this GPU): split-K partials -> sum -> slot ->
    sum over ranks -> residual -> RMSNorm, against fp32; mixed with the push protocol on the same buffers."""
    sys.path.insert(0, ROOT)
    from nkipy_b200 import ops
    from nkipy_b200.parallel.comm import TPGroup
    from nkipy_b200.parallel.symm import FusedTP

    dev = torch.device("cuda:0")
    tp = TPGroup.single(dev)
    M, K = 64, 1536
    fused = FusedTP(tp, M, N)
    try:
        g = torch.Generator(device=dev).manual_seed(5)
        resid = torch.randn(M, N, device=dev, generator=g).to(torch.bfloat16)
        wn = (1 + 0.1 * torch.randn(N, device=dev, generator=g)).to(torch.bfloat16)
        for i in range(6):
            x = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
            w = (torch.randn(N, K, device=dev, generator=g) * 0.05).to(torch.bfloat16)
            fused.exchange = "presum" if i % 3 else "push"          # both protocols share the two buffers
            fused.presum_min_splits, fused.presum_min_world = 2, 1
            if i % 2 == 0:
                fused.begin_step()
            h, nrm = fused.gemm_allreduce_add_rmsnorm(x, w, resid, wn, None, 1e-5, splits=1 + i)
            rh = (x.float() @ w.float().T + resid.float()).to(torch.bfloat16).float()
            rn = rh * torch.rsqrt(rh.pow(2).mean(-1, keepdim=True) + 1e-5) * wn.float()
            assert ((h.float() - rh).norm() / rh.norm()).item() < 1e-2
            assert ((nrm.float() - rn).norm() / rn.norm()).item() < 1e-2
        # a bf16 result (no split-K) goes through the same exchange
        y = torch.randn(M, N, device=dev, generator=g).to(torch.bfloat16)
        fused.begin_step()
        h, _ = fused.exchange_add_rmsnorm(y, resid, wn, 1e-5)
        fused.exchange_add_rmsnorm(y, resid, wn, 1e-5)
        assert ((h.float() - (y.float() + resid.float())).norm() / h.float().norm()).item() < 1e-2
        torch.cuda.synchronize()
        assert ops.device_status() == 0
    finally:
        fused.close()
