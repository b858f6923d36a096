"""Failure detection: every failure is made on the host (a rank that sleeps, skips its signal or leaves
between steps); on the GPU only a bounded wait on a flag that nothing sets is exercised."""
import os
import socket
import sys
import time

import pytest
import torch
import torch.multiprocessing as mp

from nkipy_b200.parallel.health import (CommTimeoutError, CounterProtocolSim, FaultPlan, Heartbeat,
                                        InjectedRankExit, Watchdog)

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def test_fault_plan_parsing_and_hooks():
    plan = FaultPlan.from_env("drop_flag:1:3, delay_ms:0:20:2,kill_rank:2:5")
    assert plan.drops_signal(1, 3) and not plan.drops_signal(1, 2) and not plan.drops_signal(0, 3)
    t0 = time.monotonic()
    plan.before_step(0, 2)
    assert time.monotonic() - t0 >= 0.018
    plan.before_step(2, 4)
    with pytest.raises(InjectedRankExit):
        plan.before_step(2, 5)
    with pytest.raises(ValueError):
        FaultPlan.from_env("explode:1")
    assert FaultPlan.from_env("").kill_rank == {}


def test_watchdog_fires_once_per_overrun():
    fired = []
    wd = Watchdog(on_timeout=lambda name, t: fired.append((name, t)), poll_s=0.005)
    with wd.step("fast", 0.5):
        time.sleep(0.01)
    with wd.step("slow", 0.03):
        time.sleep(0.12)
    wd.close()
    assert [n for n, _ in fired] == ["slow"] and wd.timeouts == ["slow"]


def test_counter_protocol_model():
    sim = CounterProtocolSim(3)
    out = sim.run(6)
    assert not sim.violations
    for r in range(3):
        assert out[r] == [sum(s + 1 + op for s in range(3)) for op in range(6)]
    # a rank that skips one signal: its peers (and it) run into the bounded wait, nobody reads stale data
    sim = CounterProtocolSim(3, wait_limit_s=0.1)
    out = sim.run(4, drop=(1, 2))
    assert not sim.violations
    assert all(o == "timeout" or len(o) <= 3 for o in out) and "timeout" in out


def _hb_worker(rank, port, leave_after, q):
    from torch.distributed import TCPStore

    store = TCPStore("127.0.0.1", port, 2, is_master=(rank == 0), timeout=__import__("datetime").timedelta(seconds=30))
    hb = Heartbeat(store, rank, 2, interval_s=0.05)
    if rank == 1:
        time.sleep(leave_after)
        hb.stop()                       # leaves between steps: no beat any more
        time.sleep(1.0)
        return
    seen_alive = False
    t0 = time.time()
    while time.time() - t0 < 5.0:
        dead = hb.dead_ranks(timeout_s=0.3)
        if not dead:
            seen_alive = True
        elif seen_alive:
            q.put(("dead", dead, time.time() - t0))
            return
        time.sleep(0.05)
    q.put(("never", [], 5.0))


def test_heartbeat_detects_a_rank_that_left():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_hb_worker, args=(r, port, 0.5, q)) for r in range(2)]
    for p in procs:
        p.start()
    kind, dead, t = q.get(timeout=30)
    for p in procs:
        p.join(timeout=30)
    assert kind == "dead" and dead == [1] and t < 3.0


@pytest.mark.gpu
def test_bounded_wait_reports_and_context_survives():
    """A consumer kernel waits for an arrival counter that nothing increments: after its one-second limit
    it records a status instead of hanging, the host turns that into an exception, and the context still
    runs kernels afterwards."""
    import ctypes

    from nkipy_b200 import ops
    from nkipy_b200.ops import _lib
    from nkipy_b200.parallel.health import check_device_status

    dev = torch.device("cuda:0")
    lib = _lib.lib()
    _lib.ensure_init()
    P, I = ctypes.c_void_p, ctypes.c_int
    lib.nkb_tp_reduce_rmsnorm.restype = I
    lib.nkb_tp_reduce_rmsnorm.argtypes = [P, I, P, I, P, P, P, P, P, P, I, I, ctypes.c_float, P]
    rows, hidden = 4, 256
    partials = torch.zeros((2, rows, hidden), dtype=torch.bfloat16, device=dev)
    flags = torch.zeros((2,), dtype=torch.int32, device=dev)          # never incremented
    seen = torch.zeros((1,), dtype=torch.int32, device=dev)
    done = torch.zeros((1,), dtype=torch.int32, device=dev)
    out = torch.zeros((rows, hidden), dtype=torch.bfloat16, device=dev)
    assert ops.device_status() == 0
    t0 = time.time()
    rc = lib.nkb_tp_reduce_rmsnorm(partials.data_ptr(), 2, flags.data_ptr(), 2, seen.data_ptr(), done.data_ptr(), None,
                                   None, out.data_ptr(), None, rows, hidden, 1e-5,
                                   torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert 0.9 < time.time() - t0 < 5.0
    with pytest.raises(CommTimeoutError) as e:
        check_device_status()
    assert e.value.code == 5
    assert int(seen.item()) == 0                                        # the failed use was not counted
    # the context is intact
    x = torch.randn(8, 256, device=dev).to(torch.bfloat16)
    w = torch.ones(256, device=dev, dtype=torch.bfloat16)
    y = ops.rmsnorm(x, w, 1e-5)
    torch.cuda.synchronize()
    assert torch.isfinite(y.float()).all() and ops.device_status() == 0


def _leave_worker(rank, world, port, hb_port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0", NKIPY_B200_FUSED_TP="0")
    import datetime

    from torch.distributed import TCPStore

    from nkipy_b200.parallel.comm import TPGroup

    tp = TPGroup.from_env(timeout_s=20)
    store = TCPStore("127.0.0.1", hb_port, world, is_master=(rank == 0), timeout=datetime.timedelta(seconds=30))
    hb = Heartbeat(store, rank, world, interval_s=0.05)
    plan = FaultPlan.from_env("kill_rank:1:3")
    x = torch.ones(1024, device=tp.device)
    steps_done = 0
    try:
        for step in range(6):
            plan.before_step(rank, step)                       # rank 1 leaves before step 3, nothing in flight
            time.sleep(1.0)                                    # host work between steps, well above the time-out
            dead = hb.dead_ranks(timeout_s=0.3)                # and the leaving rank announces itself in stop()
            if dead:                                           # learnt on the host, before the next launch
                q.put((rank, "peer-left", dead, steps_done))
                return
            tp.all_reduce(x)
            torch.cuda.synchronize()
            steps_done += 1
        q.put((rank, "finished", [], steps_done))
    except InjectedRankExit:
        torch.cuda.synchronize()
        hb.stop()
        q.put((rank, "left", [], steps_done))
        time.sleep(2.0)


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_rank_leaves_between_steps_and_peer_notices():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port, hb_port = _free_port(), _free_port()
    procs = [ctx.Process(target=_leave_worker, args=(r, 2, port, hb_port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict()
    for _ in range(2):
        r = q.get(timeout=120)
        res[r[0]] = r
    for p in procs:
        p.join(timeout=60)
    assert res[1][1] == "left" and res[1][3] == 3
    assert res[0][1] == "peer-left" and res[0][2] == [1] and res[0][3] == 3


# ----------------------------------------------------------------------------- recovery
def _recover_worker(role, rank, world, ports, hb_port, q, use_gpu):
    """role "first": a member of the original group (rank 1 leaves before step 2).  role "replacement": a new
    process that takes the lost rank's place.  After recovery both run one more reduced step and report it."""
    sys.path.insert(0, ROOT)
    os.environ.update(LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0", NKIPY_B200_NVLS="0")
    import datetime

    import torch.distributed as dist
    from torch.distributed import TCPStore

    from nkipy_b200.parallel.comm import TPGroup
    from nkipy_b200.parallel.health import recover

    hidden, rows = 256, 8

    def fused_step(tp, seed):
        """One row-parallel GEMM + all-reduce + residual + RMSNorm through FusedTP against an fp32 oracle."""
        from nkipy_b200 import ops

        g = torch.Generator(device="cpu").manual_seed(seed)
        x_full = torch.randn(rows, hidden * world, generator=g).to(torch.bfloat16)
        w_full = (torch.randn(hidden, hidden * world, generator=g) * 0.05).to(torch.bfloat16)
        resid = torch.randn(rows, hidden, generator=g).to(torch.bfloat16)
        norm = torch.ones(hidden).to(torch.bfloat16)
        sl = slice(tp.rank * hidden, (tp.rank + 1) * hidden)
        dev = tp.device
        tp.fused.begin_step()
        outs = [tp.fused.gemm_allreduce_add_rmsnorm(x_full[:, sl].contiguous().to(dev), w_full[:, sl].contiguous().to(dev),
                                                    resid.to(dev), norm.to(dev), None, 1e-5) for _ in range(2)]
        torch.cuda.synchronize()
        assert ops.device_status() == 0
        h = x_full.float() @ w_full.float().T + resid.float()
        want = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + 1e-5)
        got = outs[1][1].float().cpu()
        return float((got - want).norm() / want.norm())

    def plain_step(tp):
        x = torch.full((4,), float(tp.rank + 1), device=tp.device)
        tp.all_reduce(x)
        return float(x[0])

    if role == "first":
        os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(ports[0]))
        tp = TPGroup.from_env(backend="nccl" if use_gpu else "gloo", timeout_s=20)
        if use_gpu:
            from nkipy_b200.parallel.symm import FusedTP

            tp.fused = FusedTP(tp, rows, hidden)
        store = TCPStore("127.0.0.1", hb_port, world + 1, is_master=(rank == 0),
                         timeout=datetime.timedelta(seconds=60), wait_for_workers=False)
        hb = Heartbeat(store, rank, world, interval_s=0.05)
        plan = FaultPlan.from_env("kill_rank:1:2")
        try:
            for step in range(4):
                plan.before_step(rank, step)                  # rank 1 leaves before step 2, nothing in flight
                time.sleep(0.4)
                if hb.dead_ranks(timeout_s=0.3):
                    break
                fused_step(tp, step) if use_gpu else plain_step(tp)
        except InjectedRankExit:
            if use_gpu:
                torch.cuda.synchronize()
                tp.fused.abandon()                            # between steps: no kernel addresses this rank now
            hb.stop()
            q.put(("left", rank, step))
            time.sleep(1.0)
            return
        dead = hb.dead_ranks(timeout_s=0.3)
        hb.stop()
        q.put(("detected", rank, dead))
        rec = recover(tp, rank=rank, world_size=world, master_port=ports[1], generation=1, timeout_s=60,
                      backend="nccl" if use_gpu else "gloo")
    else:
        rec = recover(None, rank=rank, world_size=world, master_port=ports[1], generation=1, timeout_s=60,
                      backend="nccl" if use_gpu else "gloo",
                      fused_args=dict(max_tokens=rows, hidden=hidden) if use_gpu else None)
    tp = rec.tp
    assert tp.world_size == world and rec.generation == 1
    if use_gpu:
        assert tp.fused is not None and tp.fused.ops_issued == 0
        val = max(fused_step(tp, 100 + s) for s in range(2))
    else:
        val = plain_step(tp)
    tp.barrier()
    q.put(("recovered", rank, val, round(rec.seconds, 2)))
    if use_gpu:
        tp.fused.close()
    dist.destroy_process_group()


def _run_recovery(use_gpu):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ports, hb_port = (_free_port(), _free_port()), _free_port()
    procs = [ctx.Process(target=_recover_worker, args=("first", r, 2, ports, hb_port, q, use_gpu)) for r in range(2)]
    for p in procs:
        p.start()
    events, replacement = [], None
    try:
        while sum(e[0] == "recovered" for e in events) < 2:
            e = q.get(timeout=180)
            events.append(e)
            if e[0] == "left" and replacement is None:
                replacement = ctx.Process(target=_recover_worker, args=("replacement", 1, 2, ports, hb_port, q, use_gpu))
                replacement.start()
    finally:
        for p in procs + ([replacement] if replacement else []):
            p.join(timeout=90)
            if p.is_alive():
                p.kill()
    kinds = [e[0] for e in events]
    assert kinds.count("left") == 1 and ("detected", 0, [1]) in events
    return {e[1]: e for e in events if e[0] == "recovered"}


def test_recover_rebuilds_the_group_with_a_replacement_rank_gloo():
    rec = _run_recovery(use_gpu=False)
    assert set(rec) == {0, 1} and all(e[2] == 3.0 for e in rec.values())       # 1 + 2 over the new group


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_recover_rebuilds_fused_tp_after_a_rank_left():
    """A rank leaves between steps (NVLS and multimem off), the survivor learns of it from the heartbeat,
    abandons its symmetric buffers and its NCCL group, a replacement process joins, and a fused GEMM +
    all-reduce + RMSNorm step is right again on both."""
    rec = _run_recovery(use_gpu=True)
    assert set(rec) == {0, 1} and all(e[2] < 2e-2 for e in rec.values()), rec


def test_departure_is_announced_and_seen_at_once():
    """A rank that stops its heartbeat writes an explicit key; its peer lists it as gone without waiting for the
    beat to age, and a rank that merely beats late is not listed before the time-out."""
    class DictStore:
        def __init__(self):
            self.d = {}

        def set(self, k, v):
            self.d[k] = v

        def get(self, k):
            return self.d[k]

    store = DictStore()
    a = Heartbeat(store, 0, 2, interval_s=0.02)
    b = Heartbeat(store, 1, 2, interval_s=0.02)
    try:
        assert a.dead_ranks(timeout_s=5.0) == []
        assert not a.has_left(1)
        b.stop()
        assert a.has_left(1)
        assert a.dead_ranks(timeout_s=5.0) == [1]            # far inside the time-out
        assert b.dead_ranks(timeout_s=5.0) == []             # rank 0 still beats
    finally:
        a.stop()
