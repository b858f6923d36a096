"""Failure detection for the multi-GPU runtime: device wait time-outs, a host watchdog, rank heartbeats,
host-side fault injection and a thread model of the arrival-counter protocol.

The reference has no failure handling: a hung collective simply hangs, and errors of the runtime surface
as typed exceptions with the runtime's status code (spike/src/error.h:24-43, nrt_wrapper.cpp:12-43).
Here every device-side wait is bounded (one second) and reports through a status word; this module turns
that word into exceptions, adds a per-step host deadline and rank liveness, and lets tests provoke the
failure paths from the host only (a rank that sleeps, skips its signal or leaves between steps) — nothing
here makes a GPU fault, trap or spin without bound.

Recovery is a restart of the communication layer, not of the GPU: close the symmetric buffers
(`FusedTP.close`), re-create the process group without the dead rank, reload that rank's weight shards,
rebuild `FusedTP`; KV caches are lost and requests are re-prefilled.
"""

from __future__ import annotations

import dataclasses
import os
import threading
import time
from typing import Callable, Dict, List, Optional

ERR_NAMES = {1: "producer waited for a free shared-memory stage", 2: "MMA warp waited for TMA data",
             3: "MMA warp waited for the epilogue", 4: "epilogue waited for the MMA",
             5: "a peer / producer flag never arrived", 6: "bad argument", 7: "softmax hand-off"}


class CommTimeoutError(RuntimeError):
    """A bounded device-side wait expired; `code` / `detail` decode the status word."""

    def __init__(self, status: int):
        self.status = status
        self.code = status & 0xFF
        self.detail = status >> 8
        super().__init__(f"device wait timed out: {ERR_NAMES.get(self.code, 'unknown')} "
                         f"(code {self.code}, detail 0x{self.detail:x})")


def check_device_status(reset: bool = True) -> None:
    """Raise `CommTimeoutError` if a kernel of the library recorded an expired wait."""
    from .. import ops

    st = ops.device_status(reset=reset) if _accepts_reset(ops.device_status) else ops.device_status()
    if st:
        raise CommTimeoutError(st)


def _accepts_reset(fn) -> bool:
    import inspect

    try:
        return "reset" in inspect.signature(fn).parameters
    except (TypeError, ValueError):
        return False


# ----------------------------------------------------------------------------- watchdog
class Watchdog:
    """Host thread that fires `on_timeout(step_name, elapsed)` when a guarded step overruns its deadline.

        wd = Watchdog(on_timeout=lambda name, t: log.error(...))
        with wd.step("decode", deadline_s=2.0):
            engine.step()
    """

    def __init__(self, on_timeout: Optional[Callable[[str, float], None]] = None, poll_s: float = 0.02):
        self.on_timeout = on_timeout
        self.poll_s = poll_s
        self.timeouts: List[str] = []
        self._lock = threading.Lock()
        self._active: Optional[tuple] = None      # (name, start, deadline, fired)
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def _run(self):
        while not self._stop.wait(self.poll_s):
            with self._lock:
                a = self._active
                if a and not a[3] and time.monotonic() - a[1] > a[2]:
                    self._active = (a[0], a[1], a[2], True)
                    self.timeouts.append(a[0])
                    cb, name, el = self.on_timeout, a[0], time.monotonic() - a[1]
                else:
                    cb = None
            if cb:
                cb(name, el)

    class _Step:
        def __init__(self, wd, name, deadline_s):
            self.wd, self.name, self.deadline_s = wd, name, deadline_s

        def __enter__(self):
            with self.wd._lock:
                self.wd._active = (self.name, time.monotonic(), self.deadline_s, False)
            return self

        def __exit__(self, *exc):
            with self.wd._lock:
                self.wd._active = None
            return False

    def step(self, name: str, deadline_s: float) -> "_Step":
        return Watchdog._Step(self, name, deadline_s)

    def close(self):
        self._stop.set()
        self._thread.join(timeout=1.0)


# ----------------------------------------------------------------------------- heartbeat
class Heartbeat:
    """Rank liveness through a key-value store (a `torch.distributed.TCPStore` or anything with
    `set(key, value)` / `get(key)`): every rank publishes a timestamp from a thread; `dead_ranks`
    lists the ranks whose last beat is older than `timeout_s`."""

    def __init__(self, store, rank: int, world_size: int, interval_s: float = 0.1):
        self.store, self.rank, self.world_size, self.interval_s = store, rank, world_size, interval_s
        self._stop = threading.Event()
        self._beat()
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def _beat(self):
        self.store.set(f"hb/{self.rank}", repr(time.time()))

    def _run(self):
        while not self._stop.wait(self.interval_s):
            try:
                self._beat()
            except Exception:
                return

    def last_seen(self, rank: int) -> Optional[float]:
        try:
            v = self.store.get(f"hb/{rank}")
        except Exception:
            return None
        return float(v.decode() if isinstance(v, (bytes, bytearray)) else v)

    def has_left(self, rank: int) -> bool:
        """True once `rank` has announced its departure with `stop()`."""
        key = f"left/{rank}"
        check = getattr(self.store, "check", None)
        try:
            if check is not None:                 # TCPStore: `get` would block on a missing key
                return bool(check([key]))
            self.store.get(key)
            return True
        except Exception:
            return False

    def dead_ranks(self, timeout_s: float = 1.0) -> List[int]:
        """Ranks that announced their departure or whose last beat is older than `timeout_s`.  The announcement
        makes a clean departure visible at once, whatever the beat interval and the scheduler did."""
        now = time.time()
        dead = []
        for r in range(self.world_size):
            if r == self.rank:
                continue
            if self.has_left(r):
                dead.append(r)
                continue
            t = self.last_seen(r)
            if t is None or now - t > timeout_s:
                dead.append(r)
        return dead

    def stop(self):
        """Stop beating and announce the departure (what a leaving rank does between steps)."""
        self._stop.set()
        self._thread.join(timeout=1.0)
        try:
            self.store.set(f"left/{self.rank}", "1")
        except Exception:
            pass


# ----------------------------------------------------------------------------- fault injection (host only)
class InjectedRankExit(SystemExit):
    """Raised on the rank chosen by a `kill_rank` fault, between steps (no kernel in flight)."""


@dataclasses.dataclass
class FaultPlan:
    """Parsed `B200_FAULT` specification: ``drop_flag:<rank>:<step>``, ``delay_ms:<rank>:<ms>[:<step>]`` or
    ``kill_rank:<rank>:<step>``; several faults separated by commas."""
    drop_flag: Dict[int, int] = dataclasses.field(default_factory=dict)     # rank -> step
    delay_ms: Dict[int, tuple] = dataclasses.field(default_factory=dict)    # rank -> (ms, step or None)
    kill_rank: Dict[int, int] = dataclasses.field(default_factory=dict)     # rank -> step

    @classmethod
    def from_env(cls, value: Optional[str] = None) -> "FaultPlan":
        spec = os.environ.get("B200_FAULT", "") if value is None else value
        plan = cls()
        for item in filter(None, (s.strip() for s in spec.split(","))):
            parts = item.split(":")
            kind = parts[0]
            if kind == "drop_flag" and len(parts) == 3:
                plan.drop_flag[int(parts[1])] = int(parts[2])
            elif kind == "delay_ms" and len(parts) in (3, 4):
                plan.delay_ms[int(parts[1])] = (int(parts[2]), int(parts[3]) if len(parts) == 4 else None)
            elif kind == "kill_rank" and len(parts) == 3:
                plan.kill_rank[int(parts[1])] = int(parts[2])
            else:
                raise ValueError(f"bad B200_FAULT item '{item}'")
        return plan

    def before_step(self, rank: int, step: int) -> None:
        """Call between steps (nothing of this rank in flight): sleeps or leaves as planned."""
        if rank in self.delay_ms:
            ms, at = self.delay_ms[rank]
            if at is None or at == step:
                time.sleep(ms / 1e3)
        if self.kill_rank.get(rank) == step:
            raise InjectedRankExit(f"rank {rank} leaves before step {step} (injected)")

    def drops_signal(self, rank: int, step: int) -> bool:
        """True when `rank` must skip signalling its peers in `step` (they then run into their bounded wait)."""
        return self.drop_flag.get(rank) == step


# ----------------------------------------------------------------------------- protocol model (CPU threads)
class CounterProtocolSim:
    """Thread model of the push / arrival-counter protocol of `FusedTP`: `n` ranks, two alternating buffers,
    counters that only grow.  `run(ops, drop=(rank, op))` executes `ops` fused operations on `n` threads and
    returns per-rank results (sums seen) or the string "timeout" for a rank whose wait expired.  It checks
    the invariant the kernels rely on: a buffer is never overwritten while a peer still reads it."""

    def __init__(self, n: int, wait_limit_s: float = 0.2):
        self.n, self.wait_limit_s = n, wait_limit_s
        self.lock = threading.Lock()
        self.flags = [[[0] * n for _ in range(2)] for _ in range(n)]          # [dest][buffer][src]
        self.slots = [[[None] * n for _ in range(2)] for _ in range(n)]       # [dest][buffer][src] -> (op, value)
        self.reading = [[-1, -1] for _ in range(n)]                           # op a rank is reading, per buffer
        self.violations: List[str] = []

    def _rank(self, r: int, ops: int, drop, out: list):
        seen = [0, 0]
        for op in range(ops):
            b = op & 1
            for d in range(self.n):                                           # push partial + signal
                with self.lock:
                    if self.reading[d][b] not in (-1, op):
                        self.violations.append(f"rank {r} overwrote buffer {b} of rank {d} during op "
                                               f"{self.reading[d][b]}")
                    self.slots[d][b][r] = (op, r + 1 + op)
                    if drop != (r, op):
                        self.flags[d][b][r] += 1
            t0 = time.monotonic()                                             # bounded wait for all sources
            while True:
                with self.lock:
                    ready = all(self.flags[r][b][s] >= seen[b] + 1 for s in range(self.n))
                    if ready:
                        self.reading[r][b] = op
                        break
                if time.monotonic() - t0 > self.wait_limit_s:
                    out[r] = "timeout"
                    return
                time.sleep(0.0005)
            with self.lock:
                vals = [self.slots[r][b][s] for s in range(self.n)]
                self.reading[r][b] = -1
            if any(v is None or v[0] != op for v in vals):
                self.violations.append(f"rank {r} read a stale slot in op {op}")
            out[r].append(sum(v[1] for v in vals))
            seen[b] += 1

    def run(self, ops: int, drop=None):
        out: list = [[] for _ in range(self.n)]
        threads = [threading.Thread(target=self._rank, args=(r, ops, drop, out)) for r in range(self.n)]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        return out


# ----------------------------------------------------------------------------- recovery
@dataclasses.dataclass
class Recovered:
    """What `recover` hands back: the new group (with `.fused` rebuilt when the old one had it), the generation
    number that names this incarnation of the group, and how long the restart took."""
    tp: "object"
    generation: int
    seconds: float


def _release_comm_objects(tp, extra=()) -> int:
    """Release, without any collective, every symmetric buffer that hangs off the group or was passed in."""
    n = 0
    fused = getattr(tp, "fused", None)
    for obj in (fused, *extra):
        if obj is None:
            continue
        (getattr(obj, "abandon", None) or obj.close)()
        n += 1
    if fused is not None:
        tp.fused = None
    return n


def _drop_process_group() -> None:
    """End the current default process group although some of its ranks may be gone: abort where the backend
    offers it (NCCL: no handshake with the peers), destroy otherwise."""
    import torch.distributed as dist

    if not dist.is_initialized():
        return
    abort = getattr(dist.distributed_c10d, "_abort_process_group", None)
    try:
        if abort is not None and dist.get_backend() == "nccl":
            abort()
            return
    except Exception:
        pass
    if dist.is_initialized():
        dist.destroy_process_group()


def recover(tp, *, rank: int, world_size: int, master_port: int, generation: int = 1,
            master_addr: str = "127.0.0.1", timeout_s: int = 60, extra=(), fused_args: Optional[dict] = None,
            backend: Optional[str] = None) -> Recovered:
    """Restart the communication layer of this process after a rank was lost (or to join as its replacement).

    Survivors pass their old group as `tp`; a replacement process passes None.  Steps, all on the host:

      1. no kernel of this process is in flight (device synchronize), the device status word is cleared;
      2. the symmetric buffers reachable from `tp` (`tp.fused`) and those in `extra` (sequence-parallel GEMM
         pairs, the expert all-to-all) are released without a barrier (`abandon`);
      3. the old process group is aborted;
      4. a new group of `world_size` ranks is formed at `master_port` (a port not used by the old group: the
         old store may live in a process that is gone) under the new `generation`;
      5. `FusedTP` is rebuilt with its old sizes (or `fused_args`), which zeroes its flags and restarts its
         call counters, so no stale arrival count survives.

    `rank` / `world_size` describe the NEW group: the same numbers when a replacement process takes the lost
    rank's place, fewer ranks when the job shrinks (the caller then reloads weight shards for the new
    sharding).  KV caches are not carried over; requests in flight are prefilled again.  The reference has
    no counterpart: its runtime reports a failed collective as a status code and stops
    (spike/src/error.h:24-43)."""
    import datetime

    import torch
    import torch.distributed as dist

    from .comm import TPGroup

    t0 = time.time()
    use_cuda = torch.cuda.is_available()
    if tp is not None:
        fused = getattr(tp, "fused", None)
        if fused_args is None and fused is not None:
            fused_args = dict(max_tokens=fused.max_tokens, hidden=fused.hidden, max_splits=fused.max_splits)
        if use_cuda:
            torch.cuda.synchronize()
            from .. import ops

            ops.device_status(reset=True) if _accepts_reset(ops.device_status) else ops.device_status()
        _release_comm_objects(tp, extra)
        _drop_process_group()
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    if tp is not None and tp.device is not None:
        device = tp.device
    else:
        device = torch.device(f"cuda:{local}") if use_cuda else torch.device("cpu")
    if use_cuda:
        torch.cuda.set_device(device)
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world_size), MASTER_ADDR=master_addr,
                      MASTER_PORT=str(master_port), NKIPY_B200_GENERATION=str(generation))
    if world_size == 1:
        new_tp = TPGroup(0, 1, None, device)
    else:
        if backend is None:
            backend = "nccl" if use_cuda else "gloo"
        kwargs = {"device_id": device} if backend == "nccl" else {}
        dist.init_process_group(backend=backend, init_method=f"tcp://{master_addr}:{master_port}", rank=rank,
                                world_size=world_size, timeout=datetime.timedelta(seconds=timeout_s), **kwargs)
        new_tp = TPGroup(rank, world_size, dist.group.WORLD, device)
        new_tp.barrier()
    if fused_args and use_cuda:
        from .symm import FusedTP

        new_tp.fused = FusedTP(new_tp, **fused_args)
    return Recovered(new_tp, generation, time.time() - t0)
