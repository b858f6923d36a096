"""Symmetric (peer-mapped) device memory and the fused tensor-parallel decode ops.

`SymmetricMemory` gives every rank of a group a same-sized device buffer that all
peers can address directly: the buffer is allocated by the kernel library, exported as
a CUDA IPC handle, the handles are exchanged over the process group and every peer's
buffer is mapped into this process (NVLink peer loads / stores).  `FusedTP` builds the
"row-parallel GEMM -> all-reduce -> residual -> RMSNorm" step of decode on it as two
kernels with no library collective in between: the GEMM's epilogue pushes its partial
tiles into every peer's buffer, the norm kernel waits for all arrival counters and
sums the partials (csrc/kernels/gemm_tcgen05.cu push mode, csrc/kernels/comm.cu).

The reference performs these reductions with all-reduce instructions inside the
compiled graph (examples/models/qwen3/kernels/attention.py:150-154); this is the
NVLink-native counterpart.
"""

from __future__ import annotations

import ctypes
from typing import List, Optional, Tuple

import torch

from ..ops import _lib
from .comm import TPGroup


class _CudaArray:
    """Minimal __cuda_array_interface__ carrier so torch can view raw device memory."""

    def __init__(self, ptr: int, nbytes: int, owner):
        self.__cuda_array_interface__ = {
            "shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3, "strides": None,
        }
        self._owner = owner


def exchange_fds(tp: TPGroup, fd: int, only_from: Optional[int] = None) -> List[Optional[int]]:
    """Pass file descriptors between the rank processes of one node over Unix sockets (SCM_RIGHTS).

    Every rank listens on an abstract socket whose name is all-gathered.  With ``only_from`` None every
    rank sends `fd` to every other rank and the result holds the descriptor received from each rank
    (None at this rank's own index); with ``only_from`` = r only rank r sends (fd is ignored elsewhere)
    and the others get its descriptor at index r.  Received descriptors belong to the caller."""
    import os
    import socket
    import uuid

    n, me = tp.world_size, tp.rank
    out: List[Optional[int]] = [None] * n
    if n == 1:
        return out
    srv = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    name = f"\0nkipy-b200-symm-{os.getpid()}-{uuid.uuid4().hex}"
    srv.bind(name)
    srv.listen(n)
    srv.settimeout(60.0)
    try:
        names = tp.all_gather_object(name)
        senders = list(range(n)) if only_from is None else [only_from]
        if me in senders:
            for p in range(n):
                if p == me:
                    continue
                c = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
                c.settimeout(60.0)
                c.connect(names[p])          # queues in the listener's backlog: no accept needed yet
                socket.send_fds(c, [me.to_bytes(4, "little")], [fd])
                c.close()
        expect = [r for r in senders if r != me]
        for _ in expect:
            conn, _addr = srv.accept()
            msg, fds, _flags, _a = socket.recv_fds(conn, 4, 1)
            conn.close()
            if len(msg) != 4 or len(fds) != 1:
                raise RuntimeError("descriptor exchange: short message")
            out[int.from_bytes(msg, "little")] = fds[0]
        tp.barrier()
    finally:
        srv.close()
    return out


def _vmm_runtime():
    """The C++ runtime module when it offers `SymmetricBuffer`, else None."""
    try:
        from ..spike import _spike
    except Exception:      # noqa: BLE001 - the runtime module is optional for the IPC path
        return None
    return _spike if hasattr(_spike, "SymmetricBuffer") else None


class SymmetricMemory:
    """One device allocation per rank, mapped into every rank of the group.

    backend "vmm" (default where supported): the C++ runtime's `SymmetricBuffer` -- `cuMemCreate` with POSIX
    file-descriptor handles, every peer mapped with `cuMemMap`, and with ``multicast=True`` an NVLink
    multicast object bound to all ranks' memory, so kernels can use `multimem` stores / reductions through
    `mc_ptr` (0 when there is none).  backend "ipc": `cudaMalloc` + CUDA IPC handles (no multicast).
    ``NKIPY_B200_SYMM=ipc`` forces the latter, ``NKIPY_B200_NVLS=0`` turns multicast off."""

    def __init__(self, tp: TPGroup, nbytes: int, multicast: bool = False, backend: Optional[str] = None):
        import os

        self.tp = tp
        self.nbytes = int(nbytes)
        self.mc_ptr = 0
        self._closed = False
        self._buf = None
        rt = _vmm_runtime()
        dev_index = tp.device.index if tp.device is not None and tp.device.index is not None else 0
        if backend is None:
            backend = os.environ.get("NKIPY_B200_SYMM", "vmm")
        ok = backend == "vmm" and rt is not None and rt.SymmetricBuffer.supported(dev_index)
        # every rank must take the same path
        if not all(tp.all_gather_object(bool(ok))):
            ok = False
        self.backend = "vmm" if ok else "ipc"
        if self.backend == "vmm":
            want_mc = (multicast and tp.world_size > 1 and os.environ.get("NKIPY_B200_NVLS", "1") != "0"
                       and rt.SymmetricBuffer.multicast_supported(dev_index))
            want_mc = all(tp.all_gather_object(bool(want_mc)))
            self._init_vmm(rt, dev_index, want_mc)
        else:
            self._init_ipc()

    def _device_sync(self) -> None:
        """Wait for this process's device work; a group without a CUDA device (host-side tests) has none."""
        dev = self.tp.device
        if dev is not None and getattr(dev, "type", "cuda") == "cuda":
            torch.cuda.synchronize()

    # ------------------------------------------------------------------ VMM + multicast
    def _init_vmm(self, rt, dev_index: int, want_mc: bool) -> None:
        import os

        tp = self.tp
        self._device_sync()
        buf = rt.SymmetricBuffer(dev_index, self.nbytes)
        self._buf = buf
        buf.zero()
        self.local_ptr = int(buf.local_ptr)
        fd = buf.export_fd()
        try:
            got = exchange_fds(tp, fd)
        finally:
            os.close(fd)
        self.ptrs: List[int] = []
        for r, pfd in enumerate(got):
            if r == tp.rank:
                self.ptrs.append(self.local_ptr)
                continue
            try:
                buf.import_peer(r, pfd)
            finally:
                os.close(pfd)
            self.ptrs.append(int(buf.peer_ptr(r)))
        tp.barrier()
        if want_mc:
            mfd = buf.multicast_create(tp.world_size) if tp.rank == 0 else -1
            try:
                got = exchange_fds(tp, mfd, only_from=0)
            finally:
                if mfd >= 0:
                    os.close(mfd)
            if tp.rank != 0:
                try:
                    buf.multicast_import(got[0])
                finally:
                    os.close(got[0])
            buf.multicast_add_device()
            tp.barrier()                      # every device is part of the object before anyone binds
            buf.multicast_bind()
            tp.barrier()
            self.mc_ptr = int(buf.multicast_ptr)

    # ------------------------------------------------------------------ cudaMalloc + CUDA IPC
    def _init_ipc(self) -> None:
        tp = self.tp
        lib = _lib.lib()
        for name, res, args in (
            ("nkb_symm_alloc", ctypes.c_int, [ctypes.POINTER(ctypes.c_void_p), ctypes.c_longlong]),
            ("nkb_symm_free", ctypes.c_int, [ctypes.c_void_p]),
            ("nkb_ipc_get_handle", ctypes.c_int, [ctypes.c_void_p, ctypes.c_char_p]),
            ("nkb_ipc_open", ctypes.c_int, [ctypes.c_char_p, ctypes.POINTER(ctypes.c_void_p)]),
            ("nkb_ipc_close", ctypes.c_int, [ctypes.c_void_p]),
        ):
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        self._lib = lib
        local = ctypes.c_void_p()
        _lib.check(lib.nkb_symm_alloc(ctypes.byref(local), self.nbytes), "nkb_symm_alloc")
        self.local_ptr = int(local.value)
        handle = ctypes.create_string_buffer(64)
        _lib.check(lib.nkb_ipc_get_handle(local, handle), "nkb_ipc_get_handle")
        handles = tp.all_gather_object(bytes(handle.raw))
        self.ptrs = []
        self._opened: List[int] = []
        for r, h in enumerate(handles):
            if r == tp.rank:
                self.ptrs.append(self.local_ptr)
                continue
            p = ctypes.c_void_p()
            _lib.check(lib.nkb_ipc_open(ctypes.create_string_buffer(h, 64), ctypes.byref(p)), "nkb_ipc_open")
            self.ptrs.append(int(p.value))
            self._opened.append(int(p.value))
        tp.barrier()

    def view(self, offset: int, nbytes: int, dtype: torch.dtype, shape: Tuple[int, ...]) -> torch.Tensor:
        """torch view of a region of the *local* buffer."""
        raw = torch.as_tensor(_CudaArray(self.local_ptr + offset, nbytes, self), device=self.tp.device)
        return raw.view(dtype).view(shape)

    def abandon(self) -> None:
        """Release this rank's mappings and memory WITHOUT talking to the peers: the recovery path, for when a
        peer has left and a barrier would never complete.  The caller guarantees that no kernel of this process
        that touches the buffer is in flight (a device synchronize is done here) and that this rank will not be
        addressed by a live peer's kernel any more -- a peer that left between steps satisfies both."""
        if self._closed:
            return
        self._closed = True
        self._device_sync()
        if self.backend == "vmm":
            self._buf.close()
            return
        for p in self._opened:
            self._lib.nkb_ipc_close(ctypes.c_void_p(p))
        self._lib.nkb_symm_free(ctypes.c_void_p(self.local_ptr))

    def close(self) -> None:
        """Collective: every rank calls it.  Nothing is unmapped or released while a peer may still use it."""
        if self._closed:
            return
        self._closed = True
        self._device_sync()
        self.tp.barrier()
        if self.backend == "vmm":
            self._buf.close()
            self.tp.barrier()
            return
        for p in self._opened:
            self._lib.nkb_ipc_close(ctypes.c_void_p(p))
        self.tp.barrier()
        self._lib.nkb_symm_free(ctypes.c_void_p(self.local_ptr))


class FusedTP:
    """Fused row-parallel GEMM + all-reduce + residual + RMSNorm for decode-sized batches.  One rank is allowed
    (the same two kernels, the only "peer" being this GPU): single-GPU tests and profiles use it."""

    FLAG_BYTES = 16384
    ARGMAX_FLAG_OFFSET = 1024      # byte offset of the argmax arrival counters inside the flag page
    ROWFLAG_OFFSET = 4096          # per-row arrival counters of the pre-summing exchange: [2 buffers][8 ranks][128 rows]
    ROWFLAG_ROWS = 128

    def __init__(self, tp: TPGroup, max_tokens: int, hidden: int, max_splits: int = 8):
        if tp.world_size > 8:
            raise ValueError("FusedTP supports up to 8 ranks (one NVSwitch domain)")
        self.tp = tp
        self.max_tokens, self.hidden, self.max_splits = max_tokens, hidden, max_splits
        n = tp.world_size
        self.buf_bytes = n * max_splits * max_tokens * hidden * 2
        self.buf_bytes = (self.buf_bytes + 255) // 256 * 256
        self.pair_bytes = (2 * n * max_tokens * 8 + 255) // 256 * 256
        self.mem = SymmetricMemory(tp, self.FLAG_BYTES + 2 * self.buf_bytes + self.pair_bytes, multicast=True)
        dev = tp.device
        self.seen = torch.zeros((4,), dtype=torch.int32, device=dev)   # [buffer 0, buffer 1, argmax, spare]
        # uses of each buffer by the pre-summing exchange (its row counters advance only with those uses)
        self.seen_rows = torch.zeros((2,), dtype=torch.int32, device=dev)
        self.done = torch.zeros((4,), dtype=torch.int32, device=dev)   # [producer, reduce0, reduce1, spare]
        self._parity = 0
        self.ops_issued = 0
        # how the producer sums its split-K partials: see ops.DECODE_GEMM_IMPL ("legacy" pushes one partial per split)
        from .. import ops as _ops

        self.impl = _ops.DECODE_GEMM_IMPL
        # "presum" (default): the GEMM leaves fp32 split-K partials locally and one kernel sums them, exchanges one
        # bf16 row per rank, sums over ranks and norms; "push": the GEMM epilogue pushes one partial per split
        import os as _os

        self.exchange = _os.environ.get("NKIPY_B200_TP_EXCHANGE", "presum")
        # the pre-summing kernel pays one more hop of latency (sum, store, flag, wait, sum) and wins when it saves
        # traffic: from this many split-K partials on; below, the GEMM pushes its partials itself
        self.presum_min_splits = int(_os.environ.get("NKIPY_B200_PRESUM_MIN_SPLITS", "3"))
        # ... and from this many ranks on (measured: 2 ranks 15.3K tok/s with the push against 15.1K, Qwen3 12.3K
        # against 11.5K; 4 ranks 20.3K against 18.0K; 8 ranks 20.9K against 19.8K)
        self.presum_min_world = int(_os.environ.get("NKIPY_B200_PRESUM_MIN_WORLD", "4"))
        lib = _lib.lib()
        P, I, LL = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
        PP = ctypes.POINTER(P)
        lib.nkb_gemm_bf16_push.restype = I
        lib.nkb_gemm_bf16_push.argtypes = [P, P, I, I, I, LL, LL, LL, I, P, I, PP, PP, I, I, P, P, P, P]
        lib.nkb_tp_reduce_rmsnorm.restype = I
        lib.nkb_tp_reduce_rmsnorm.argtypes = [P, I, P, I, P, P, P, P, P, P, I, I, ctypes.c_float, P]
        lib.nkb_tp_exchange_reduce_rmsnorm.restype = I
        lib.nkb_tp_exchange_reduce_rmsnorm.argtypes = [P, I, LL, P, PP, PP, P, P, I, I, P, P, P, P, P, P, P, P, I, I,
                                                       ctypes.c_float, P]
        lib.nkb_moe_combine_push.restype = I
        lib.nkb_moe_combine_push.argtypes = [P, P, P, I, I, I, PP, PP, I, I, P, P, P, P]
        lib.nkb_argmax_exchange.restype = I
        lib.nkb_argmax_exchange.argtypes = [P, P, I, I, I, PP, PP, I, I, P, P, P, P, P]
        self._lib = lib
        self._peer_out = [(P * n)(*[p + self.FLAG_BYTES + b * self.buf_bytes for p in self.mem.ptrs])
                          for b in range(2)]
        self._peer_flag = [(P * n)(*[p + (b * n + tp.rank) * 4 for p in self.mem.ptrs]) for b in range(2)]
        # the same two locations inside the NVLink multicast mapping (None without one): a store there lands
        # in every rank's buffer, so a partial crosses this GPU's links once instead of once per peer
        mc = self.mem.mc_ptr
        self._mc_out = [P(mc + self.FLAG_BYTES + b * self.buf_bytes) if mc else None for b in range(2)]
        self._mc_flag = [P(mc + (b * n + tp.rank) * 4) if mc else None for b in range(2)]
        rf = self.ROWFLAG_OFFSET
        rf_bytes = 8 * self.ROWFLAG_ROWS * 4
        self._peer_rowflag = [(P * n)(*[p + rf + b * rf_bytes for p in self.mem.ptrs]) for b in range(2)]
        self._mc_rowflag = [P(mc + rf + b * rf_bytes) if mc else None for b in range(2)]
        self._rowflag_bytes = rf_bytes
        pair_off = self.FLAG_BYTES + 2 * self.buf_bytes
        self._pair_off = pair_off
        self._peer_pairs = (P * n)(*[p + pair_off for p in self.mem.ptrs])
        self._peer_aflag = (P * n)(*[p + self.ARGMAX_FLAG_OFFSET + tp.rank * 4 for p in self.mem.ptrs])

    def begin_step(self) -> None:
        """Call at the start of every decode body: buffers alternate per operation and a
        step must contain an even number of fused operations."""
        if self.ops_issued % 2:
            raise RuntimeError("a decode step must issue an even number of fused TP operations")
        self._parity = 0

    def _buffer(self, b: int) -> dict:
        """Addresses of buffer b for a kernel that runs both halves of a fused operation itself."""
        n, base = self.tp.world_size, self.mem.local_ptr
        return dict(n=n, rank=self.tp.rank, max_slots=n * self.max_splits, peer_out=self._peer_out[b],
                    peer_flag=self._peer_flag[b], mc_out=self._mc_out[b], mc_flag=self._mc_flag[b],
                    slabs=base + self.FLAG_BYTES + b * self.buf_bytes, flags=base + b * n * 4,
                    seen=self.seen.data_ptr() + 4 * b, done=self.done.data_ptr())

    def buffer(self, b: int) -> dict:
        return self._buffer(b)

    def next_buffer(self, tokens: int, hidden: int) -> dict:
        """The buffer of ONE fused operation whose two halves run inside another kernel (counts as one)."""
        if tokens > self.max_tokens or hidden != self.hidden:
            raise ValueError(f"FusedTP sized for [{self.max_tokens}, {self.hidden}], got [{tokens}, {hidden}]")
        b = self._parity
        self._parity ^= 1
        self.ops_issued += 1
        return self._buffer(b)

    def layer_buffers(self, tokens: int, hidden: int):
        """The two buffers (o_proj, down) of one launch of the persistent decode-layer kernel
        (`ops.decode_layer.decode_layer`): counts as two fused operations of the step."""
        if tokens > self.max_tokens or hidden != self.hidden:
            raise ValueError(f"FusedTP sized for [{self.max_tokens}, {self.hidden}], got [{tokens}, {hidden}]")
        b = self._parity
        self.ops_issued += 2
        return self._buffer(b), self._buffer(b ^ 1)

    def gemm_allreduce_add_rmsnorm(self, x: torch.Tensor, w: torch.Tensor, resid: Optional[torch.Tensor],
                                   next_norm: Optional[torch.Tensor], bias: Optional[torch.Tensor], eps: float,
                                   splits: int = 1):
        """``h = sum_ranks(x @ w.T) (+ bias) + resid``; returns (h as bf16, rmsnorm(h) * next_norm)."""
        from .. import ops

        M, K = x.shape
        N = w.shape[0]
        if M > self.max_tokens or N != self.hidden:
            raise ValueError(f"FusedTP sized for [{self.max_tokens}, {self.hidden}], got [{M}, {N}]")
        lib = self._lib
        block_n = 32 if M <= 32 else (64 if M <= 64 else 128)
        stream = torch.cuda.current_stream().cuda_stream
        n = self.tp.world_size
        if self.impl == "fixup" and M <= 128:
            # split-K summed inside the producer (last-arriver fix-up): exactly one bf16 partial leaves this rank
            b = self._parity
            self._parity ^= 1
            self.ops_issued += 1
            part, ctr = ops.fix_scratch(x.device, lib.nkb_gemm_fix_scratch_floats(N, M, K, max(1, int(splits))))
            rc = lib.nkb_gemm_fix_push(w.data_ptr(), x.data_ptr(), N, M, K, w.stride(0), x.stride(0),
                                       max(1, int(splits)), None if bias is None else bias.data_ptr(),
                                       self._peer_out[b], self._peer_flag[b], n, self.tp.rank, self.done.data_ptr(),
                                       self._mc_out[b], self._mc_flag[b], part.data_ptr(), ctr.data_ptr(), block_n,
                                       stream)
            _lib.check(rc, "nkb_gemm_fix_push")
            ops._launches += 1
            return self._reduce(b, n, M, resid, next_norm, eps, x.device)
        if self.impl == "cluster" and M <= 128:
            # split-K summed inside the producer (CTA clusters): exactly one bf16 partial leaves this rank
            b = self._parity
            self._parity ^= 1
            self.ops_issued += 1
            rc = lib.nkb_decode_gemm_push(w.data_ptr(), x.data_ptr(), N, M, K, w.stride(0), x.stride(0), N,
                                          max(1, int(splits)), None if bias is None else bias.data_ptr(), block_n,
                                          self._peer_out[b], self._peer_flag[b], n, self.tp.rank,
                                          self.done.data_ptr(), self._mc_out[b], self._mc_flag[b], stream)
            _lib.check(rc, "nkb_decode_gemm_push")
            ops._launches += 1
            return self._reduce(b, n, M, resid, next_norm, eps, x.device)
        if (self.exchange == "presum" and M <= self.ROWFLAG_ROWS and int(splits) >= self.presum_min_splits
                and self.tp.world_size >= self.presum_min_world):
            return self.exchange_add_rmsnorm(ops.linear(x, w, bias=bias, splits=int(splits)), resid, next_norm, eps)
        eff = lib.nkb_gemm_effective_splits(K, max(1, min(splits, self.max_splits)))
        b = self._parity
        self._parity ^= 1
        self.ops_issued += 1
        rc = lib.nkb_gemm_bf16_push(w.data_ptr(), x.data_ptr(), N, M, K, w.stride(0), x.stride(0), N, eff,
                                    None if bias is None else bias.data_ptr(), block_n, self._peer_out[b],
                                    self._peer_flag[b], n, self.tp.rank, self.done.data_ptr(), self._mc_out[b],
                                    self._mc_flag[b], stream)
        _lib.check(rc, "nkb_gemm_bf16_push")
        ops._launches += 1
        return self._reduce(b, n * eff, M, resid, next_norm, eps, x.device)

    def exchange_add_rmsnorm(self, parts: torch.Tensor, resid: Optional[torch.Tensor],
                             next_norm: Optional[torch.Tensor], eps: float):
        """parts: this rank's result of a row-parallel GEMM, fp32 split-K partials [S, M, N] (or bf16 [M, N]).
        One launch sums the partials, sends one bf16 row per rank over NVLink, sums over ranks, adds the residual
        and applies the RMSNorm.  Returns (new residual bf16, normed)."""
        from .. import ops

        if parts.dim() == 3:
            S, M, N = parts.shape
            p_ptr, y_ptr, stride = parts.data_ptr(), None, M * N
        else:
            (M, N), S = parts.shape, 0
            p_ptr, y_ptr, stride = None, parts.data_ptr(), 0
        if M > min(self.max_tokens, self.ROWFLAG_ROWS) or N != self.hidden:
            raise ValueError(f"exchange sized for [{min(self.max_tokens, self.ROWFLAG_ROWS)}, {self.hidden}]")
        b = self._parity
        self._parity ^= 1
        self.ops_issued += 1
        n, base, dev = self.tp.world_size, self.mem.local_ptr, parts.device
        resid_out = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
        normed = torch.empty((M, N), dtype=torch.bfloat16, device=dev) if next_norm is not None else None
        rc = self._lib.nkb_tp_exchange_reduce_rmsnorm(
            p_ptr, S, stride, y_ptr, self._peer_out[b], self._peer_rowflag[b], self._mc_out[b], self._mc_rowflag[b], n,
            self.tp.rank, base + self.FLAG_BYTES + b * self.buf_bytes,
            base + self.ROWFLAG_OFFSET + b * self._rowflag_bytes, self.seen_rows.data_ptr() + 4 * b,
            self.done.data_ptr() + 4 * (1 + b), None if resid is None else resid.data_ptr(),
            None if next_norm is None else next_norm.data_ptr(), resid_out.data_ptr(),
            None if normed is None else normed.data_ptr(), M, N, float(eps), torch.cuda.current_stream().cuda_stream)
        _lib.check(rc, "nkb_tp_exchange_reduce_rmsnorm")
        ops._launches += 1
        return resid_out, normed

    def _reduce(self, b: int, slots: int, M: int, resid, next_norm, eps: float, device):
        """Consumer of buffer b: wait for all ranks, sum the slots, add the residual, RMSNorm."""
        from .. import ops

        n, N = self.tp.world_size, self.hidden
        resid_out = torch.empty((M, N), dtype=torch.bfloat16, device=device)
        normed = torch.empty((M, N), dtype=torch.bfloat16, device=device) if next_norm is not None else None
        rc = self._lib.nkb_tp_reduce_rmsnorm(
            self.mem.local_ptr + self.FLAG_BYTES + b * self.buf_bytes, slots, self.mem.local_ptr + b * n * 4, n,
            self.seen.data_ptr() + 4 * b, self.done.data_ptr() + 4 * (1 + b),
            None if resid is None else resid.data_ptr(), None if next_norm is None else next_norm.data_ptr(),
            resid_out.data_ptr(), None if normed is None else normed.data_ptr(), M, N, float(eps),
            torch.cuda.current_stream().cuda_stream)
        _lib.check(rc, "nkb_tp_reduce_rmsnorm")
        ops._launches += 1
        return resid_out, normed

    def moe_combine_allreduce_add_rmsnorm(self, y_sorted: torch.Tensor, pair_pos: torch.Tensor,
                                          weights: torch.Tensor, tokens: int, resid: Optional[torch.Tensor],
                                          next_norm: Optional[torch.Tensor], eps: float):
        """Expert-parallel combine: the weighted sum of this rank's expert outputs per token is pushed into
        every peer's partial buffer by the combine kernel itself; the consumer sums over ranks, adds the
        residual and applies the next RMSNorm.  Returns (new residual, normed)."""
        from .. import ops

        if tokens > self.max_tokens or y_sorted.shape[1] != self.hidden:
            raise ValueError(f"FusedTP sized for [{self.max_tokens}, {self.hidden}]")
        b = self.moe_combine_push(y_sorted, pair_pos, weights, tokens)
        return self._reduce(b, self.tp.world_size, tokens, resid, next_norm, eps, y_sorted.device)

    def moe_combine_push(self, y_sorted: torch.Tensor, pair_pos: torch.Tensor, weights: torch.Tensor,
                         tokens: int) -> int:
        """The producer half alone: this rank's weighted expert outputs go into slot [rank] of the next buffer on
        every rank.  Returns the buffer index; the caller runs the consumer (`_reduce`, or the reducing stage of the
        persistent layer kernel through `buffer(b)`)."""
        from .. import ops

        if tokens > self.max_tokens or y_sorted.shape[1] != self.hidden:
            raise ValueError(f"FusedTP sized for [{self.max_tokens}, {self.hidden}]")
        b = self._parity
        self._parity ^= 1
        self.ops_issued += 1
        n = self.tp.world_size
        rc = self._lib.nkb_moe_combine_push(y_sorted.data_ptr(), pair_pos.data_ptr(), weights.data_ptr(), tokens,
                                            weights.shape[1], self.hidden, self._peer_out[b], self._peer_flag[b], n,
                                            self.tp.rank, self.done.data_ptr(), self._mc_out[b], self._mc_flag[b],
                                            torch.cuda.current_stream().cuda_stream)
        _lib.check(rc, "nkb_moe_combine_push")
        ops._launches += 1
        return b

    def argmax_exchange(self, vals: torch.Tensor, ids: torch.Tensor, id_offset: int,
                        out_ids: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Global arg-max of a vocabulary-parallel head: vals / ids are this rank's per-row maximum (fp32)
        and local index (int32); returns the global ids (int32 [rows]) on every rank."""
        from .. import ops

        rows = vals.shape[0]
        if rows > self.max_tokens:
            raise ValueError(f"FusedTP sized for {self.max_tokens} rows, got {rows}")
        if out_ids is None:
            out_ids = torch.empty((rows,), dtype=torch.int32, device=vals.device)
        rc = self._lib.nkb_argmax_exchange(vals.data_ptr(), ids.data_ptr(), rows, self.max_tokens, int(id_offset),
                                           self._peer_pairs, self._peer_aflag, self.tp.world_size, self.tp.rank,
                                           self.mem.local_ptr + self._pair_off,
                                           self.mem.local_ptr + self.ARGMAX_FLAG_OFFSET,
                                           self.seen.data_ptr() + 8, out_ids.data_ptr(),
                                           torch.cuda.current_stream().cuda_stream)
        _lib.check(rc, "nkb_argmax_exchange")
        ops._launches += 1
        return out_ids

    def close(self) -> None:
        self.mem.close()

    def abandon(self) -> None:
        """Non-collective release for the recovery path (`SymmetricMemory.abandon`)."""
        self.mem.abandon()


class _FusedGemmCollective:
    """Shared plumbing of `GemmReduceScatter` and `AllGatherGemm`: two alternating symmetric buffers
    plus one array of arrival counters per rank, and the call counter the kernels compare against."""

    FLAG_BYTES = 8192

    @classmethod
    def max_rows(cls, world: int) -> int:
        """Largest total row count the counter array can describe."""
        return cls.FLAG_BYTES // (4 * world) * 128 * world

    def __init__(self, tp: TPGroup, buf_bytes: int, rows_per_rank: int):
        if tp.world_size > 8:
            raise ValueError("fused GEMM collectives support up to 8 ranks (one NVSwitch domain)")
        self.tp = tp
        self.flag_stride = (rows_per_rank + 127) // 128
        if tp.world_size * self.flag_stride * 4 > self.FLAG_BYTES:
            raise ValueError("too many row tiles per rank for the counter array")
        self.buf_bytes = (int(buf_bytes) + 255) // 256 * 256
        self.mem = SymmetricMemory(tp, self.FLAG_BYTES + 2 * self.buf_bytes)
        P = ctypes.c_void_p
        n = tp.world_size
        self._bufs = [(P * n)(*[p + self.FLAG_BYTES + b * self.buf_bytes for p in self.mem.ptrs]) for b in range(2)]
        self._flags = (P * n)(*self.mem.ptrs)
        self.epoch = 0
        self._lib = _lib.lib()

    def _next(self):
        self.epoch += 1
        return self.epoch, self._bufs[self.epoch & 1]

    def close(self) -> None:
        self.mem.close()

    def abandon(self) -> None:
        self.mem.abandon()


class GemmReduceScatter(_FusedGemmCollective):
    """``out[M/tp, N] = reduce_scatter_rows(x[M, K/tp] @ w[N, K/tp].T)`` as one kernel per rank
    (csrc/kernels/gemm_comm.cu): finished tiles are stored into the owner rank's staging buffer over
    NVLink while later tiles are computed; the owner's CTAs sum the tp partials at the end."""

    def __init__(self, tp: TPGroup, m: int, n: int):
        """m is the capacity: calls may pass any row count up to it (a multiple of the number of ranks)."""
        if m % tp.world_size:
            raise ValueError("m must be divisible by the number of ranks")
        self.m, self.n = m, n
        super().__init__(tp, m * n * 2, m // tp.world_size)
        I, LL, P, U = ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_uint
        self._lib.nkb_gemm_rs.restype = I
        self._lib.nkb_gemm_rs.argtypes = [P, P, P, I, I, I, LL, LL, LL, ctypes.POINTER(P), ctypes.POINTER(P), I, I, I,
                                          U, P]

    def __call__(self, x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        from .. import ops

        m, k = x.shape
        n = w.shape[0]
        if m > self.m or m % self.tp.world_size or n != self.n or w.shape[1] != k:
            raise ValueError(f"GemmReduceScatter sized for up to [{self.m}, {self.n}], got x {tuple(x.shape)} "
                             f"w {tuple(w.shape)}")
        tp = self.tp
        if out is None:
            out = torch.empty((m // tp.world_size, n), dtype=torch.bfloat16, device=x.device)
        epoch, bufs = self._next()
        rc = self._lib.nkb_gemm_rs(x.data_ptr(), w.data_ptr(), out.data_ptr(), m, n, k, x.stride(0), w.stride(0),
                                   out.stride(0), bufs, self._flags, self.flag_stride, tp.world_size, tp.rank, epoch,
                                   torch.cuda.current_stream().cuda_stream)
        _lib.check(rc, "nkb_gemm_rs")
        ops._launches += 1
        return out


class AllGatherGemm(_FusedGemmCollective):
    """``out[M, N/tp] = all_gather_rows(x_local[M/tp, K]) @ w[N/tp, K].T`` as one kernel per rank
    (csrc/kernels/gemm_comm.cu): a few CTAs push this rank's slab chunk by chunk into every peer's
    gather buffer while the others multiply the slabs in arrival order."""

    def __init__(self, tp: TPGroup, m: int, k: int, comm_ctas: int = 0):
        """m is the capacity: calls may gather any row count up to it (the same on every rank)."""
        if m % tp.world_size:
            raise ValueError("m must be divisible by the number of ranks")
        self.m, self.k, self.comm_ctas = m, k, comm_ctas
        super().__init__(tp, m * k * 2, m // tp.world_size)
        I, LL, P, U = ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_uint
        self._lib.nkb_ag_gemm.restype = I
        self._lib.nkb_ag_gemm.argtypes = [P, P, P, I, I, I, LL, LL, LL, ctypes.POINTER(P), ctypes.POINTER(P), I, I, I,
                                          U, I, I, P]

    @staticmethod
    def _swiglu(gu: torch.Tensor) -> torch.Tensor:
        from .. import ops

        i = gu.shape[1] // 2
        if i % 8 == 0:
            return ops.silu_mul(gu)
        return (torch.nn.functional.silu(gu[:, :i].float()) * gu[:, i:].float()).to(gu.dtype)

    def __call__(self, x_local: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None,
                 gated: bool = False) -> torch.Tensor:
        """gated: w holds [gate; up] rows (2 * I) and the result is ``silu(x @ gate.T) * (x @ up.T)`` [M, I]
        (SwiGLU in the epilogue; falls back to a separate activation kernel when the shape does not take the
        CTA-pair kernel)."""
        from .. import ops

        rows, k = x_local.shape
        n = w.shape[0] // 2 if gated else w.shape[0]
        tp = self.tp
        m = rows * tp.world_size
        if m > self.m or k != self.k or w.shape[1] != k:
            raise ValueError(f"AllGatherGemm sized for up to [{self.m}, {self.k}], got x {tuple(x_local.shape)} "
                             f"w {tuple(w.shape)}")
        if out is None:
            out = torch.empty((m, n), dtype=torch.bfloat16, device=x_local.device)
        if gated and (m < 256 or n < 128 or n % 8):
            return self._swiglu(self(x_local, w))
        epoch, bufs = self._next()
        rc = self._lib.nkb_ag_gemm(x_local.data_ptr(), w.data_ptr(), out.data_ptr(), m, n, k, x_local.stride(0),
                                   w.stride(0), out.stride(0), bufs, self._flags, self.flag_stride, tp.world_size,
                                   tp.rank, epoch, self.comm_ctas, 1 if gated else 0,
                                   torch.cuda.current_stream().cuda_stream)
        if rc == -5 and gated:
            self.epoch -= 1
            return self._swiglu(self(x_local, w))
        _lib.check(rc, "nkb_ag_gemm")
        ops._launches += 1
        return out
