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


class SymmetricMemory:
    """One device allocation per rank, mapped into every rank of the group."""

    def __init__(self, tp: TPGroup, nbytes: int):
        self.tp = tp
        self.nbytes = int(nbytes)
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
        self.ptrs: List[int] = []
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
        self._closed = False

    def view(self, offset: int, nbytes: int, dtype: torch.dtype, shape: Tuple[int, ...]) -> torch.Tensor:
        """torch view of a region of the *local* buffer."""
        raw = torch.as_tensor(_CudaArray(self.local_ptr + offset, nbytes, self), device=self.tp.device)
        return raw.view(dtype).view(shape)

    def close(self) -> None:
        if self._closed:
            return
        self._closed = True
        torch.cuda.synchronize()
        self.tp.barrier()
        for p in self._opened:
            self._lib.nkb_ipc_close(ctypes.c_void_p(p))
        self.tp.barrier()
        self._lib.nkb_symm_free(ctypes.c_void_p(self.local_ptr))


class FusedTP:
    """Fused row-parallel GEMM + all-reduce + residual + RMSNorm for decode-sized batches."""

    FLAG_BYTES = 4096

    def __init__(self, tp: TPGroup, max_tokens: int, hidden: int, max_splits: int = 8):
        if tp.world_size < 2:
            raise ValueError("FusedTP needs at least two ranks")
        if tp.world_size > 8:
            raise ValueError("FusedTP supports up to 8 ranks (one NVSwitch domain)")
        self.tp = tp
        self.max_tokens, self.hidden, self.max_splits = max_tokens, hidden, max_splits
        self.buf_bytes = tp.world_size * max_splits * max_tokens * hidden * 2
        self.buf_bytes = (self.buf_bytes + 255) // 256 * 256
        self.mem = SymmetricMemory(tp, self.FLAG_BYTES + 2 * self.buf_bytes)
        dev = tp.device
        self.seen = torch.zeros((2,), dtype=torch.int32, device=dev)
        self.done = torch.zeros((4,), dtype=torch.int32, device=dev)   # [gemm, reduce0, reduce1, spare]
        self._parity = 0
        self.ops_issued = 0
        lib = _lib.lib()
        P, I, LL = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
        lib.nkb_gemm_bf16_push.restype = I
        lib.nkb_gemm_bf16_push.argtypes = [P, P, I, I, I, LL, LL, LL, I, P, I, ctypes.POINTER(P), ctypes.POINTER(P),
                                           I, I, P, P]
        lib.nkb_tp_reduce_rmsnorm.restype = I
        lib.nkb_tp_reduce_rmsnorm.argtypes = [P, I, P, I, P, P, P, P, P, P, I, I, ctypes.c_float, P]
        self._lib = lib
        n = tp.world_size
        self._peer_out = [(P * n)(*[p + self.FLAG_BYTES + b * self.buf_bytes for p in self.mem.ptrs])
                          for b in range(2)]
        self._peer_flag = [(P * n)(*[p + (b * n + tp.rank) * 4 for p in self.mem.ptrs]) for b in range(2)]

    def begin_step(self) -> None:
        """Call at the start of every decode body: buffers alternate per operation and a
        step must contain an even number of fused operations."""
        if self.ops_issued % 2:
            raise RuntimeError("a decode step must issue an even number of fused TP operations")
        self._parity = 0

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
        eff = lib.nkb_gemm_effective_splits(K, max(1, min(splits, self.max_splits)))
        b = self._parity
        self._parity ^= 1
        self.ops_issued += 1
        n = self.tp.world_size
        block_n = 32 if M <= 32 else (64 if M <= 64 else 128)
        stream = torch.cuda.current_stream().cuda_stream
        rc = lib.nkb_gemm_bf16_push(w.data_ptr(), x.data_ptr(), N, M, K, w.stride(0), x.stride(0), N, eff,
                                    None if bias is None else bias.data_ptr(), block_n, self._peer_out[b],
                                    self._peer_flag[b], n, self.tp.rank, self.done.data_ptr(), stream)
        _lib.check(rc, "nkb_gemm_bf16_push")
        resid_out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
        normed = torch.empty((M, N), dtype=torch.bfloat16, device=x.device) if next_norm is not None else None
        rc = lib.nkb_tp_reduce_rmsnorm(
            self.mem.local_ptr + self.FLAG_BYTES + b * self.buf_bytes, n * eff, self.mem.local_ptr + b * n * 4, n,
            self.seen.data_ptr() + 4 * b, self.done.data_ptr() + 4 * (1 + b),
            None if resid is None else resid.data_ptr(), None if next_norm is None else next_norm.data_ptr(),
            resid_out.data_ptr(), None if normed is None else normed.data_ptr(), M, N, float(eps), stream)
        _lib.check(rc, "nkb_tp_reduce_rmsnorm")
        ops._launches += 2
        return resid_out, normed

    def close(self) -> None:
        self.mem.close()
