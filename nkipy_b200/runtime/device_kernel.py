"""Compile-once / load-once device kernels with an on-disk cache and SPMD / MPMD builds.

`DeviceKernel.compile_and_load(kernel, *args, name=..., is_spmd=..., ...)` traces the kernel
on the given example arguments (NumPy arrays or `DeviceTensor`s), derives the cache key
``{name}_{content_hash}`` from the IR and the compiler arguments, reuses
``{build_dir}/{key}/{name}.cubin`` when present, and loads it once per process
(`_LOADED_KERNELS`).  Under `torch.distributed`: SPMD — rank 0 compiles and broadcasts the
artifact path, all ranks barrier, then load; MPMD — every rank compiles into
``build_dir/rank_{r}``.  Same contract as nkipy/src/nkipy/runtime/device_kernel.py:52-270.
"""

from __future__ import annotations

import os
import time
from typing import Dict, Optional

import numpy as np

from ..core.compile import CompilationTarget, _get_build_dir, compile_to_neff, trace
from ..core.logger import get_logger
from ..core.trace import NKIPyKernel
from ..spike.spike_model import SpikeModel
from .device_tensor import DeviceTensor

logger = get_logger()
_LOADED_KERNELS: Dict[str, "DeviceKernel"] = {}


def _dist():
    try:
        import torch.distributed as dist

        return dist
    except ImportError:          # pragma: no cover
        return None


def _is_distributed() -> bool:
    dist = _dist()
    return bool(dist and dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1)


class DeviceKernel(SpikeModel):
    @classmethod
    def compile_and_load(cls, kernel, *args, name: Optional[str] = None, additional_compiler_args: str = "",
                         use_cached_if_exists: bool = True, build_dir: Optional[str] = None,
                         target: CompilationTarget = CompilationTarget.DEFAULT, is_spmd: bool = True,
                         cc_enabled: Optional[bool] = None, rank_id: Optional[int] = None,
                         world_size: Optional[int] = None, core_id: int = 0, **kwargs) -> "DeviceKernel":
        if not isinstance(kernel, NKIPyKernel):
            kernel = trace(kernel)
        name = name or kernel.__name__
        build_dir = build_dir or _get_build_dir()
        distributed = _is_distributed()
        dist = _dist()
        dist_rank = dist.get_rank() if distributed else 0
        if not is_spmd:
            # MPMD: every rank traces its own program, so nothing is broadcast and nobody waits; the artifacts of
            # different ranks live side by side under rank_<r> (explicit rank first, else the group's)
            ns = rank_id if rank_id is not None else (dist_rank if distributed else None)
            if ns is not None:
                build_dir = os.path.join(build_dir, f"rank_{ns}")
            neff_path, key = cls._trace_and_compile(kernel, name, build_dir, additional_compiler_args,
                                                    use_cached_if_exists, target, args, kwargs)
        elif distributed:
            payload = [None, None]
            if dist_rank == 0:
                payload = list(cls._trace_and_compile(kernel, name, build_dir, additional_compiler_args,
                                                      use_cached_if_exists, target, args, kwargs))
            dist.broadcast_object_list(payload, src=0)
            neff_path, key = payload
        else:
            neff_path, key = cls._trace_and_compile(kernel, name, build_dir, additional_compiler_args,
                                                    use_cached_if_exists, target, args, kwargs)
        if use_cached_if_exists and key in _LOADED_KERNELS:
            return _LOADED_KERNELS[key]
        # collectives: on by default when running distributed; explicit rank / world win over the group's
        if cc_enabled is None:
            cc_enabled = distributed
        if cc_enabled:
            if rank_id is None and distributed:
                rank_id = dist_rank
            if world_size is None and distributed:
                world_size = dist.get_world_size()
            if rank_id is None or world_size is None:
                raise ValueError("rank_id and world_size are required when cc_enabled=True and no process group "
                                 "is initialised")
            if not (0 <= rank_id < world_size):
                raise ValueError(f"rank_id {rank_id} outside world of size {world_size}")
        else:
            rank_id, world_size = 0, 1
        if distributed and is_spmd:
            dist.barrier()        # the artifact must be visible on every rank's file system view
        loaded = cls.load_from_neff(neff_path, name=name, core_id=core_id, cc_enabled=cc_enabled, rank_id=rank_id,
                                    world_size=world_size)
        if use_cached_if_exists:
            _LOADED_KERNELS[key] = loaded
        return loaded

    @staticmethod
    def _trace_and_compile(kernel, name, build_dir, compiler_args, use_cached, target, args, kwargs):
        def as_numpy(a):
            if isinstance(a, DeviceTensor) or hasattr(a, "tensor_ref"):
                return np.zeros(a.shape, dtype=a.dtype)      # only shape / dtype matter for tracing
            return a

        np_args = [as_numpy(a) for a in args]
        np_kwargs = {k: as_numpy(v) for k, v in kwargs.items()}
        t0 = time.perf_counter()
        ir = kernel.specialize(*np_args, **np_kwargs)
        key = f"{name}_{ir.content_hash(compiler_args)}"
        out_dir = os.path.join(build_dir, key)
        neff_path = os.path.join(out_dir, f"{name}.cubin")
        if use_cached and os.path.exists(neff_path) and os.path.exists(os.path.join(out_dir, f"{name}.json")):
            logger.info("using cached kernel %s", neff_path)
            return neff_path, key
        compile_to_neff(ir, out_dir, f"{name}.cubin", additional_compiler_args=compiler_args, target=target)
        logger.info("compiled %s in %.2f s", name, time.perf_counter() - t0)
        return neff_path, key
