"""Hand-written kernels behind one handle that works under every tracing backend.

The reference has two ways of putting a hand kernel into a traced program (nkipy/src/nkipy/core/nki_op.py): a
kernel that was traced ahead of time for fixed operand shapes (`wrap_nki_kernel` -> `NKICustomOp`, lines 603-774) and
a handle that carries both that form and a builder function for the nkigen backend (`nki_custom_op` ->
`NKICustomOpHandle`, lines 800-884).  On this target a hand kernel is CUDA C++ source with one `extern "C"
__global__` entry, so the two forms become

* a kernel whose source is already written (`CudaCustomOp`, or `wrap_cuda_kernel` which also pins operand shapes), and
* a *kernel builder*: a Python function of the operand and result specs that returns the source (and, optionally, the
  launch geometry), called once the specs are known.

`nki_custom_op(nki_kernel=..., kernel_builder=..., input_specs=..., output_specs=...)` accepts either or both and
returns a handle.  Called while tracing, the handle emits a `custom_call` node: under the "hlo" backend it prefers the
pre-written kernel, under "nkigen" the builder, and falls back to the other one because both lower to the same node
here.  Called on NumPy arrays it runs the kernel's NumPy reference when it has one and raises otherwise (the
reference's handle always raises there).  Operand count, shapes and dtypes are checked against `input_specs`.
"""

from __future__ import annotations

from typing import Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np

from .backend import get_backend
from .cuda_op import CudaCustomOp, cuda_custom_op
from .dtypes import dtype_from_name, dtype_name

CUDA_AVAILABLE = True          # the custom-op frontend itself needs no toolchain until compile time
BETA3_COMPILE_MODES = ()       # no alternative kernel frontends on this target

Spec = Tuple[Tuple[int, ...], str]


def _norm_specs(specs) -> List[Spec]:
    out = []
    for shape, dt in specs:
        name = dt if isinstance(dt, str) else dtype_name(np.dtype(dt))
        dtype_from_name(name)                      # unknown names fail here, not at code generation
        out.append((tuple(int(d) for d in shape), name))
    return out


def _spec_of(x) -> Spec:
    return tuple(int(d) for d in x.shape), dtype_name(np.dtype(x.dtype))


def _check_operands(what: str, specs: Sequence[Spec], operands) -> None:
    if len(operands) != len(specs):
        raise ValueError(f"{what} takes {len(specs)} operand(s), got {len(operands)}")
    for i, (want, got) in enumerate(zip(specs, (_spec_of(o) for o in operands))):
        if want != got:
            raise ValueError(f"{what}: operand {i} is {got[1]}{list(got[0])}, the kernel was built for "
                             f"{want[1]}{list(want[0])}")


class NKICustomOp:
    """A pre-written kernel pinned to the operand shapes it was written for (what `wrap_cuda_kernel` returns)."""

    def __init__(self, kernel: CudaCustomOp, operands: Iterable, grid: Optional[Sequence[int]] = (),
                 block: Optional[Sequence[int]] = ()):
        if not isinstance(kernel, CudaCustomOp):
            raise TypeError("kernel must be a CudaCustomOp (source, entry point and result specs)")
        self.input_specs = [_spec_of(o) for o in operands]
        self.kernel = kernel
        if grid or block:
            self.kernel = CudaCustomOp(kernel.name, kernel.source, kernel.entry, kernel.output_specs,
                                       tuple(grid) or kernel.grid, tuple(block) or kernel.block, kernel.smem,
                                       kernel.reference, dict(kernel.aliases), kernel.has_collectives)

    @property
    def config(self) -> Dict:
        k = self.kernel
        return {"target": k.name, "entry": k.entry, "grid": list(k.grid), "block": list(k.block), "smem": k.smem,
                "aliases": dict(k.aliases), "has_collectives": k.has_collectives,
                "input_specs": list(self.input_specs), "output_specs": list(k.output_specs)}

    def __call__(self, *operands):
        _check_operands(f"custom op '{self.kernel.name}'", self.input_specs, operands)
        return self.kernel(*operands)


def wrap_cuda_kernel(kernel: CudaCustomOp, operands: Iterable, grid: Optional[Sequence[int]] = (),
                     block: Optional[Sequence[int]] = (), **ignored) -> NKICustomOp:
    """Pin a hand-written kernel to example operands (only their shape and dtype are used); `grid` / `block`
    override the kernel's own launch geometry.  Keyword arguments that select a kernel frontend or a platform in the
    reference's signature are accepted and have no meaning here."""
    return NKICustomOp(kernel, operands, grid, block)


wrap_nki_kernel = wrap_cuda_kernel


class NKICustomOpHandle:
    """What `nki_custom_op` returns; see the module docstring for how a call is dispatched."""

    def __init__(self, nki_kernel, kernel_builder, input_specs, output_specs, launch: Dict):
        self._kernel = nki_kernel
        self._builder = kernel_builder
        self.input_specs = _norm_specs(input_specs) if input_specs is not None else None
        self.output_specs = _norm_specs(output_specs) if output_specs is not None else None
        self._launch = launch
        self._built: Optional[CudaCustomOp] = None

    # -- the builder form, realised once
    def _from_builder(self) -> CudaCustomOp:
        if self._built is None:
            made = self._builder(input_specs=self.input_specs, output_specs=self.output_specs,
                                 **self._launch.get("builder_kwargs", {}))
            geometry = {}
            if isinstance(made, dict):
                geometry = {k: made[k] for k in ("entry", "grid", "block", "smem") if k in made}
                made = made["source"]
            if not isinstance(made, str):
                raise TypeError("a kernel builder returns CUDA source, or a dict with 'source' and launch geometry")
            name = self._launch.get("name") or getattr(self._builder, "__name__", "custom")
            entry = geometry.get("entry") or self._launch.get("entry") or name
            self._built = cuda_custom_op(
                name=name, source=made, entry=entry, output_specs=self.output_specs,
                grid=geometry.get("grid", self._launch.get("grid", (1,))),
                block=geometry.get("block", self._launch.get("block", (256,))),
                smem=geometry.get("smem", self._launch.get("smem", 0)), reference=self._launch.get("reference"),
                aliases=self._launch.get("aliases"), has_collectives=self._launch.get("has_collectives", False))
        return self._built

    def _reference(self) -> Optional[Callable]:
        if self._launch.get("reference") is not None:
            return self._launch["reference"]
        k = self._kernel.kernel if isinstance(self._kernel, NKICustomOp) else self._kernel
        return getattr(k, "reference", None)

    def __call__(self, *operands):
        backend = get_backend()
        if self.input_specs is not None:
            _check_operands("custom op", self.input_specs, operands)
        if backend == "cpu" and self._reference() is None:
            raise RuntimeError("this custom op is not supported on backend 'cpu': it has no NumPy reference; "
                               "call it inside a traced kernel")
        order = [self._kernel, self._builder] if backend == "hlo" else [self._builder, self._kernel]
        chosen = next(c for c in order if c is not None)
        if chosen is self._builder:
            return self._from_builder()(*operands)
        return chosen(*operands)


def nki_custom_op(*, nki_kernel=None, kernel_builder: Optional[Callable] = None, input_specs=None, output_specs=None,
                  **launch) -> NKICustomOpHandle:
    """A hand kernel usable under every backend.

    `nki_kernel` is a pre-written kernel (`CudaCustomOp` or the result of `wrap_cuda_kernel`); `kernel_builder` is a
    function `(input_specs, output_specs, **builder_kwargs) -> source | {"source", "entry", "grid", "block", "smem"}`
    and needs both spec lists.  `launch` may carry `name`, `entry`, `grid`, `block`, `smem`, `reference`, `aliases`,
    `has_collectives` and `builder_kwargs` for the builder form."""
    if nki_kernel is None and kernel_builder is None:
        raise ValueError("At least one of nki_kernel or kernel_builder is needed")
    if kernel_builder is not None and (input_specs is None or output_specs is None):
        raise ValueError("kernel_builder needs input_specs and output_specs")
    if nki_kernel is not None and not isinstance(nki_kernel, (CudaCustomOp, NKICustomOp)):
        raise TypeError("nki_kernel must be a CudaCustomOp or a wrapped kernel")
    unknown = set(launch) - {"name", "entry", "grid", "block", "smem", "reference", "aliases", "has_collectives",
                             "builder_kwargs"}
    if unknown:
        raise TypeError(f"unknown argument(s) {sorted(unknown)}")
    return NKICustomOpHandle(nki_kernel, kernel_builder, input_specs, output_specs, launch)


NKIOp = NKICustomOpHandle
