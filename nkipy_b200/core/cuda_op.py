"""Hand-written CUDA kernels as operations of traced programs.

Counterpart of the reference's NKI custom-kernel hook (nkipy/src/nkipy/core/nki_op.py:304-884:
calling an `@nki.jit` kernel while tracing emits a custom-call with operand -> output
aliasing).  Here a custom op is a piece of CUDA C++ source with one ``extern "C" __global__``
entry point plus a NumPy reference implementation:

    op = cuda_custom_op(name="scale_add", source=SRC, entry="scale_add_kernel",
                        output_specs=[((128, 512), "f32")], grid=(256,), block=(256,),
                        reference=lambda a, b: 2 * a + b, aliases={0: 0})
    y = op(a, b)          # in a traced kernel: a custom_call node; on NumPy arrays: the reference

While tracing the call becomes a `custom_call` node carrying the source, launch geometry
and alias map (output index -> operand index; an aliased operand that is a kernel parameter
is marked mutated).  In CPU direct mode and in the IR interpreter the reference runs.  The
code generator emits the source verbatim into the translation unit and one launch whose
arguments are the operand pointers followed by the output pointers.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np

from .backend import get_backend
from .dtypes import dtype_from_name, dtype_name


@dataclass
class CudaCustomOp:
    name: str
    source: str
    entry: str
    output_specs: List[Tuple[Tuple[int, ...], str]]
    grid: Tuple[int, ...] = (1,)
    block: Tuple[int, ...] = (256,)
    smem: int = 0
    reference: Optional[Callable] = None
    aliases: Dict[int, int] = field(default_factory=dict)   # output index -> operand index
    has_collectives: bool = False

    @classmethod
    def from_kernel_builder(cls, kernel_builder: Callable[..., str], *, name: str, entry: str, input_specs,
                            output_specs, grid, block, reference=None, aliases=None, **builder_kwargs):
        """Build the CUDA source from a Python function of the input specs (mirrors the
        reference's builder-style custom ops)."""
        src = kernel_builder(input_specs=input_specs, output_specs=output_specs, **builder_kwargs)
        return cls(name, src, entry, [(tuple(s), d) for s, d in output_specs], tuple(grid), tuple(block), 0,
                   reference, dict(aliases or {}))

    def __call__(self, *operands):
        if get_backend() == "cpu":
            if self.reference is None:
                raise NotImplementedError(f"custom op '{self.name}' has no CPU reference implementation")
            res = self.reference(*operands)
            for out_idx, op_idx in self.aliases.items():
                val = res[out_idx] if isinstance(res, (tuple, list)) else res
                np.copyto(operands[op_idx], val)
            return res
        from .ops import _ir_impls as I

        vals = [I.as_value(o) for o in operands]
        attrs = {
            "target": self.name, "entry": self.entry, "source": self.source,
            "grid": list(self.grid) + [1] * (3 - len(self.grid)), "block": list(self.block) + [1] * (3 - len(self.block)),
            "smem": int(self.smem), "aliases": {str(k): int(v) for k, v in self.aliases.items()},
            "has_collectives": bool(self.has_collectives),
            "result_types": [[list(s), d if isinstance(d, str) else dtype_name(d)] for s, d in self.output_specs],
        }
        if self.reference is not None:
            attrs["reference"] = self.reference
        outs = I.G().add_node("custom_call", vals, attrs)
        refs = [I.wrap(o) for o in outs]
        for out_idx, op_idx in self.aliases.items():
            target = operands[op_idx]
            if hasattr(target, "_rebind"):
                target._rebind(refs[out_idx])
        return refs[0] if len(refs) == 1 else tuple(refs)


def cuda_custom_op(name: str, source: str, entry: str, output_specs: Sequence[Tuple[Sequence[int], str]],
                   grid: Sequence[int] = (1,), block: Sequence[int] = (256,), smem: int = 0,
                   reference: Optional[Callable] = None, aliases: Optional[Dict[int, int]] = None,
                   input_specs=None, has_collectives: bool = False) -> CudaCustomOp:
    if not output_specs:
        raise ValueError("a custom op needs at least one output spec")
    for s, d in output_specs:
        dtype_from_name(d) if isinstance(d, str) else np.dtype(d)
    return CudaCustomOp(name, source, entry, [(tuple(s), d) for s, d in output_specs], tuple(grid), tuple(block), smem,
                        reference, dict(aliases or {}), has_collectives)
