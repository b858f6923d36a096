"""Device tensor with NumPy and PyTorch interop
(nkipy/src/nkipy/runtime/device_tensor.py:1-103 in the reference)."""

from __future__ import annotations

from typing import Optional

import numpy as np

from ..core.dtypes import bfloat16, float8_e4m3, float8_e5m2
from ..spike.spike_tensor import SpikeTensor


def _torch_maps():
    import torch

    t2n = {torch.float16: np.dtype(np.float16), torch.float32: np.dtype(np.float32), torch.bfloat16: bfloat16,
           torch.float8_e5m2: float8_e5m2, torch.float8_e4m3fn: float8_e4m3, torch.int32: np.dtype(np.int32),
           torch.uint32: np.dtype(np.uint32), torch.int8: np.dtype(np.int8), torch.uint8: np.dtype(np.uint8),
           torch.int16: np.dtype(np.int16), torch.bool: np.dtype(np.bool_), torch.int64: np.dtype(np.int64),
           torch.float64: np.dtype(np.float64)}
    n2t = {v: k for k, v in t2n.items()}
    return t2n, n2t


class DeviceTensor(SpikeTensor):
    """A `SpikeTensor` that converts from / to torch tensors as well."""

    @classmethod
    def from_torch(cls, tensor, name: Optional[str] = None, core_id: int = 0) -> "DeviceTensor":
        import torch

        t2n, _ = _torch_maps()
        if tensor.dtype not in t2n:
            raise TypeError(f"unsupported torch dtype {tensor.dtype}")
        src = tensor.detach().contiguous().cpu()
        raw = src.view(torch.uint8).numpy() if src.numel() else np.empty((0,), dtype=np.uint8)
        out = cls.empty(tuple(src.shape), t2n[tensor.dtype], name, core_id)
        if raw.size:
            from ..spike.spike_singleton import get_spike_singleton

            get_spike_singleton().tensor_write(out.tensor_ref, raw.reshape(-1), 0)
        return out

    def torch(self):
        import torch

        _, n2t = _torch_maps()
        dt = n2t[self.dtype]
        raw = np.empty((self.nbytes,), dtype=np.uint8)
        if raw.size:
            from ..spike.spike_singleton import get_spike_singleton

            get_spike_singleton().tensor_read_to_buffer(self.tensor_ref, raw, 0)
        return torch.from_numpy(raw).view(dt).reshape(self.shape)

    def write_from_torch(self, tensor) -> None:
        """Overwrite in place from a torch tensor (no reallocation); byte sizes must match."""
        import torch

        src = tensor.detach().contiguous().cpu()
        if src.numel() * src.element_size() != self.nbytes:
            raise ValueError(f"size mismatch: tensor holds {self.nbytes} bytes, source has "
                             f"{src.numel() * src.element_size()}")
        if self.nbytes:
            from ..spike.spike_singleton import get_spike_singleton

            get_spike_singleton().tensor_write(self.tensor_ref, src.view(torch.uint8).numpy().reshape(-1), 0)
