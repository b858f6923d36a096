"""Device tensor with shape / dtype metadata on top of a raw runtime allocation
(spike/src/spike/spike_tensor.py:9-83 in the reference)."""

from __future__ import annotations

from typing import Optional, Tuple

import numpy as np

from .spike_singleton import get_spike_singleton


class SpikeTensor:
    def __init__(self, tensor_ref, shape: Tuple[int, ...], dtype, name: Optional[str] = None):
        self.tensor_ref = tensor_ref
        self.shape = tuple(int(s) for s in shape)
        self.dtype = np.dtype(dtype)
        self.name = name or getattr(tensor_ref, "name", "")

    @property
    def nbytes(self) -> int:
        return int(np.prod(self.shape, dtype=np.int64)) * self.dtype.itemsize

    @property
    def core_id(self) -> int:
        return self.tensor_ref.core_id

    @property
    def va(self) -> int:
        """Device address (usable with torch / ctypes kernels)."""
        return self.tensor_ref.va

    @classmethod
    def empty(cls, shape, dtype, name: Optional[str] = None, core_id: int = 0) -> "SpikeTensor":
        dtype = np.dtype(dtype)
        nbytes = int(np.prod(shape, dtype=np.int64)) * dtype.itemsize
        ref = get_spike_singleton().allocate_tensor(max(nbytes, 1), core_id, name or "")
        return cls(ref, shape, dtype, name)

    @classmethod
    def from_numpy(cls, array: np.ndarray, name: Optional[str] = None, core_id: int = 0) -> "SpikeTensor":
        shape = np.shape(array)                      # ascontiguousarray turns a 0-d array into shape (1,)
        array = np.ascontiguousarray(array)
        t = cls.empty(shape, array.dtype, name, core_id)
        if array.nbytes:
            get_spike_singleton().tensor_write(t.tensor_ref, array.view(np.uint8).reshape(-1), 0)
        return t

    def numpy(self) -> np.ndarray:
        flat = np.empty(int(np.prod(self.shape, dtype=np.int64)), dtype=self.dtype)    # 1-d: a 0-d array has no byte view
        if flat.nbytes:
            get_spike_singleton().tensor_read_to_buffer(self.tensor_ref, flat.view(np.uint8), 0)
        return flat.reshape(self.shape)

    def write_from_numpy(self, array: np.ndarray) -> None:
        """Overwrite the contents in place (no reallocation); sizes must match."""
        array = np.ascontiguousarray(array)
        if array.nbytes != self.nbytes:
            raise ValueError(f"size mismatch: tensor holds {self.nbytes} bytes, array has {array.nbytes}")
        if array.nbytes:
            get_spike_singleton().tensor_write(self.tensor_ref, array.view(np.uint8).reshape(-1), 0)

    def slice_bytes(self, offset: int, shape, dtype=None, name: Optional[str] = None) -> "SpikeTensor":
        dtype = np.dtype(dtype or self.dtype)
        nbytes = int(np.prod(shape, dtype=np.int64)) * dtype.itemsize
        ref = get_spike_singleton().slice_from_tensor(self.tensor_ref, offset, nbytes, name or "")
        return SpikeTensor(ref, shape, dtype, name)

    def free(self) -> None:
        get_spike_singleton().free_tensor(self.tensor_ref)

    def __repr__(self):
        return f"SpikeTensor(name={self.name!r}, shape={self.shape}, dtype={self.dtype})"
