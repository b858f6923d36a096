"""Annotation aliases for kernel signatures (nkipy/src/nkipy/core/typing.py:5-10)."""
from typing import Any

import numpy as np

tensor = np.ndarray
mutable_tensor = np.ndarray


class mutable:          # noqa: N801  (marker used in annotations: the kernel writes this argument)
    pass


class immutable:        # noqa: N801
    pass
