"""Catalogue of target NumPy operations and per-operation unit tests
(reference: tools/kernel_agent/ops.py:12-259)."""

from __future__ import annotations

from typing import Callable, Dict, List, Optional, Tuple

import numpy as np

from .executor import ExecutionResult, run_kernel

TARGET_OPS: Dict[str, List[str]] = {
    "binary": ["add", "subtract", "multiply", "divide", "power", "maximum", "minimum", "floor_divide", "mod",
               "bitwise_and", "bitwise_or", "bitwise_xor", "logical_and", "logical_or", "logical_xor"],
    "comparison": ["equal", "not_equal", "greater", "greater_equal", "less", "less_equal"],
    "unary": ["abs", "exp", "log", "sqrt", "square", "negative", "sign", "sin", "cos", "tan", "arctan", "tanh",
              "ceil", "floor", "rint", "trunc", "reciprocal", "logical_not"],
    "reduction": ["sum", "max", "min", "mean", "prod", "argmax", "argmin", "any", "all", "var", "std"],
    "linalg": ["matmul", "dot"],
    "transform": ["reshape", "transpose", "expand_dims", "squeeze", "concatenate", "stack", "broadcast_to", "repeat",
                  "tile", "flip", "swapaxes", "split"],
    "indexing": ["where", "take", "take_along_axis", "clip"],
    "creation": ["zeros_like", "ones_like", "full_like"],
}

_INT_OPS = {"bitwise_and", "bitwise_or", "bitwise_xor"}
_BOOL_OPS = {"logical_and", "logical_or", "logical_xor", "logical_not", "any", "all"}
_POSITIVE = {"log", "sqrt", "power", "reciprocal"}


def all_ops() -> List[Tuple[str, str]]:
    return [(cat, op) for cat, ops in TARGET_OPS.items() for op in ops]


def _inputs(op: str, shape, rng, n: int):
    arrs = []
    for _ in range(n):
        if op in _INT_OPS:
            arrs.append(rng.integers(0, 64, size=shape).astype(np.int32))
        elif op in _BOOL_OPS:
            arrs.append(rng.random(shape) > 0.5)
        elif op in _POSITIVE or op in ("floor_divide", "mod", "divide"):
            arrs.append((rng.random(shape) + 0.5).astype(np.float32))
        else:
            arrs.append(rng.standard_normal(shape).astype(np.float32))
    return arrs


def build_kernel(category: str, op: str, shape=(8, 16)) -> Optional[Tuple[Callable, list]]:
    """(kernel function, inputs) exercising `np.<op>`; None when the catalogue has no recipe."""
    rng = np.random.default_rng(abs(hash(op)) % (2 ** 31))
    f = getattr(np, op, None)
    if f is None:
        return None
    if category in ("binary", "comparison"):
        return (lambda a, b: f(a, b)), _inputs(op, shape, rng, 2)
    if category == "unary":
        return (lambda a: f(a)), _inputs(op, shape, rng, 1)
    if category == "reduction":
        if op in ("argmax", "argmin"):
            return (lambda a: f(a, axis=-1)), _inputs(op, shape, rng, 1)
        return (lambda a: f(a, axis=-1)), _inputs(op, shape, rng, 1)
    if category == "linalg":
        a = rng.standard_normal((shape[0], shape[1])).astype(np.float32)
        b = rng.standard_normal((shape[1], shape[0])).astype(np.float32)
        return (lambda x, y: f(x, y)), [a, b]
    x = rng.standard_normal(shape).astype(np.float32)
    recipes = {
        "reshape": lambda a: np.reshape(a, (shape[1], shape[0])),
        "transpose": lambda a: np.transpose(a, (1, 0)),
        "expand_dims": lambda a: np.expand_dims(a, 0),
        "squeeze": lambda a: np.squeeze(np.expand_dims(a, 0), 0),
        "concatenate": lambda a: np.concatenate([a, a], axis=0),
        "stack": lambda a: np.stack([a, a], axis=0),
        "broadcast_to": lambda a: np.broadcast_to(a[:1], shape) + 0.0,
        "repeat": lambda a: np.repeat(a, 2, axis=0),
        "tile": lambda a: np.tile(a, (2, 1)),
        "flip": lambda a: np.flip(a, axis=1),
        "swapaxes": lambda a: np.swapaxes(a, 0, 1),
        "split": lambda a: np.split(a, 2, axis=0)[1],
        "where": lambda a: np.where(a > 0, a, 0.5 * a),
        "take": lambda a: np.take(a, np.array([0, 2, 1]), axis=0),
        "take_along_axis": lambda a: np.take_along_axis(a, np.argsort(a, axis=-1)[:, :4], axis=-1)
        if hasattr(np, "argsort") else a,
        "clip": lambda a: np.clip(a, -0.5, 0.5),
        "zeros_like": lambda a: np.zeros_like(a) + a,
        "ones_like": lambda a: np.ones_like(a) * a,
        "full_like": lambda a: np.full_like(a, 2.0) * a,
    }
    if op == "take_along_axis":
        idx = rng.integers(0, shape[1], size=(shape[0], 4)).astype(np.int32)
        return (lambda a, i: np.take_along_axis(a, i, axis=-1)), [x, idx]
    if op in recipes:
        return recipes[op], [x]
    return None


def test_op(category: str, op: str, shape=(8, 16), use_gpu: Optional[bool] = None) -> Optional[ExecutionResult]:
    built = build_kernel(category, op, shape)
    if built is None:
        return None
    fn, inputs = built
    return run_kernel(fn, inputs, use_gpu=use_gpu)


def discover(use_gpu: Optional[bool] = None) -> Dict[str, Dict]:
    """Run every catalogue operation through the pipeline; returns op -> result dict."""
    out = {}
    for cat, op in all_ops():
        r = test_op(cat, op, use_gpu=use_gpu)
        out[f"{cat}.{op}"] = {"status": "no-recipe"} if r is None else dict(r.as_dict(), status="pass" if r.passed
                                                                          else "fail")
    return out
