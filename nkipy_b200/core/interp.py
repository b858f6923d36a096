"""NumPy evaluation of a captured `Graph`.

Second oracle of the frontend (the first is running the kernel function directly on
NumPy arrays, "CPU direct mode"): it executes exactly what was traced, so a tracing
or lowering bug shows up as a mismatch between direct mode and this interpreter,
without a GPU.  It also backs `stop_after`-style checks of the native compiler
passes and is the semantics reference for the CUDA code generator.  Collectives are
evaluated for one process under the reference's "all ranks hold the same data"
convention (nkipy/src/nkipy/core/ops/collectives.py:15-88) unless a `world` of
per-rank inputs is interpreted with `evaluate_spmd`.
"""

from __future__ import annotations

import math
from typing import Dict, List, Sequence

import numpy as np

from .ir import Graph, Node, Value

_UNARY = {
    "abs": np.abs, "neg": np.negative, "exp": np.exp, "log": np.log, "sqrt": np.sqrt, "sin": np.sin, "cos": np.cos,
    "tanh": np.tanh, "ceil": np.ceil, "floor": np.floor, "sign": np.sign, "round_even": np.rint, "copy": np.array,
}
_BINARY = {
    "add": np.add, "sub": np.subtract, "mul": np.multiply, "max": np.maximum, "min": np.minimum, "atan2": np.arctan2,
}
_COMPARE = {"EQ": np.equal, "NE": np.not_equal, "LT": np.less, "LE": np.less_equal, "GT": np.greater,
            "GE": np.greater_equal}
_REDUCE = {"sum": np.add, "max": np.maximum, "min": np.minimum, "prod": np.multiply, "and": np.logical_and,
           "or": np.logical_or}

_erf = np.vectorize(math.erf, otypes=[np.float64])


def _compute(x):
    """Low-precision floats are evaluated in float32 and rounded back, like the device does."""
    if x.dtype.kind == "f" and x.dtype.itemsize >= 4:
        return x
    if x.dtype.kind in "iub":
        return x
    return x.astype(np.float32)


def _dot(a, b, attrs, out_dtype):
    lb, rb, lc, rc = attrs["lhs_batch"], attrs["rhs_batch"], attrs["lhs_contract"], attrs["rhs_contract"]
    lfree = [i for i in range(a.ndim) if i not in lb and i not in lc]
    rfree = [i for i in range(b.ndim) if i not in rb and i not in rc]
    at = np.transpose(a, list(lb) + lfree + list(lc))
    bt = np.transpose(b, list(rb) + list(rc) + rfree)
    bshape = [a.shape[i] for i in lb]
    m = int(np.prod([a.shape[i] for i in lfree], dtype=np.int64))
    k = int(np.prod([a.shape[i] for i in lc], dtype=np.int64))
    n = int(np.prod([b.shape[i] for i in rfree], dtype=np.int64))
    nb = int(np.prod(bshape, dtype=np.int64))
    acc = np.float64 if a.dtype == np.float64 else (np.float32 if a.dtype.kind == "f" or a.dtype.kind == "V"
                                                    else a.dtype)
    a3 = at.reshape(nb, m, k).astype(acc)
    b3 = bt.reshape(nb, k, n).astype(acc)
    out = np.matmul(a3, b3)
    shape = bshape + [a.shape[i] for i in lfree] + [b.shape[i] for i in rfree]
    return out.reshape(shape).astype(out_dtype)


def _conv(x, w, b, attrs, out_dtype):
    nsp = x.ndim - 2
    stride, pad, dil, groups = attrs["stride"], attrs["padding"], attrs["dilation"], attrs["groups"]
    xp = np.pad(x.astype(np.float32), [(0, 0), (0, 0)] + [(p, p) for p in pad])
    N, C = x.shape[:2]
    O = w.shape[0]
    cg, og = C // groups, O // groups
    out_sp = [(xp.shape[2 + i] - ((w.shape[2 + i] - 1) * dil[i] + 1)) // stride[i] + 1 for i in range(nsp)]
    out = np.zeros([N, O] + out_sp, dtype=np.float32)
    wf = w.astype(np.float32)
    for g in range(groups):
        xs = xp[:, g * cg:(g + 1) * cg]
        ws = wf[g * og:(g + 1) * og]
        for kidx in np.ndindex(*w.shape[2:]):
            sl = [slice(None), slice(None)]
            for i in range(nsp):
                start = kidx[i] * dil[i]
                sl.append(slice(start, start + (out_sp[i] - 1) * stride[i] + 1, stride[i]))
            patch = xs[tuple(sl)]                                  # [N, cg, *out_sp]
            wk = ws[(slice(None), slice(None)) + kidx]             # [og, cg]
            out[:, g * og:(g + 1) * og] += np.einsum("nc...,oc->no...", patch, wk)
    if b is not None:
        out += b.astype(np.float32).reshape([1, O] + [1] * nsp)
    return out.astype(out_dtype)


def _eval_loop(n: Node, ins: List[np.ndarray]) -> List[np.ndarray]:
    from .ir import loop_body

    body = loop_body(n)
    nc = int(n.attrs["num_carried"])
    carried, captured = list(ins[:nc]), list(ins[nc:])
    for i in range(int(n.attrs["lower"]), int(n.attrs["upper"]), int(n.attrs.get("step", 1))):
        outs = evaluate(body, [np.asarray(i, dtype=np.int32)] + carried + captured)
        # results of bool dtype come back as uint8 from `evaluate`; carried values keep their dtype
        carried = [np.asarray(o).astype(c.dtype) for o, c in zip(outs, carried)]
    return carried


def _eval_node(n: Node, ins: List[np.ndarray], world: int = 1) -> List[np.ndarray]:
    op, a = n.opcode, n.attrs
    if op == "loop":
        return _eval_loop(n, ins)
    odt = n.outputs[0].dtype
    if op in _UNARY:
        return [np.asarray(_UNARY[op](_compute(ins[0]))).astype(odt)]
    if op == "rsqrt":
        return [(1.0 / np.sqrt(_compute(ins[0]))).astype(odt)]
    if op == "erf":
        return [_erf(ins[0].astype(np.float64)).astype(odt)]
    if op == "not":
        return [np.logical_not(ins[0]) if ins[0].dtype == np.bool_ else np.invert(ins[0])]
    if op == "is_finite":
        return [np.isfinite(_compute(ins[0]))]
    if op in _BINARY:
        return [np.asarray(_BINARY[op](_compute(ins[0]), _compute(ins[1]))).astype(odt)]
    if op == "div":
        x, y = ins
        if odt.kind in "iu":
            with np.errstate(divide="ignore"):
                q = np.trunc(x.astype(np.float64) / np.where(y == 0, 1, y).astype(np.float64))
            return [q.astype(odt)]
        with np.errstate(divide="ignore", invalid="ignore"):
            return [(_compute(x) / _compute(y)).astype(odt)]
    if op == "pow":
        with np.errstate(all="ignore"):
            return [np.power(_compute(ins[0]), _compute(ins[1])).astype(odt)]
    if op == "rem":
        with np.errstate(all="ignore"):
            return [np.fmod(_compute(ins[0]), _compute(ins[1])).astype(odt)]
    if op in ("and", "or", "xor"):
        fn = {"and": (np.logical_and, np.bitwise_and), "or": (np.logical_or, np.bitwise_or),
              "xor": (np.logical_xor, np.bitwise_xor)}[op]
        return [fn[0](ins[0], ins[1]) if odt == np.bool_ else fn[1](ins[0], ins[1])]
    if op == "compare":
        return [_COMPARE[a["direction"]](_compute(ins[0]), _compute(ins[1]))]
    if op == "select":
        return [np.where(ins[0], ins[1], ins[2])]
    if op == "convert":
        x = ins[0]
        if odt == np.bool_:
            return [x != 0]
        if odt.kind in "iu" and x.dtype.kind not in "iub":
            with np.errstate(invalid="ignore"):
                return [np.trunc(x.astype(np.float64)).astype(odt)]
        return [x.astype(odt)]
    if op == "broadcast":
        x = ins[0]
        shape, dims = a["shape"], a["dims"]
        expanded = [1] * len(shape)
        for i, d in enumerate(dims):
            expanded[d] = x.shape[i]
        return [np.broadcast_to(x.reshape(expanded), shape).copy()]
    if op == "reshape":
        return [ins[0].reshape(a["shape"])]
    if op == "transpose":
        return [np.ascontiguousarray(np.transpose(ins[0], a["perm"]))]
    if op == "slice":
        sl = tuple(slice(s, l, st) for s, l, st in zip(a["start"], a["limit"], a["stride"]))
        return [ins[0][sl].copy()]
    if op == "concat":
        return [np.concatenate(ins, axis=a["axis"])]
    if op == "pad":
        x, v = ins
        return [np.pad(x, list(zip(a["low"], a["high"])), constant_values=v.reshape(()).astype(x.dtype))]
    if op == "iota":
        shape, dim = a["shape"], a["dim"]
        ar = np.arange(shape[dim]).astype(odt)
        view = [1] * len(shape)
        view[dim] = shape[dim]
        return [np.broadcast_to(ar.reshape(view), shape).copy()]
    if op == "constant":
        return [np.array(a["value"])]
    if op == "reduce":
        x = ins[0]
        axes = tuple(a["axes"])
        kind = a["kind"]
        if kind in ("and", "or"):
            return [_REDUCE[kind].reduce(x.astype(bool), axis=axes).astype(odt)] if axes else [x.copy()]
        if not axes:
            return [x.copy()]
        xc = _compute(x)
        return [np.asarray(_REDUCE[kind].reduce(xc, axis=axes)).astype(odt)]
    if op == "dot":
        return [_dot(ins[0], ins[1], a, odt)]
    if op == "softmax":
        x = ins[0].astype(np.float32)
        e = np.exp(x - x.max(axis=-1, keepdims=True))
        return [(e / e.sum(axis=-1, keepdims=True)).astype(odt)]
    if op == "rms_norm":
        x = ins[0].astype(np.float32)
        y = x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + np.float32(a["eps"]))
        if len(ins) > 1:
            y = y * ins[1].astype(np.float32)
        return [y.astype(odt)]
    if op == "conv":
        return [_conv(ins[0], ins[1], ins[2] if len(ins) > 2 else None, a, odt)]
    if op == "take":
        idx = ins[1].astype(np.int64)
        dim = ins[0].shape[a["axis"]]
        idx = np.where(idx < 0, idx + dim, idx)
        return [np.take(ins[0], np.clip(idx, 0, dim - 1), axis=a["axis"])]
    if op == "take_along_axis":
        idx = ins[1].astype(np.int64)
        dim = ins[0].shape[a["axis"]]
        idx = np.where(idx < 0, idx + dim, idx)
        return [np.take_along_axis(ins[0], np.clip(idx, 0, dim - 1), axis=a["axis"])]
    if op == "scatter_along_axis":
        x, idx, upd = ins
        out = x.copy()
        sl = [slice(None)] * x.ndim
        sl[a["axis"]] = idx.astype(np.int64)
        out[tuple(sl)] = upd
        return [out]
    if op == "put_along_axis":
        x, idx, upd = ins
        out = x.copy()
        np.put_along_axis(out, idx.astype(np.int64), upd, axis=a["axis"])
        return [out]
    if op == "update_slice":
        x, upd = ins
        out = x.copy()
        sl = tuple(slice(s, s + (d - 1) * st + 1, st) for s, st, d in zip(a["start"], a["stride"], upd.shape))
        out[sl] = upd
        return [out]
    if op == "dynamic_update_slice":
        x, upd = ins[0], ins[1]
        starts = [int(np.clip(int(s.reshape(())), 0, x.shape[i] - upd.shape[i])) for i, s in enumerate(ins[2:])]
        out = x.copy()
        out[tuple(slice(s, s + d) for s, d in zip(starts, upd.shape))] = upd
        return [out]
    if op == "dynamic_slice":
        x = ins[0]
        sizes = a["sizes"]
        starts = [int(np.clip(int(s.reshape(())), 0, x.shape[i] - sizes[i])) for i, s in enumerate(ins[1:])]
        return [x[tuple(slice(s, s + d) for s, d in zip(starts, sizes))].copy()]
    if op == "topk":
        x = _compute(ins[0])
        k = a["k"]
        order = np.argsort(-x, axis=-1, kind="stable")[..., :k]
        vals = np.take_along_axis(ins[0], order, axis=-1)
        return [vals, order.astype(np.uint32)]
    if op == "custom_call":
        fn = a.get("reference")
        if fn is None:
            raise NotImplementedError(f"custom_call {a.get('target')!r} has no CPU reference")
        res = fn(*ins)
        return list(res) if isinstance(res, (tuple, list)) else [res]
    # collectives under "every rank holds the same data"
    n_ranks = len((a.get("replica_groups") or [[0]])[0])
    if op == "all_reduce":
        x = ins[0]
        kind = a.get("op", "add")
        if kind == "add":
            return [(_compute(x) * n_ranks).astype(odt)]
        if kind == "multiply":
            return [np.power(_compute(x), n_ranks).astype(odt)]
        return [x.copy()]
    if op == "all_gather":
        return [np.concatenate([ins[0]] * n_ranks, axis=a["dim"])]
    if op == "reduce_scatter":
        x = ins[0]
        part = np.split(x, n_ranks, axis=a["dim"])[0]
        kind = a.get("op", "add")
        if kind == "add":
            return [(_compute(part) * n_ranks).astype(odt)]
        if kind == "multiply":
            return [np.power(_compute(part), n_ranks).astype(odt)]
        return [part.copy()]
    if op == "all_to_all":
        parts = np.split(ins[0], n_ranks, axis=a["split_dim"])
        return [np.concatenate([parts[0]] * n_ranks, axis=a["concat_dim"])]
    raise NotImplementedError(f"interpreter has no rule for opcode {op!r}")


def evaluate(graph: Graph, inputs: Sequence[np.ndarray]) -> List[np.ndarray]:
    """Run the graph on NumPy inputs (positional, one per parameter); returns the results."""
    if len(inputs) != len(graph.params):
        raise ValueError(f"graph {graph.name} takes {len(graph.params)} inputs, got {len(inputs)}")
    env: Dict[int, np.ndarray] = {}
    for p, x in zip(graph.params, inputs):
        x = np.asarray(x)
        if tuple(x.shape) != p.shape:
            raise ValueError(f"input {p.name}: expected shape {p.shape}, got {x.shape}")
        env[p.id] = x.astype(p.dtype, copy=False)
    for n in graph.nodes:
        outs = _eval_node(n, [env[v.id] for v in n.inputs])
        for v, o in zip(n.outputs, outs):
            o = np.asarray(o)
            if o.dtype != v.dtype:
                o = o.astype(v.dtype)
            if tuple(o.shape) != v.shape:
                raise AssertionError(f"{n.opcode}: interpreter produced {o.shape}, IR says {v.shape}")
            env[v.id] = o
    results = []
    for v in graph.results:
        r = env[v.id]
        results.append(r.astype(np.uint8) if r.dtype == np.bool_ else r)
    return results
