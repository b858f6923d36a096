"""Tensor IR captured by the tracing frontend.

A `Graph` is a flat SSA list of `Node`s over statically shaped `Value`s.  It plays
the role of the reference's HLOModule (nkipy/src/nkipy/core/backend/hlo.py:330-1000):
parameters, operations, results, input/output aliases, source locations, and a
content hash used as the compile-cache key — but it is a compact IR of its own with
a line-oriented text form that the native compiler (csrc/compiler) parses, instead
of an XLA protobuf.

Opcode vocabulary (shape rules in `_INFER`):
  elementwise  add sub mul div pow max min rem atan2 and or xor | abs neg exp log sqrt rsqrt sin cos
               tanh ceil floor sign not round_even is_finite erf | compare select convert
  shape        broadcast reshape transpose slice concat pad copy iota constant
  reduce       reduce {kind: sum max min prod and or, axes}
  linalg       dot {lhs_batch rhs_batch lhs_contract rhs_contract}, conv {...}
  indexing     take take_along_axis scatter_along_axis put_along_axis update_slice dynamic_update_slice
               dynamic_slice
  multi-result topk custom_call
  collectives  all_gather all_reduce reduce_scatter all_to_all
"""

from __future__ import annotations

import base64
import hashlib
import json
import re
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np

from .dtypes import dtype_from_name, dtype_name

Shape = Tuple[int, ...]


@dataclass(eq=False)
class Value:
    id: int
    shape: Shape
    dtype: np.dtype
    name: str = ""
    producer: Optional["Node"] = None
    index: int = 0          # which result of the producer

    @property
    def ndim(self) -> int:
        return len(self.shape)

    @property
    def size(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n

    def type_str(self) -> str:
        return f"{dtype_name(self.dtype)}[{','.join(str(s) for s in self.shape)}]"

    def __repr__(self) -> str:
        return f"%{self.id}:{self.type_str()}"


@dataclass(eq=False)
class Node:
    opcode: str
    inputs: List[Value]
    attrs: Dict[str, Any]
    outputs: List[Value] = field(default_factory=list)
    loc: Optional[Tuple[str, int]] = None


ELEMENTWISE_BINARY = {"add", "sub", "mul", "div", "pow", "max", "min", "rem", "atan2", "and", "or", "xor"}
ELEMENTWISE_UNARY = {"abs", "neg", "exp", "log", "sqrt", "rsqrt", "sin", "cos", "tanh", "ceil", "floor", "sign", "not",
                     "round_even", "is_finite", "erf", "copy"}
COLLECTIVES = {"all_gather", "all_reduce", "reduce_scatter", "all_to_all"}


class IRError(ValueError):
    pass


def _norm_axis(axis: int, ndim: int) -> int:
    if axis < -ndim or axis >= ndim:
        raise np.exceptions.AxisError(axis, ndim)
    return axis % ndim


# --------------------------------------------------------------------------- shape inference
def _same(ins, attrs):
    return [(ins[0].shape, ins[0].dtype)]


def _binary(ins, attrs):
    a, b = ins
    if a.shape != b.shape:
        raise IRError(f"elementwise operands differ in shape: {a.shape} vs {b.shape}")
    if a.dtype != b.dtype:
        raise IRError(f"elementwise operands differ in dtype: {a.dtype} vs {b.dtype}")
    return [(a.shape, a.dtype)]


def _compare(ins, attrs):
    a, b = ins
    if a.shape != b.shape or a.dtype != b.dtype:
        raise IRError(f"compare operands differ: {a} vs {b}")
    if attrs["direction"] not in ("EQ", "NE", "LT", "LE", "GT", "GE"):
        raise IRError(f"bad compare direction {attrs['direction']}")
    return [(a.shape, np.dtype(np.bool_))]


def _select(ins, attrs):
    p, a, b = ins
    if p.dtype != np.bool_ or p.shape != a.shape or a.shape != b.shape or a.dtype != b.dtype:
        raise IRError("select needs pred/on_true/on_false of one shape, pred bool")
    return [(a.shape, a.dtype)]


def _convert(ins, attrs):
    return [(ins[0].shape, dtype_from_name(attrs["dtype"]))]


def _broadcast(ins, attrs):
    shape, dims = tuple(attrs["shape"]), tuple(attrs["dims"])
    x = ins[0]
    if len(dims) != x.ndim:
        raise IRError("broadcast dims must map every operand dim")
    for i, d in enumerate(dims):
        if x.shape[i] != 1 and x.shape[i] != shape[d]:
            raise IRError(f"cannot broadcast {x.shape} to {shape} via dims {dims}")
    return [(shape, x.dtype)]


def _reshape(ins, attrs):
    shape = tuple(attrs["shape"])
    if int(np.prod(shape, dtype=np.int64)) != ins[0].size:
        raise IRError(f"cannot reshape {ins[0].shape} to {shape}")
    return [(shape, ins[0].dtype)]


def _transpose(ins, attrs):
    perm = tuple(attrs["perm"])
    x = ins[0]
    if sorted(perm) != list(range(x.ndim)):
        raise IRError(f"bad permutation {perm} for rank {x.ndim}")
    return [(tuple(x.shape[p] for p in perm), x.dtype)]


def _slice(ins, attrs):
    x = ins[0]
    out = []
    for s, l, st, dim in zip(attrs["start"], attrs["limit"], attrs["stride"], x.shape):
        if not (0 <= s <= l <= dim) or st < 1:
            raise IRError(f"bad slice [{s}:{l}:{st}] of dim {dim}")
        out.append((l - s + st - 1) // st)
    return [(tuple(out), x.dtype)]


def _concat(ins, attrs):
    axis = attrs["axis"]
    base = list(ins[0].shape)
    total = 0
    for v in ins:
        if v.dtype != ins[0].dtype or v.ndim != len(base):
            raise IRError("concat operands must share dtype and rank")
        for i, (a, b) in enumerate(zip(v.shape, base)):
            if i != axis and a != b:
                raise IRError("concat operands differ outside the concat axis")
        total += v.shape[axis]
    base[axis] = total
    return [(tuple(base), ins[0].dtype)]


def _pad(ins, attrs):
    x = ins[0]
    return [(tuple(d + lo + hi for d, lo, hi in zip(x.shape, attrs["low"], attrs["high"])), x.dtype)]


def _iota(ins, attrs):
    return [(tuple(attrs["shape"]), dtype_from_name(attrs["dtype"]))]


def _constant(ins, attrs):
    v = attrs["value"]
    return [(tuple(v.shape), v.dtype)]


def _reduce(ins, attrs):
    x = ins[0]
    axes = sorted(set(attrs["axes"]))
    if attrs["kind"] not in ("sum", "max", "min", "prod", "and", "or"):
        raise IRError(f"bad reduce kind {attrs['kind']}")
    return [(tuple(d for i, d in enumerate(x.shape) if i not in axes), x.dtype)]


def _dot(ins, attrs):
    a, b = ins
    lb, rb = attrs["lhs_batch"], attrs["rhs_batch"]
    lc, rc = attrs["lhs_contract"], attrs["rhs_contract"]
    if a.dtype != b.dtype:
        raise IRError("dot operands differ in dtype")
    for i, j in zip(lb, rb):
        if a.shape[i] != b.shape[j]:
            raise IRError("dot batch dims differ")
    for i, j in zip(lc, rc):
        if a.shape[i] != b.shape[j]:
            raise IRError(f"dot contracting dims differ: {a.shape} x {b.shape}")
    batch = [a.shape[i] for i in lb]
    lfree = [d for i, d in enumerate(a.shape) if i not in lb and i not in lc]
    rfree = [d for i, d in enumerate(b.shape) if i not in rb and i not in rc]
    return [(tuple(batch + lfree + rfree), a.dtype)]


def _take(ins, attrs):
    x, idx = ins
    axis = attrs["axis"]
    return [(x.shape[:axis] + idx.shape + x.shape[axis + 1:], x.dtype)]


def _take_along(ins, attrs):
    x, idx = ins
    if idx.ndim != x.ndim:
        raise IRError("take_along_axis needs indices of the operand's rank")
    return [(idx.shape, x.dtype)]


def _scatter_like(ins, attrs):
    return [(ins[0].shape, ins[0].dtype)]


def _dynamic_slice(ins, attrs):
    return [(tuple(attrs["sizes"]), ins[0].dtype)]


def _topk(ins, attrs):
    x = ins[0]
    shape = x.shape[:-1] + (attrs["k"],)
    return [(shape, x.dtype), (shape, np.dtype(np.uint32))]


def _custom_call(ins, attrs):
    return [(tuple(s), dtype_from_name(d)) for s, d in attrs["result_types"]]


def _conv(ins, attrs):
    x, w = ins[0], ins[1]
    nsp = x.ndim - 2
    out = [x.shape[0], w.shape[0]]
    for i in range(nsp):
        eff = (w.shape[2 + i] - 1) * attrs["dilation"][i] + 1
        out.append((x.shape[2 + i] + 2 * attrs["padding"][i] - eff) // attrs["stride"][i] + 1)
    return [(tuple(out), x.dtype)]


def _group_size(attrs) -> int:
    groups = attrs.get("replica_groups") or [[0]]
    return len(groups[0])


def _all_gather(ins, attrs):
    x = ins[0]
    s = list(x.shape)
    s[attrs["dim"]] *= _group_size(attrs)
    return [(tuple(s), x.dtype)]


def _reduce_scatter(ins, attrs):
    x = ins[0]
    s = list(x.shape)
    n = _group_size(attrs)
    if s[attrs["dim"]] % n:
        raise IRError("reduce_scatter dim must divide by the group size")
    s[attrs["dim"]] //= n
    return [(tuple(s), x.dtype)]


def _all_to_all(ins, attrs):
    x = ins[0]
    s = list(x.shape)
    n = _group_size(attrs)
    if s[attrs["split_dim"]] % n:
        raise IRError("all_to_all split dim must divide by the group size")
    s[attrs["split_dim"]] //= n
    s[attrs["concat_dim"]] *= n
    return [(tuple(s), x.dtype)]


def _loop(ins, attrs):
    """Counted loop: inputs = carried initial values then captured values; attrs lower / upper / step,
    num_carried and `body` = text of a nested graph with parameters (index i32[], carried..., captured...)
    whose results are the next carried values.  Outputs: the carried values after the last iteration."""
    n = int(attrs["num_carried"])
    if n > len(ins):
        raise IRError("loop: more carried values than inputs")
    return [(v.shape, v.dtype) for v in ins[:n]]


_INFER = {
    "loop": _loop,
    **{op: _binary for op in ELEMENTWISE_BINARY},
    **{op: _same for op in ELEMENTWISE_UNARY},
    "is_finite": lambda ins, attrs: [(ins[0].shape, np.dtype(np.bool_))],
    "compare": _compare, "select": _select, "convert": _convert, "broadcast": _broadcast, "reshape": _reshape,
    "transpose": _transpose, "slice": _slice, "concat": _concat, "pad": _pad, "iota": _iota, "constant": _constant,
    "reduce": _reduce, "dot": _dot, "take": _take, "take_along_axis": _take_along,
    "scatter_along_axis": _scatter_like, "put_along_axis": _scatter_like, "update_slice": _scatter_like,
    "dynamic_update_slice": _scatter_like, "dynamic_slice": _dynamic_slice, "topk": _topk,
    "custom_call": _custom_call, "conv": _conv, "all_gather": _all_gather, "all_reduce": _same,
    "reduce_scatter": _reduce_scatter, "all_to_all": _all_to_all,
    # row operations over the last axis: softmax(x); rms_norm(x[, weight]) with attr eps (fp32 statistics)
    "softmax": _same, "rms_norm": _same,
}

OPCODES = tuple(sorted(_INFER))


# --------------------------------------------------------------------------- graph
@dataclass
class TensorPlaceholder:
    """Name / shape / dtype of a kernel input or output as the runtime sees it."""
    name: str
    shape: Shape
    dtype: np.dtype
    original_name: Optional[str] = None

    def __post_init__(self):
        if self.original_name is None:
            self.original_name = self.name


@dataclass(frozen=True)
class AliasInfo:
    """Output `output_index` shares its buffer with parameter `param_index`."""
    output_index: int
    param_index: int
    param_name: str
    is_user_returned: bool


class Graph:
    def __init__(self, name: str = "kernel"):
        self.name = name
        self.params: List[Value] = []
        self.nodes: List[Node] = []
        self.results: List[Value] = []
        self.result_names: List[str] = []
        self.alias_list: List[AliasInfo] = []
        self._next_id = 0
        self._loc: Optional[Tuple[str, int]] = None

    # -- construction
    def _value(self, shape, dtype, name="") -> Value:
        v = Value(self._next_id, tuple(int(s) for s in shape), np.dtype(dtype), name)
        self._next_id += 1
        return v

    def add_parameter(self, shape, dtype, name: str = "") -> Value:
        v = self._value(shape, dtype, name or f"arg{len(self.params)}")
        self.params.append(v)
        return v

    def add_node(self, opcode: str, inputs: Sequence[Value], attrs: Optional[Dict[str, Any]] = None) -> List[Value]:
        attrs = dict(attrs or {})
        try:
            infer = _INFER[opcode]
        except KeyError:
            raise IRError(f"unknown opcode {opcode!r}") from None
        types = infer(list(inputs), attrs)
        node = Node(opcode, list(inputs), attrs, loc=self._loc)
        for i, (shape, dtype) in enumerate(types):
            v = self._value(shape, dtype)
            v.producer, v.index = node, i
            node.outputs.append(v)
        self.nodes.append(node)
        return node.outputs

    def op(self, opcode: str, *inputs: Value, **attrs) -> Value:
        return self.add_node(opcode, inputs, attrs)[0]

    def set_source_location(self, loc: Optional[Tuple[str, int]]) -> None:
        self._loc = loc

    def set_results(self, values: Sequence[Value], names: Sequence[str],
                    aliases: Sequence[AliasInfo] = ()) -> None:
        self.results = list(values)
        self.result_names = list(names)
        self.alias_list = list(aliases)

    # -- protocol shared with the runtime (the reference's ComputationIR)
    @property
    def inputs(self) -> List[TensorPlaceholder]:
        return [TensorPlaceholder(p.name, p.shape, p.dtype) for p in self.params]

    @property
    def outputs(self) -> List[TensorPlaceholder]:
        out = []
        for v, n in zip(self.results, self.result_names):
            dt = np.dtype(np.uint8) if v.dtype == np.bool_ else v.dtype   # bool results surface as uint8
            out.append(TensorPlaceholder(n, v.shape, dt))
        return out

    @property
    def aliases(self) -> List[AliasInfo]:
        return list(self.alias_list)

    @property
    def auto_aliased_indices(self) -> set:
        return {a.output_index for a in self.alias_list if not a.is_user_returned}

    def content_hash(self, compiler_args: str = "") -> str:
        h = hashlib.sha256()
        h.update(self.to_text(with_locations=False).encode())
        h.update(b"\0")
        h.update(compiler_args.encode())
        return h.hexdigest()[:12]

    # -- text form
    def to_text(self, with_locations: bool = True) -> str:
        lines = [f"graph @{self.name} {{"]
        for p in self.params:
            lines.append(f"  %{p.id} = param() {json.dumps({'name': p.name})} : {p.type_str()}")
        for n in self.nodes:
            outs = ", ".join(f"%{o.id}" for o in n.outputs)
            ins = ", ".join(f"%{i.id}" for i in n.inputs)
            attrs = _attrs_to_json(n.attrs)
            types = ", ".join(o.type_str() for o in n.outputs)
            loc = f"  // {n.loc[0]}:{n.loc[1]}" if (with_locations and n.loc) else ""
            lines.append(f"  {outs} = {n.opcode}({ins}) {attrs} : {types}{loc}")
        rets = ", ".join(f"%{v.id} {json.dumps({'name': nm})}" for v, nm in zip(self.results, self.result_names))
        lines.append(f"  return {rets}")
        for a in self.alias_list:
            lines.append(f"  alias {a.output_index} {a.param_index} {int(a.is_user_returned)}")
        lines.append("}")
        return "\n".join(lines) + "\n"

    __str__ = to_text

    @classmethod
    def from_text(cls, text: str) -> "Graph":
        g = None
        values: Dict[int, Value] = {}
        node_re = re.compile(r"^\s*(%[\d%, ]+?)\s*=\s*(\w+)\((.*?)\)\s*(\{.*\})\s*:\s*(.*?)\s*(?://\s*(.*))?$")
        for raw in text.splitlines():
            line = raw.rstrip()
            if not line.strip():
                continue
            m = re.match(r"^\s*graph\s+@(\S+)\s*\{", line)
            if m:
                g = cls(m.group(1))
                continue
            if g is None:
                raise IRError("text does not start with 'graph @name {'")
            if line.strip() == "}":
                continue
            if line.strip().startswith("return"):
                body = line.strip()[len("return"):].strip()
                vals, names = [], []
                for vm in re.finditer(r"%(\d+)\s*(\{[^}]*\})", body):
                    vals.append(values[int(vm.group(1))])
                    names.append(json.loads(vm.group(2))["name"])
                g.results, g.result_names = vals, names
                continue
            if line.strip().startswith("alias"):
                _, oi, pi, ur = line.split()
                g.alias_list.append(AliasInfo(int(oi), int(pi), g.params[int(pi)].name, bool(int(ur))))
                continue
            m = node_re.match(line)
            if not m:
                raise IRError(f"cannot parse IR line: {line!r}")
            out_ids = [int(t.strip()[1:]) for t in m.group(1).split(",")]
            opcode = m.group(2)
            in_ids = [int(t.strip()[1:]) for t in m.group(3).split(",") if t.strip()]
            attrs = _attrs_from_json(m.group(4))
            types = _parse_types(m.group(5))
            loc = None
            if m.group(6) and ":" in m.group(6):
                f, _, ln = m.group(6).rpartition(":")
                if ln.strip().isdigit():
                    loc = (f, int(ln))
            if opcode == "param":
                shape, dtype = types[0]
                v = Value(out_ids[0], shape, dtype, attrs.get("name", ""))
                g.params.append(v)
                values[v.id] = v
                g._next_id = max(g._next_id, v.id + 1)
                continue
            node = Node(opcode, [values[i] for i in in_ids], attrs, loc=loc)
            inferred = _INFER[opcode](node.inputs, attrs)
            if [(tuple(s), np.dtype(d)) for s, d in inferred] != types:
                raise IRError(f"declared result types of {opcode} do not match inference: {line!r}")
            for k, (oid, (shape, dtype)) in enumerate(zip(out_ids, types)):
                v = Value(oid, shape, dtype, "", node, k)
                node.outputs.append(v)
                values[oid] = v
                g._next_id = max(g._next_id, oid + 1)
            g.nodes.append(node)
        if g is None:
            raise IRError("empty IR text")
        return g


def loop_body(node: "Node") -> "Graph":
    """The nested graph of a `loop` node."""
    return Graph.from_text(node.attrs["body"])


def expand_loops(graph: "Graph") -> "Graph":
    """A copy of `graph` with every `loop` node replaced by its unrolled iterations (the index becomes a
    constant per iteration).  The IR keeps loops through the whole pass pipeline; the code generator
    expands them when it emits launches."""
    if not any(n.opcode == "loop" for n in graph.nodes):
        return graph
    out = Graph(graph.name)
    env: Dict[int, Value] = {}
    for p in graph.params:
        env[id(p)] = out.add_parameter(p.shape, p.dtype, p.name)

    def clone_into(src: "Graph", bind: Dict[int, Value]) -> List[Value]:
        local = dict(bind)
        for n in src.nodes:
            out.set_source_location(n.loc)
            ins = [local[id(v)] for v in n.inputs]
            if n.opcode == "loop":
                body = loop_body(n)
                nc = int(n.attrs["num_carried"])
                carried, captured = ins[:nc], ins[nc:]
                for i in range(int(n.attrs["lower"]), int(n.attrs["upper"]), int(n.attrs.get("step", 1))):
                    idx = out.op("constant", value=np.asarray(i, dtype=np.int32))
                    b = {id(body.params[0]): idx}
                    for bp, v in zip(body.params[1:1 + nc], carried):
                        b[id(bp)] = v
                    for bp, v in zip(body.params[1 + nc:], captured):
                        b[id(bp)] = v
                    carried = clone_into(body, b)
                outs = carried
            else:
                outs = out.add_node(n.opcode, ins, dict(n.attrs))
            for o, v in zip(n.outputs, outs):
                local[id(o)] = v
        return [local[id(r)] for r in src.results]

    results = clone_into(graph, env)
    out.set_results(results, list(graph.result_names), list(graph.alias_list))
    return out


def _parse_types(s: str):
    out = []
    for m in re.finditer(r"(\w+)\[([\d,]*)\]", s):
        shape = tuple(int(x) for x in m.group(2).split(",") if x)
        out.append((shape, dtype_from_name(m.group(1))))
    return out


def _attrs_to_json(attrs: Dict[str, Any]) -> str:
    def enc(v):
        if isinstance(v, np.ndarray):
            data = np.require(v, requirements="C")
            return {"__tensor__": dtype_name(data.dtype), "shape": list(data.shape),
                    "data": base64.b64encode(data.tobytes()).decode()}
        if isinstance(v, (np.integer,)):
            return int(v)
        if isinstance(v, (np.floating,)):
            return float(v)
        if isinstance(v, (tuple, list)):
            return [enc(x) for x in v]
        if isinstance(v, dict):
            return {k: enc(x) for k, x in v.items()}
        return v

    return json.dumps({k: enc(v) for k, v in sorted(attrs.items()) if not callable(v)}, separators=(", ", ": "))


def _attrs_from_json(s: str) -> Dict[str, Any]:
    def dec(v):
        if isinstance(v, dict):
            if "__tensor__" in v:
                dt = dtype_from_name(v["__tensor__"])
                return np.frombuffer(base64.b64decode(v["data"]), dtype=dt).reshape(v["shape"]).copy()
            return {k: dec(x) for k, x in v.items()}
        if isinstance(v, list):
            return [dec(x) for x in v]
        return v

    return {k: dec(v) for k, v in json.loads(s).items()}


def prepare_io_mapping(inputs: List[TensorPlaceholder], aliases: List[AliasInfo], original_inputs: Dict[str, Any]):
    """Map user arrays (keyed by parameter name) to IR input names and resolve which input
    each aliased output shares its buffer with."""
    if len(original_inputs) != len(inputs):
        raise RuntimeError(f"Expected {len(inputs)} tensor arguments, got {len(original_inputs)}")
    arrays = {inp.name: original_inputs[inp.original_name] for inp in inputs}
    alias_names = {a.output_index: inputs[a.param_index].name for a in aliases}
    return arrays, alias_names
