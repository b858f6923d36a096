"""Traced kernels that contain collectives.

The reference compiles `all_reduce` / `all_gather` / `reduce_scatter` / `all_to_all` into the device
program and loads it with rank and world size (`nrt_load_collectives`, spike/src/model.cpp:38-46;
nkipy/src/nkipy/core/ops/collectives.py:15-88).  A generated CUDA module here has no communicator, so a
graph with collectives is cut at every collective node: each compute piece becomes its own module
(or, on CPU ranks, runs through the IR interpreter) and the collectives in between run on the pieces'
buffers through `torch.distributed` (NCCL on the device buffers themselves — the C++ runtime uses the
primary context, so its allocations are directly addressable by torch; gloo on NumPy data).

    k = SegmentedKernel.compile(fn, *example_args)            # fn uses nkipy_b200.distributed.collectives
    outs = k(*arrays)                                         # every rank calls it with its own data
"""

from __future__ import annotations

import os
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from ..core.compile import compile_to_neff, trace
from ..core.interp import evaluate
from ..core.ir import Graph, Node, Value
from ..core.trace import NKIPyKernel

COLLECTIVES = ("all_reduce", "all_gather", "reduce_scatter", "all_to_all")


class Segment:
    """A compute piece: `graph` takes the values `in_ids` (ids of the original graph) and yields `out_ids`."""

    def __init__(self, graph: Graph, in_ids: List[int], out_ids: List[int]):
        self.graph, self.in_ids, self.out_ids = graph, in_ids, out_ids
        self.kernel = None                     # DeviceKernel once loaded


def split_at_collectives(g: Graph) -> List[object]:
    """[Segment | Node(collective)] in execution order."""
    # which values are needed after each position
    last_use: Dict[int, int] = {}
    for i, n in enumerate(g.nodes):
        for v in n.inputs:
            last_use[v.id] = i
    for v in g.results:
        last_use[v.id] = len(g.nodes)
    steps: List[object] = []
    cur: List[Tuple[int, Node]] = []

    def flush(end: int):
        if not cur:
            return
        produced = {v.id for _, n in cur for v in n.outputs}
        sub = Graph(f"{g.name}_seg{len(steps)}")
        mapping: Dict[int, Value] = {}
        in_ids: List[int] = []
        for _, n in cur:
            for v in n.inputs:
                if v.id not in produced and v.id not in mapping:
                    mapping[v.id] = sub.add_parameter(v.shape, v.dtype, f"v{v.id}")
                    in_ids.append(v.id)
        for _, n in cur:
            sub.set_source_location(n.loc)
            outs = sub.add_node(n.opcode, [mapping[v.id] for v in n.inputs], n.attrs)
            for o_old, o_new in zip(n.outputs, outs):
                mapping[o_old.id] = o_new
        out_ids = [vid for vid in sorted(produced) if last_use.get(vid, -1) >= end]
        sub.set_results([mapping[i] for i in out_ids], [f"v{i}" for i in out_ids])
        steps.append(Segment(sub, in_ids, out_ids))
        cur.clear()

    for i, n in enumerate(g.nodes):
        if n.opcode in COLLECTIVES:
            flush(i)
            steps.append(n)
        else:
            cur.append((i, n))
    flush(len(g.nodes))
    return steps


# ------------------------------------------------------------------------------- collectives on torch tensors
def _run_collective(n: Node, x, dist, group=None):
    """x: torch tensor (CPU or CUDA) holding this rank's operand; returns the result tensor."""
    import torch

    a = n.attrs
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        groups = a.get("replica_groups") or [[0]]
        if len(groups[0]) != 1:
            raise RuntimeError(f"kernel was traced for {len(groups[0])} ranks but runs on one")
    red = {"add": dist.ReduceOp.SUM, "multiply": dist.ReduceOp.PRODUCT, "maximum": dist.ReduceOp.MAX,
           "minimum": dist.ReduceOp.MIN}
    op = n.opcode
    if op == "all_reduce":
        out = x.clone()
        if world > 1:
            dist.all_reduce(out, op=red[a.get("op", "add")], group=group)
        return out
    if op == "all_gather":
        dim = a["dim"]
        parts = [torch.empty_like(x) for _ in range(world)]
        if world > 1:
            dist.all_gather(parts, x.contiguous(), group=group)
        else:
            parts = [x]
        return torch.cat(parts, dim=dim).contiguous()
    if op == "reduce_scatter":
        dim = a["dim"]
        chunks = [c.contiguous() for c in torch.chunk(x, world, dim=dim)]
        out = torch.empty_like(chunks[0])
        if world > 1:
            # all-reduce + slice keeps this independent of the backend's reduce_scatter support (gloo has none)
            full = x.clone()
            dist.all_reduce(full, op=red[a.get("op", "add")], group=group)
            out = torch.chunk(full, world, dim=dim)[dist.get_rank(group)].contiguous()
        else:
            out = chunks[0]
        return out
    if op == "all_to_all":
        sd, cd = a["split_dim"], a["concat_dim"]
        send = [c.contiguous() for c in torch.chunk(x, world, dim=sd)]
        recv = [torch.empty_like(s) for s in send]
        if world > 1:
            if x.is_cuda:
                dist.all_to_all(recv, send, group=group)
            else:                                       # gloo: exchange through all_gather of the pieces
                rank = dist.get_rank(group)
                for src in range(world):
                    bucket = [torch.empty_like(send[0]) for _ in range(world)]
                    dist.all_gather(bucket, send[src], group=group)
                    # bucket[r] = what rank r sends to rank `src`
                    if src == rank:
                        recv = bucket
        else:
            recv = send
        return torch.cat(recv, dim=cd).contiguous()
    raise NotImplementedError(op)


class SegmentedKernel:
    def __init__(self, graph: Graph, steps: List[object], backend: str, name: str):
        self.graph, self.steps, self.backend, self.name = graph, steps, backend, name

    @property
    def num_segments(self) -> int:
        return sum(isinstance(s, Segment) for s in self.steps)

    @property
    def num_collectives(self) -> int:
        return sum(not isinstance(s, Segment) for s in self.steps)

    @classmethod
    def compile(cls, kernel, *args, name: Optional[str] = None, backend: Optional[str] = None,
                build_dir: Optional[str] = None, **kwargs) -> "SegmentedKernel":
        """backend "device": one cubin per compute piece, NCCL in between; "interp": IR interpreter + the
        process group's CPU backend.  Default: "device" when CUDA is available."""
        import torch

        if not isinstance(kernel, NKIPyKernel):
            kernel = trace(kernel)
        name = name or kernel.__name__
        graph = kernel.specialize(*args, **kwargs)
        if backend is None:
            backend = "device" if torch.cuda.is_available() else "interp"
        steps = split_at_collectives(graph)
        self = cls(graph, steps, backend, name)
        if backend == "device":
            from .device_kernel import DeviceKernel
            from ..core.compile import _get_build_dir

            root = build_dir or os.path.join(_get_build_dir(), f"{name}_{graph.content_hash()}")
            for i, s in enumerate(steps):
                if isinstance(s, Segment):
                    out_dir = os.path.join(root, f"seg{i}")
                    cubin = os.path.join(out_dir, f"{name}_seg{i}.cubin")
                    if not os.path.exists(cubin):
                        compile_to_neff(s.graph, out_dir, f"{name}_seg{i}.cubin")
                    s.kernel = DeviceKernel.load_from_neff(cubin, name=f"{name}_seg{i}")
        return self

    # ------------------------------------------------------------------ execution
    def __call__(self, *arrays: np.ndarray):
        if len(arrays) != len(self.graph.params):
            raise ValueError(f"{self.name} takes {len(self.graph.params)} arrays")
        return self._run_device(arrays) if self.backend == "device" else self._run_interp(arrays)

    def _run_interp(self, arrays):
        import torch
        import torch.distributed as dist

        env: Dict[int, np.ndarray] = {p.id: np.asarray(a) for p, a in zip(self.graph.params, arrays)}
        for s in self.steps:
            if isinstance(s, Segment):
                outs = evaluate(s.graph, [env[i] for i in s.in_ids])
                env.update(dict(zip(s.out_ids, outs)))
            else:
                x = env[s.inputs[0].id]
                t = torch.from_numpy(np.ascontiguousarray(x.astype(np.float32) if x.dtype.kind == "V" else x))
                env[s.outputs[0].id] = _run_collective(s, t, dist).numpy().astype(s.outputs[0].dtype, copy=False)
        res = [env[v.id] for v in self.graph.results]
        return res[0] if len(res) == 1 else tuple(res)

    def _run_device(self, arrays):
        import torch
        import torch.distributed as dist

        from .device_tensor import DeviceTensor, _torch_maps

        _, n2t = _torch_maps()
        env: Dict[int, DeviceTensor] = {
            p.id: DeviceTensor.from_numpy(np.ascontiguousarray(np.asarray(a).astype(p.dtype, copy=False)), f"v{p.id}")
            for p, a in zip(self.graph.params, arrays)}

        def view(t: DeviceTensor):
            class _Arr:
                __cuda_array_interface__ = {"shape": (t.nbytes,), "typestr": "|u1", "data": (int(t.tensor_ref.va), False),
                                            "version": 3, "strides": None}
            return torch.as_tensor(_Arr(), device="cuda").view(n2t[np.dtype(t.dtype)]).view(tuple(t.shape))

        for s in self.steps:
            if isinstance(s, Segment):
                ins = {f"v{i}": env[i] for i in s.in_ids}
                outs = s.kernel(ins)
                for i in s.out_ids:
                    env[i] = outs[f"v{i}"]
            else:
                src = env[s.inputs[0].id]
                res = _run_collective(s, view(src), dist)
                torch.cuda.synchronize()
                out = DeviceTensor.empty(tuple(res.shape), s.outputs[0].dtype, f"v{s.outputs[0].id}")
                view(out).copy_(res)
                torch.cuda.synchronize()
                env[s.outputs[0].id] = out
        res = [env[v.id].numpy() for v in self.graph.results]
        return res[0] if len(res) == 1 else tuple(res)
