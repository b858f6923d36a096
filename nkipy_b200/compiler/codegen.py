"""IR -> CUDA C++ code generator.

Replaces the reference's HLO -> neuronx-cc lowering
(nkipy/src/nkipy/core/compile.py:158-203): a traced `Graph` becomes one CUDA C++
translation unit plus a launch plan (JSON sidecar) that the C++ runtime executes
(csrc/runtime).  Design:

* **Views instead of data movement.**  `transpose`, `slice`, `broadcast`, and
  `reshape` of a contiguous value are folded into strided *views* of the producing
  buffer; no kernel is emitted for them.
* **Pointwise fusion.**  Maximal groups of elementwise nodes of one shape are emitted
  as a single kernel; operands are loaded through their views, results are stored
  contiguously (or into a slice of a larger buffer for `concat` / `update_slice`).
* **Template library for contractions.**  bf16 `dot`s with TMA-compatible shapes
  instantiate the hand-written tcgen05/TMEM GEMM (`csrc/kernels/gemm_tcgen05.cuh`);
  the runtime encodes the tensor maps the plan describes.  Other dtypes / shapes use
  a strided shared-memory tiled SIMT GEMM with fp32 accumulation.
* Everything else (reductions, gathers, scatters, top-k, convolution) is a small
  generic kernel specialised by the generator with the static shapes.

`lower_to_cuda(graph)` returns the source, mirroring the reference's `lower_to_nki`
(nkipy/src/nkipy/core/compile.py:347-384).
"""

from __future__ import annotations

import json
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np

from ..core.dtypes import bfloat16, dtype_name, float8_e4m3, float8_e5m2
from ..core.ir import ELEMENTWISE_BINARY, ELEMENTWISE_UNARY, Graph, Node, Value

_CTYPE = {
    "pred": "unsigned char", "i8": "signed char", "i16": "short", "i32": "int", "i64": "long long",
    "u8": "unsigned char", "u16": "unsigned short", "u32": "unsigned int", "u64": "unsigned long long",
    "f16": "__half", "bf16": "__nv_bfloat16", "f32": "float", "f64": "double",
    "f8e5m2": "__nv_fp8_e5m2", "f8e4m3": "__nv_fp8_e4m3",
}
POINTWISE = (ELEMENTWISE_BINARY | ELEMENTWISE_UNARY | {"compare", "select", "convert"}) - {"copy"}


def ctype(dt) -> str:
    return _CTYPE[dtype_name(dt)]


def compute_type(dt) -> str:
    """Type arithmetic is carried in: fp32 for every float narrower than 32 bits."""
    n = dtype_name(dt)
    if n in ("f16", "bf16", "f8e5m2", "f8e4m3", "f32"):
        return "float"
    if n == "f64":
        return "double"
    if n == "pred":
        return "bool"
    return _CTYPE[n]


def _contig_strides(shape: Sequence[int]) -> List[int]:
    st, acc = [], 1
    for d in reversed(shape):
        st.append(acc)
        acc *= d
    return list(reversed(st))


@dataclass
class View:
    """A strided window of a buffer: element (i0, i1, ...) lives at offset + sum(i_k * strides_k)."""
    buffer: int
    shape: Tuple[int, ...]
    strides: Tuple[int, ...]
    offset: int
    dtype: np.dtype

    def is_contiguous(self) -> bool:
        return self.offset == 0 and list(self.strides) == _contig_strides(self.shape) or self.size() <= 1 and False

    def dense(self) -> bool:
        """Contiguous from its offset (a reshape of it is again a view)."""
        exp = 1
        for d, s in zip(reversed(self.shape), reversed(self.strides)):
            if d == 1:
                continue
            if s != exp:
                return False
            exp *= d
        return True

    def size(self) -> int:
        n = 1
        for d in self.shape:
            n *= d
        return n


@dataclass
class BufferInfo:
    index: int
    nbytes: int
    kind: str                 # "input" | "output" | "temp" | "const"
    name: str = ""
    dtype: str = ""
    shape: Tuple[int, ...] = ()
    alias_of: Optional[int] = None      # output buffer that must share memory with an input
    const_data: Optional[bytes] = None


@dataclass
class Launch:
    kernel: str
    grid: Tuple[int, int, int]
    block: Tuple[int, int, int]
    smem: int
    args: List[Dict[str, Any]]          # {"buffer": i, "offset": bytes} | {"i32": v} | {"tensormap": {...}} | ...
    loc: Optional[str] = None


@dataclass
class Program:
    source: str
    buffers: List[BufferInfo]
    launches: List[Launch]
    inputs: List[Dict[str, Any]]
    outputs: List[Dict[str, Any]]
    name: str = "kernel"
    # set when the module contains collectives: {"world": ranks, "half_bytes": bytes of one data half of the
    # symmetric workspace, "workspace_bytes": flags + two halves}
    collective: Optional[Dict[str, int]] = None

    def plan_json(self) -> str:
        def buf(b: BufferInfo):
            d = {"index": b.index, "nbytes": b.nbytes, "kind": b.kind, "name": b.name, "dtype": b.dtype,
                 "shape": list(b.shape)}
            if b.alias_of is not None:
                d["alias_of"] = b.alias_of
            if b.const_data is not None:
                import base64

                d["data"] = base64.b64encode(b.const_data).decode()
            return d

        return json.dumps({
            "name": self.name,
            "buffers": [buf(b) for b in self.buffers],
            "launches": [{"kernel": l.kernel, "grid": list(l.grid), "block": list(l.block), "smem": l.smem,
                          "args": l.args, "loc": l.loc} for l in self.launches],
            "inputs": self.inputs, "outputs": self.outputs,
            **({"collective": self.collective} if self.collective else {}),
        }, indent=1)


_PRELUDE = r"""// generated by nkipy_b200.compiler.codegen -- do not edit
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <math.h>
#include <stdint.h>
#ifdef NKB_USE_TCGEN05
#include "gemm_tcgen05.cuh"
#endif

namespace {
template <typename T> __device__ __forceinline__ float ld_f(const T* p, long long i) { return float(p[i]); }
template <> __device__ __forceinline__ float ld_f<__half>(const __half* p, long long i) { return __half2float(p[i]); }
template <> __device__ __forceinline__ float ld_f<__nv_bfloat16>(const __nv_bfloat16* p, long long i) { return __bfloat162float(p[i]); }
template <typename C, typename T> __device__ __forceinline__ C ld(const T* p, long long i) { return C(p[i]); }
template <> __device__ __forceinline__ float ld<float, __half>(const __half* p, long long i) { return __half2float(p[i]); }
template <> __device__ __forceinline__ float ld<float, __nv_bfloat16>(const __nv_bfloat16* p, long long i) { return __bfloat162float(p[i]); }
template <> __device__ __forceinline__ float ld<float, __nv_fp8_e5m2>(const __nv_fp8_e5m2* p, long long i) { return float(p[i]); }
template <> __device__ __forceinline__ float ld<float, __nv_fp8_e4m3>(const __nv_fp8_e4m3* p, long long i) { return float(p[i]); }
template <> __device__ __forceinline__ bool ld<bool, unsigned char>(const unsigned char* p, long long i) { return p[i] != 0; }
template <typename T, typename C> __device__ __forceinline__ void st(T* p, long long i, C v) { p[i] = T(v); }
template <> __device__ __forceinline__ void st<__half, float>(__half* p, long long i, float v) { p[i] = __float2half_rn(v); }
template <> __device__ __forceinline__ void st<__nv_bfloat16, float>(__nv_bfloat16* p, long long i, float v) { p[i] = __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ void st<unsigned char, bool>(unsigned char* p, long long i, bool v) { p[i] = v ? 1 : 0; }
template <typename T> __device__ __forceinline__ T sgn(T v) { return T((v > T(0)) - (v < T(0))); }
__device__ __forceinline__ float rem_f(float a, float b) { return fmodf(a, b); }
__device__ __forceinline__ double rem_f(double a, double b) { return fmod(a, b); }
template <typename T> __device__ __forceinline__ T rem_f(T a, T b) { return b == 0 ? T(0) : T(a % b); }
template <typename T> __device__ __forceinline__ T div_i(T a, T b) { return b == 0 ? T(0) : T(a / b); }
__device__ __forceinline__ float div_i(float a, float b) { return a / b; }
__device__ __forceinline__ double div_i(double a, double b) { return a / b; }
template <typename T> __device__ __forceinline__ T pow_i(T a, T b) { return T(pow(double(a), double(b))); }
__device__ __forceinline__ float pow_i(float a, float b) { return powf(a, b); }
__device__ __forceinline__ float warp_reduce_sum(float v) { for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(~0u, v, o); return v; }
}  // namespace

// ---- collectives inside a module ------------------------------------------------------------------------
// Every rank of the group loads the same module; the runtime hands each collective kernel this table: the
// module's symmetric workspace on every rank (flags, then two data halves of `half_bytes`), this rank's
// index, and two device counters.  Protocol of collective number u (u = *seen, the same on all ranks):
//   cc_push    copies the operand into slot [rank] of half (u & 1) of every rank's workspace; the last CTA
//              publishes with a system-scope fence and adds 1 to flags[rank] on every rank;
//   cc_consume waits (bounded, one second) until flags[s] >= u + 1 for every rank s, builds the result from
//              the n slots, and its last CTA advances *seen.
// Counters only grow and the halves alternate, so a rank that runs ahead cannot overwrite a slot a peer
// still reads (it needs that peer's operand of the next collective first).
struct CcTable {
  unsigned long long peer_ws[8];     // base of every rank's workspace
  unsigned long long local_ws;
  unsigned int* seen;                // collectives completed by this module
  unsigned int* done;                // [2] CTA counters of the two kernels
  int* status;                       // bounded-wait status word (0 = fine)
  long long half_bytes;
  int rank, world;
};
static constexpr long long kCcFlagBytes = 256;
__device__ __forceinline__ unsigned int cc_ld_acquire(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long cc_timer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
template <typename T>
__device__ __forceinline__ void cc_push(const T* __restrict__ in, long long n, const CcTable& t) {
  const unsigned int use = *reinterpret_cast<volatile unsigned int*>(t.seen);
  const long long slot = kCcFlagBytes + (long long)(use & 1u) * t.half_bytes + (long long)t.rank * n * (long long)sizeof(T);
  for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < n; e += (long long)gridDim.x * blockDim.x) {
    const T v = in[e];
    for (int p = 0; p < t.world; ++p) reinterpret_cast<T*>(t.peer_ws[p] + slot)[e] = v;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int old = atomicAdd(t.done, 1u);
    if (old == gridDim.x - 1) {
      *t.done = 0u;
      __threadfence_system();
      for (int p = 0; p < t.world; ++p)
        asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(t.peer_ws[p] + 4ull * t.rank), "r"(1u) : "memory");
    }
  }
}
// Returns false when a rank's operand did not arrive in time (the status word then says which).
__device__ __forceinline__ bool cc_wait(const CcTable& t, unsigned int use) {
  __shared__ int ok_s;
  if (threadIdx.x == 0) {
    int ok = 1;
    const unsigned int* flags = reinterpret_cast<const unsigned int*>(t.local_ws);
    const unsigned long long t0 = cc_timer();
    for (int s = 0; s < t.world && ok; ++s) {
      unsigned int spins = 0;
      while (int(cc_ld_acquire(flags + s) - (use + 1u)) < 0) {
        __nanosleep(64);
        if ((++spins & 255u) == 0 && cc_timer() - t0 > 1000000000ull) {
          atomicCAS(t.status, 0, 5 | (s << 8) | (9 << 16));
          ok = 0;
          break;
        }
      }
    }
    ok_s = ok;
  }
  __syncthreads();
  return ok_s != 0;
}
__device__ __forceinline__ void cc_finish(const CcTable& t, unsigned int use, bool ok) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int old = atomicAdd(t.done + 1, 1u);
    if (old == gridDim.x - 1) {
      t.done[1] = 0u;
      if (ok) *t.seen = use + 1u;
      __threadfence();
    }
  }
}
"""


class CodegenError(NotImplementedError):
    pass


class Generator:
    def __init__(self, graph: Graph, use_tcgen05: bool = True):
        self.g = graph
        self.use_tcgen05 = use_tcgen05
        self.buffers: List[BufferInfo] = []
        self.views: Dict[int, View] = {}         # value id -> view
        self.launches: List[Launch] = []
        self.kernels: List[str] = []
        self.uses: Dict[int, int] = {}
        self._k = 0
        self.uses_tcgen05 = False

    # ------------------------------------------------------------------ buffers / views
    def new_buffer(self, shape, dtype, kind="temp", name="", const: Optional[np.ndarray] = None) -> int:
        n = int(np.prod(shape, dtype=np.int64)) * np.dtype(dtype).itemsize
        b = BufferInfo(len(self.buffers), max(n, 1), kind, name, dtype_name(dtype), tuple(shape),
                       const_data=None if const is None else np.ascontiguousarray(const).tobytes())
        self.buffers.append(b)
        return b.index

    def contiguous_view(self, buf: int, shape, dtype) -> View:
        return View(buf, tuple(shape), tuple(_contig_strides(shape)), 0, np.dtype(dtype))

    def view_of(self, v: Value) -> View:
        return self.views[v.id]

    def materialize(self, v: Value) -> View:
        """A dense, zero-offset copy of the value (needed before a non-affine reshape or TMA)."""
        vw = self.view_of(v)
        if vw.offset == 0 and list(vw.strides) == _contig_strides(vw.shape):
            return vw
        buf = self.new_buffer(v.shape, v.dtype)
        out = self.contiguous_view(buf, v.shape, v.dtype)
        self.emit_pointwise([("copy", [("in", vw)], {}, v.dtype)], [out], v.shape)
        return out

    def kname(self, base: str) -> str:
        self._k += 1
        return f"k{self._k}_{base}"

    # ------------------------------------------------------------------ driver
    def run(self) -> Program:
        from ..core.ir import expand_loops

        # loops stay loops through the pass pipeline; launches are emitted per iteration
        self.g = expand_loops(self.g)
        g = self.g
        for n in g.nodes:
            for i in n.inputs:
                self.uses[i.id] = self.uses.get(i.id, 0) + 1
        for r in g.results:
            self.uses[r.id] = self.uses.get(r.id, 0) + 1
        inputs = []
        for p in g.params:
            b = self.new_buffer(p.shape, p.dtype, "input", p.name)
            self.views[p.id] = self.contiguous_view(b, p.shape, p.dtype)
            inputs.append({"name": p.name, "buffer": b, "shape": list(p.shape), "dtype": dtype_name(p.dtype)})
        pending: List[Node] = []       # pointwise nodes waiting to be flushed as one kernel
        consumed = set()               # nodes already emitted as part of a GEMM epilogue
        for idx, n in enumerate(g.nodes):
            if id(n) in consumed:
                continue
            if n.opcode in POINTWISE and self._fusable(n, pending):
                pending.append(n)
                continue
            self._flush(pending)
            pending = []
            if n.opcode in POINTWISE:
                pending.append(n)
            elif n.opcode == "dot":
                views, chain = self._epilogue_chain(idx)
                for v in views:
                    self.lower(v)
                    consumed.add(id(v))
                for c in chain:
                    consumed.add(id(c))
                self.lower_dot(n, epilogue=chain)
            else:
                self.lower(n)
        self._flush(pending)
        outputs = []
        alias = {a.output_index: a.param_index for a in g.alias_list}
        for i, (r, name) in enumerate(zip(g.results, g.result_names)):
            vw = self.materialize(r)
            b = self.buffers[vw.buffer]
            if b.kind in ("input", "const") or any(o["buffer"] == vw.buffer for o in outputs):
                nb = self.new_buffer(r.shape, r.dtype)
                out = self.contiguous_view(nb, r.shape, r.dtype)
                self.emit_pointwise([("copy", [("in", vw)], {}, r.dtype)], [out], r.shape)
                vw, b = out, self.buffers[nb]
            b.kind, b.name = "output", name
            if i in alias:
                b.alias_of = inputs[alias[i]]["buffer"]
            dt = np.dtype(np.uint8) if r.dtype == np.bool_ else r.dtype
            outputs.append({"name": name, "buffer": vw.buffer, "shape": list(r.shape), "dtype": dtype_name(dt)})
        src = _PRELUDE + "\n".join(self.kernels)
        if self.uses_tcgen05:
            src = "#define NKB_USE_TCGEN05 1\n" + src
        prog = Program(src, self.buffers, self.launches, inputs, outputs, g.name)
        if getattr(self, "cc_half_bytes", 0):
            half = (self.cc_half_bytes + 255) // 256 * 256
            prog.collective = {"world": self.cc_world, "half_bytes": half, "workspace_bytes": 256 + 2 * half}
        return prog

    def _epilogue_chain(self, idx: int):
        """Elementwise nodes the fusion pass marked as the epilogue of the dot at position idx
        (`_epilogue_of` = the dot's `_op_id`, continued through the same `_fuse_group`): they are emitted inside
        the GEMM kernel, applied to the fp32 accumulator before the single store.  Returns (view / constant
        nodes in between that only need their views set up, the chain); an empty chain means no fusion.
        The chain must be 2-D, consume the dot's result nowhere else, let only its last value escape and end in
        bf16 (what the GEMM stores)."""
        g = self.g
        dot = g.nodes[idx]
        out = dot.outputs[0]
        if "_op_id" not in dot.attrs or len(out.shape) != 2:
            return [], []
        views, chain, group = [], [], None
        j = idx + 1
        while j < len(g.nodes):
            m = g.nodes[j]
            if m.opcode in ("broadcast", "reshape", "transpose", "slice", "constant"):
                if any(i.id == out.id or any(i.id == c.outputs[0].id for c in chain) for i in m.inputs):
                    break                                   # a view of the dot result: it must be materialised
                views.append(m)
                j += 1
                continue
            if m.opcode not in POINTWISE or tuple(m.outputs[0].shape) != tuple(out.shape):
                break
            if not chain:
                if m.attrs.get("_epilogue_of") != dot.attrs["_op_id"]:
                    break
                group = m.attrs.get("_fuse_group")
            elif m.attrs.get("_fuse_group") != group:
                break
            chain.append(m)
            j += 1
        # drop trailing view nodes that no chain member reads (they belong to later code)
        if not chain:
            return [], []
        inside = {out.id} | {c.outputs[0].id for c in chain}
        internal_uses: Dict[int, int] = {}
        for c in chain:
            for i in c.inputs:
                if i.id in inside:
                    internal_uses[i.id] = internal_uses.get(i.id, 0) + 1
        # shrink the chain until exactly its last value escapes and nothing else does
        while chain:
            inside = {out.id} | {c.outputs[0].id for c in chain}
            internal_uses = {}
            for c in chain:
                for i in c.inputs:
                    if i.id in inside:
                        internal_uses[i.id] = internal_uses.get(i.id, 0) + 1
            ok = self.uses.get(out.id, 0) == internal_uses.get(out.id, 0)
            for c in chain[:-1]:
                o = c.outputs[0]
                if self.uses.get(o.id, 0) != internal_uses.get(o.id, 0):
                    ok = False
            last = chain[-1].outputs[0]
            if dtype_name(last.dtype) != "bf16":
                ok = False
            if ok:
                break
            chain = chain[:-1]
        if not chain:
            return [], []
        last_pos = g.nodes.index(chain[-1])
        views = [v for v in views if g.nodes.index(v) < last_pos]
        return views, chain

    def _fusable(self, n: Node, pending: List[Node]) -> bool:
        if not pending:
            return True
        return pending[0].outputs[0].shape == n.outputs[0].shape and len(pending) < 64

    # ------------------------------------------------------------------ pointwise groups
    def _flush(self, nodes: List[Node]) -> None:
        if not nodes:
            return
        inside = {n.outputs[0].id for n in nodes}
        shape = nodes[0].outputs[0].shape
        # values that must be written to memory: used outside the group or by a later node kind
        counts: Dict[int, int] = {}
        for n in nodes:
            for i in n.inputs:
                if i.id in inside:
                    counts[i.id] = counts.get(i.id, 0) + 1
        exprs, outs = [], []
        for n in nodes:
            o = n.outputs[0]
            ops = []
            for i in n.inputs:
                if i.id in inside:
                    ops.append(("val", i.id))
                else:
                    ops.append(("in", self.view_of(i)))
            exprs.append((n.opcode, ops, dict(n.attrs, _id=o.id, _in_dtypes=[i.dtype for i in n.inputs]), o.dtype))
            if self.uses.get(o.id, 0) > counts.get(o.id, 0):
                buf = self.new_buffer(o.shape, o.dtype)
                vw = self.contiguous_view(buf, o.shape, o.dtype)
                self.views[o.id] = vw
                outs.append((o.id, vw))
        self.emit_pointwise(exprs, [vw for _, vw in outs], shape, out_ids=[i for i, _ in outs],
                            loc=nodes[-1].loc)

    def emit_pointwise(self, exprs, out_views: List[View], shape, out_ids=None, loc=None) -> None:
        """One kernel: thread e computes all expressions at multi-index(e) and stores the outputs.
        exprs: (opcode, operands, attrs, out_dtype); operands ("in", View) | ("val", value_id)."""
        name = self.kname("pointwise")
        shape = tuple(shape)
        total = int(np.prod(shape, dtype=np.int64))
        if total == 0:
            return
        params, args, body = [], [], []
        loads: Dict[Tuple, str] = {}

        def param_for(vw: View, const=True) -> str:
            key = (vw.buffer, vw.offset)
            pname = f"p{len(params)}"
            params.append(f"{'const ' if const else ''}{ctype(vw.dtype)}* __restrict__ {pname}")
            args.append({"buffer": vw.buffer, "offset": vw.offset * vw.dtype.itemsize})
            return pname

        nd = len(shape)
        body.append("  long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x;")
        body.append(f"  if (e >= {total}LL) return;")
        if nd:
            body.append("  long long r = e;")
            for d in range(nd - 1, -1, -1):
                if d == 0:
                    body.append(f"  const long long i{d} = r;")
                else:
                    body.append(f"  const long long i{d} = r % {shape[d]}; r /= {shape[d]};")

        def index_expr(vw: View) -> str:
            if len(vw.shape) != nd:
                raise CodegenError("operand view rank differs from the kernel's index space")
            terms = [f"i{d} * {s}LL" for d, s in enumerate(vw.strides) if s != 0 and shape[d] != 1]
            return " + ".join(terms) if terms else "0"

        def operand(op, want_ctype: str) -> str:
            kind, x = op
            if kind == "val":
                return f"v{x}"
            key = (x.buffer, x.offset, x.strides, want_ctype)
            if key not in loads:
                p = param_for(x)
                var = f"l{len(loads)}"
                body.append(f"  const {want_ctype} {var} = ld<{want_ctype}>({p}, {index_expr(x)});")
                loads[key] = var
            return loads[key]

        tmp = 0
        last_vars = []
        for opcode, ops, attrs, odt in exprs:
            ct = compute_type(odt)
            in_dts = attrs.get("_in_dtypes") or [o[1].dtype if o[0] == "in" else odt for o in ops]
            a = [operand(o, compute_type(dt)) for o, dt in zip(ops, in_dts)]
            vid = attrs.get("_id")
            var = f"v{vid}" if vid is not None else f"t{tmp}"
            tmp += 1
            body.append(f"  const {ct} {var} = {self._expr(opcode, a, attrs, odt, in_dts)};")
            last_vars.append(var)
        if out_ids is None:
            out_vars = last_vars[-len(out_views):] if out_views else []
        else:
            out_vars = [f"v{i}" for i in out_ids]
        for vw, var in zip(out_views, out_vars):
            p = param_for(vw, const=False)
            body.append(f"  st({p}, {index_expr(vw)}, {var});")
        if not out_views:
            return
        src = f'extern "C" __global__ void {name}({", ".join(params)}) {{\n' + "\n".join(body) + "\n}\n"
        self.kernels.append(src)
        block = 256
        self.launches.append(Launch(name, ((total + block - 1) // block, 1, 1), (block, 1, 1), 0, args,
                                    f"{loc[0]}:{loc[1]}" if loc else None))

    def _expr(self, op: str, a: List[str], attrs, odt, in_dts) -> str:
        ct = compute_type(odt)
        f = ct in ("float", "double")
        sfx = "f" if ct == "float" else ""
        if op == "copy":
            return a[0]
        if op == "add": return f"({a[0]} + {a[1]})" if ct != "bool" else f"({a[0]} || {a[1]})"
        if op == "sub": return f"({a[0]} - {a[1]})"
        if op == "mul": return f"({a[0]} * {a[1]})" if ct != "bool" else f"({a[0]} && {a[1]})"
        if op == "div": return f"div_i({a[0]}, {a[1]})"
        if op == "pow": return f"pow_i({a[0]}, {a[1]})"
        if op == "rem": return f"rem_f({a[0]}, {a[1]})"
        if op == "max": return (f"fmax{sfx}({a[0]}, {a[1]})" if f else f"(({a[0]}) > ({a[1]}) ? ({a[0]}) : ({a[1]}))")
        if op == "min": return (f"fmin{sfx}({a[0]}, {a[1]})" if f else f"(({a[0]}) < ({a[1]}) ? ({a[0]}) : ({a[1]}))")
        if op == "atan2": return f"atan2{sfx}({a[0]}, {a[1]})"
        if op in ("and", "or", "xor"):
            if ct == "bool":
                return {"and": f"({a[0]} && {a[1]})", "or": f"({a[0]} || {a[1]})", "xor": f"({a[0]} != {a[1]})"}[op]
            return f"{ct}({a[0]} {'&' if op == 'and' else '|' if op == 'or' else '^'} {a[1]})"
        if op == "not": return f"(!{a[0]})" if ct == "bool" else f"{ct}(~{a[0]})"
        if op == "abs": return f"fabs{sfx}({a[0]})" if f else (a[0] if ct.startswith("unsigned") or ct == "bool"
                                                               else f"{ct}({a[0]} < 0 ? -{a[0]} : {a[0]})")
        if op == "neg": return f"(-{a[0]})" if ct != "bool" else a[0]
        if op == "sign": return f"sgn({a[0]})" if ct != "bool" else a[0]
        if op == "rsqrt": return f"(1.0{sfx} / sqrt{sfx}({a[0]}))"
        if op == "round_even": return f"rint{sfx}({a[0]})"
        if op == "is_finite": return f"isfinite({a[0]})"
        if op in ("exp", "log", "sqrt", "sin", "cos", "tanh", "ceil", "floor", "erf"):
            return f"{op}{sfx}({a[0]})"
        if op == "compare":
            sym = {"EQ": "==", "NE": "!=", "LT": "<", "LE": "<=", "GT": ">", "GE": ">="}[attrs["direction"]]
            return f"({a[0]} {sym} {a[1]})"
        if op == "select": return f"({a[0]} ? {a[1]} : {a[2]})"
        if op == "convert":
            src_ct = compute_type(in_dts[0])
            if ct == "bool":
                return f"({a[0]} != 0)"
            if ct not in ("float", "double") and src_ct in ("float", "double"):
                return f"{ct}(trunc{'f' if src_ct == 'float' else ''}({a[0]}))"
            if ct == "float" and dtype_name(odt) in ("f16", "bf16", "f8e5m2", "f8e4m3"):
                # value is carried in fp32 but must be rounded to the narrow type now
                t = ctype(odt)
                return f"float({t}({src_ct == 'bool' and '(float)' or ''}{a[0]}))" if src_ct != "bool" \
                    else f"float({t}(float({a[0]})))"
            return f"{ct}({a[0]})"
        raise CodegenError(f"no pointwise rule for {op}")

    # ------------------------------------------------------------------ other nodes
    def lower(self, n: Node) -> None:
        fn = getattr(self, f"lower_{n.opcode}", None)
        if fn is None:
            raise CodegenError(f"code generation for '{n.opcode}' is not implemented")
        fn(n)

    def lower_copy(self, n):
        o = n.outputs[0]
        buf = self.new_buffer(o.shape, o.dtype)
        out = self.contiguous_view(buf, o.shape, o.dtype)
        self.emit_pointwise([("copy", [("in", self.view_of(n.inputs[0]))], {}, o.dtype)], [out], o.shape, loc=n.loc)
        self.views[o.id] = out

    def lower_constant(self, n):
        o = n.outputs[0]
        arr = np.asarray(n.attrs["value"])
        buf = self.new_buffer(o.shape, o.dtype, "const", const=arr)
        self.views[o.id] = self.contiguous_view(buf, o.shape, o.dtype)

    def lower_reshape(self, n):
        x, o = n.inputs[0], n.outputs[0]
        vw = self.view_of(x)
        if not vw.dense():
            vw = self.materialize(x)
        self.views[o.id] = View(vw.buffer, o.shape, tuple(_contig_strides(o.shape)), vw.offset, vw.dtype)

    def lower_transpose(self, n):
        vw = self.view_of(n.inputs[0])
        perm = n.attrs["perm"]
        self.views[n.outputs[0].id] = View(vw.buffer, tuple(vw.shape[p] for p in perm),
                                           tuple(vw.strides[p] for p in perm), vw.offset, vw.dtype)

    def lower_slice(self, n):
        vw = self.view_of(n.inputs[0])
        off = vw.offset + sum(s * st for s, st in zip(n.attrs["start"], vw.strides))
        self.views[n.outputs[0].id] = View(vw.buffer, n.outputs[0].shape,
                                           tuple(st * k for st, k in zip(vw.strides, n.attrs["stride"])), off, vw.dtype)

    def lower_broadcast(self, n):
        vw = self.view_of(n.inputs[0])
        shape, dims = n.attrs["shape"], n.attrs["dims"]
        strides = [0] * len(shape)
        for i, d in enumerate(dims):
            strides[d] = 0 if vw.shape[i] == 1 else vw.strides[i]
        self.views[n.outputs[0].id] = View(vw.buffer, tuple(shape), tuple(strides), vw.offset, vw.dtype)

    def lower_iota(self, n):
        o = n.outputs[0]
        name = self.kname("iota")
        total = o.size
        buf = self.new_buffer(o.shape, o.dtype)
        inner = int(np.prod(o.shape[n.attrs["dim"] + 1:], dtype=np.int64))
        self.kernels.append(
            f'extern "C" __global__ void {name}({ctype(o.dtype)}* __restrict__ out) {{\n'
            f"  long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x;\n  if (e >= {total}LL) return;\n"
            f"  out[e] = ({ctype(o.dtype)})((e / {inner}LL) % {o.shape[n.attrs['dim']]}LL);\n}}\n")
        self.launches.append(Launch(name, ((total + 255) // 256, 1, 1), (256, 1, 1), 0, [{"buffer": buf, "offset": 0}]))
        self.views[o.id] = self.contiguous_view(buf, o.shape, o.dtype)

    def lower_concat(self, n):
        o = n.outputs[0]
        buf = self.new_buffer(o.shape, o.dtype)
        full = self.contiguous_view(buf, o.shape, o.dtype)
        axis, off = n.attrs["axis"], 0
        for x in n.inputs:
            dst = View(buf, x.shape, full.strides, off * full.strides[axis], o.dtype)
            self.emit_pointwise([("copy", [("in", self.view_of(x))], {}, o.dtype)], [dst], x.shape, loc=n.loc)
            off += x.shape[axis]
        self.views[o.id] = full

    def lower_pad(self, n):
        x, pv = n.inputs
        o = n.outputs[0]
        xv, pvv = self.view_of(x), self.view_of(pv)
        name = self.kname("pad")
        buf = self.new_buffer(o.shape, o.dtype)
        nd = len(o.shape)
        lines = [f"  long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x;", f"  if (e >= {o.size}LL) return;",
                 "  long long r = e; bool inside = true; long long src = 0;"]
        for d in range(nd - 1, -1, -1):
            lines.append(f"  {{ long long i = r % {o.shape[d]}; r /= {o.shape[d]}; long long j = i - {n.attrs['low'][d]};"
                         f" inside = inside && j >= 0 && j < {x.shape[d]}; src += j * {xv.strides[d]}LL; }}")
        lines.append("  out[e] = inside ? x[src] : pv[0];")
        t = ctype(o.dtype)
        self.kernels.append(f'extern "C" __global__ void {name}(const {t}* __restrict__ x, const {t}* __restrict__ pv, '
                            f"{t}* __restrict__ out) {{\n" + "\n".join(lines) + "\n}\n")
        self.launches.append(Launch(name, ((o.size + 255) // 256, 1, 1), (256, 1, 1), 0, [
            {"buffer": xv.buffer, "offset": xv.offset * xv.dtype.itemsize},
            {"buffer": pvv.buffer, "offset": pvv.offset * pvv.dtype.itemsize}, {"buffer": buf, "offset": 0}]))
        self.views[o.id] = self.contiguous_view(buf, o.shape, o.dtype)

    def lower_reduce(self, n):
        x, o = n.inputs[0], n.outputs[0]
        xv = self.view_of(x)
        axes = sorted(n.attrs["axes"])
        kind = n.attrs["kind"]
        if not axes:
            return self.lower_copy(n)
        keep = [d for d in range(len(x.shape)) if d not in axes]
        kshape = [x.shape[d] for d in keep]
        rshape = [x.shape[d] for d in axes]
        outer = int(np.prod(kshape, dtype=np.int64))
        inner = int(np.prod(rshape, dtype=np.int64))
        ct = compute_type(o.dtype)
        init = {"sum": "0", "prod": "1", "and": "true", "or": "false",
                "max": "-INFINITY" if ct in ("float", "double") else f"({ct})({_int_min(o.dtype)})",
                "min": "INFINITY" if ct in ("float", "double") else f"({ct})({_int_max(o.dtype)})"}[kind]
        comb = {"sum": "acc + v", "prod": "acc * v", "and": "acc && v", "or": "acc || v",
                "max": "(v > acc ? v : acc)", "min": "(v < acc ? v : acc)"}[kind]
        name = self.kname("reduce")
        buf = self.new_buffer(o.shape, o.dtype)
        t_in, t_out = ctype(x.dtype), ctype(o.dtype)
        lines = ["  const int lane = threadIdx.x & 31;",
                 "  const long long w = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;",
                 f"  if (w >= {max(outer, 1)}LL) return;", "  long long base = 0; { long long r = w;"]
        for d, dim in zip(reversed(keep), reversed(kshape)):
            lines.append(f"    base += (r % {dim}) * {xv.strides[d]}LL; r /= {dim};")
        lines.append("  }")
        lines.append(f"  {ct} acc = {init};")
        lines.append(f"  for (long long j = lane; j < {inner}LL; j += 32) {{ long long r = j, off = base;")
        for d, dim in zip(reversed(axes), reversed(rshape)):
            lines.append(f"    off += (r % {dim}) * {xv.strides[d]}LL; r /= {dim};")
        lines.append(f"    const {ct} v = ld<{ct}>(x, off); acc = {comb}; }}")
        lines.append("  for (int o = 16; o; o >>= 1) {")
        if ct == "bool":
            lines.append("    const bool v = __shfl_xor_sync(~0u, (int)acc, o) != 0;")
        elif ct in ("long long", "unsigned long long", "double"):
            lines.append(f"    const {ct} v = __shfl_xor_sync(~0u, acc, o);")
        else:
            lines.append(f"    const {ct} v = ({ct})__shfl_xor_sync(~0u, acc, o);")
        lines.append(f"    acc = {comb}; }}")
        lines.append("  if (lane == 0) st(out, w, acc);")
        self.kernels.append(f'extern "C" __global__ void {name}(const {t_in}* __restrict__ x, {t_out}* __restrict__ out) '
                            "{\n" + "\n".join(lines) + "\n}\n")
        warps = max(outer, 1)
        self.launches.append(Launch(name, ((warps * 32 + 255) // 256, 1, 1), (256, 1, 1), 0, [
            {"buffer": xv.buffer, "offset": xv.offset * xv.dtype.itemsize}, {"buffer": buf, "offset": 0}],
            f"{n.loc[0]}:{n.loc[1]}" if n.loc else None))
        self.views[o.id] = self.contiguous_view(buf, o.shape, o.dtype)

    # -- dot -----------------------------------------------------------------------------
    def lower_dot(self, n, epilogue: Optional[List[Node]] = None):
        a, b = n.inputs
        o = n.outputs[0]
        at = n.attrs
        lb, rb, lc, rc = at["lhs_batch"], at["rhs_batch"], at["lhs_contract"], at["rhs_contract"]
        lfree = [i for i in range(len(a.shape)) if i not in lb and i not in lc]
        rfree = [i for i in range(len(b.shape)) if i not in rb and i not in rc]
        av, bv = self.view_of(a), self.view_of(b)
        # canonical 3-D strided operands: A[batch, M, K], B[batch, K, N]; multi-dim groups need dense merges
        def group(vw: View, dims: List[int]):
            if not dims:
                return 1, 0
            size = int(np.prod([vw.shape[d] for d in dims], dtype=np.int64))
            stride = vw.strides[dims[-1]]
            exp = stride
            for d in reversed(dims):
                if vw.shape[d] != 1 and vw.strides[d] != exp:
                    return size, None
                exp *= vw.shape[d]
            return size, stride

        def canon(val: Value, vw: View, groups):
            res = [group(vw, gdims) for gdims in groups]
            if any(s is None for _, s in res):
                vw = self.materialize(val)
                res = [group(vw, gdims) for gdims in groups]
            return vw, res

        av, (ab, am, ak) = canon(a, av, [lb, lfree, lc])
        bv, (bb, bk, bn) = canon(b, bv, [rb, rc, rfree])
        B, M, K, N = ab[0], am[0], ak[0], bn[0]
        buf = self.new_buffer(o.shape, o.dtype)
        self.views[o.id] = self.contiguous_view(buf, o.shape, o.dtype)
        if B * M * N == 0:
            self._flush(list(epilogue or []))
            return
        # the layout pass may have ruled the tensor-core path out for this node ("_path": "simt")
        want_tc = n.attrs.get("_path", "tcgen05") == "tcgen05"
        if (self.use_tcgen05 and want_tc and dtype_name(a.dtype) == "bf16" and B == 1 and K % 8 == 0 and N % 8 == 0
                and ak[1] == 1 and am[1] % 8 == 0 and av.offset % 8 == 0 and K >= 16):
            return self._dot_tcgen05(n, av, bv, (am, ak), (bk, bn), M, N, K, buf, epilogue=epilogue)
        name = self.kname("gemm_simt")
        ta, tb, to = ctype(a.dtype), ctype(b.dtype), ctype(o.dtype)
        acc = "double" if dtype_name(o.dtype) == "f64" else ("float" if compute_type(o.dtype) == "float" else
                                                             compute_type(o.dtype))
        self.kernels.append(f"""extern "C" __global__ void {name}(const {ta}* __restrict__ A, const {tb}* __restrict__ Bm, {to}* __restrict__ C) {{
  __shared__ {acc} As[16][17];
  __shared__ {acc} Bs[16][17];
  const int tx = threadIdx.x, ty = threadIdx.y;
  const long long bz = blockIdx.z;
  const long long row = blockIdx.y * 16LL + ty, col = blockIdx.x * 16LL + tx;
  {acc} acc = 0;
  for (long long k0 = 0; k0 < {K}LL; k0 += 16) {{
    As[ty][tx] = (row < {M}LL && k0 + tx < {K}LL) ? ld<{acc}>(A, bz * {ab[1]}LL + row * {am[1]}LL + (k0 + tx) * {ak[1]}LL) : ({acc})0;
    Bs[ty][tx] = (col < {N}LL && k0 + ty < {K}LL) ? ld<{acc}>(Bm, bz * {bb[1]}LL + (k0 + ty) * {bk[1]}LL + col * {bn[1]}LL) : ({acc})0;
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 16; ++k) acc += As[ty][k] * Bs[k][tx];
    __syncthreads();
  }}
  if (row < {M}LL && col < {N}LL) st(C, bz * {M * N}LL + row * {N}LL + col, acc);
}}
""")
        self.launches.append(Launch(name, ((N + 15) // 16, (M + 15) // 16, B), (16, 16, 1), 0, [
            {"buffer": av.buffer, "offset": av.offset * av.dtype.itemsize},
            {"buffer": bv.buffer, "offset": bv.offset * bv.dtype.itemsize}, {"buffer": buf, "offset": 0}],
            f"{n.loc[0]}:{n.loc[1]}" if n.loc else None))
        self._flush(list(epilogue or []))

    def _dot_tcgen05(self, n, av: View, bv: View, a_ms, b_ks, M, N, K, out_buf, epilogue=None):
        """bf16 GEMM on the hand-written tcgen05 kernel: A [M, K] K-major via TMA; B must be [N, K]
        K-major, so a [K, N] operand is transposed once into a temporary.

        What the native pass pipeline decided for this node is taken from its attributes: the CTA tile width
        and the persistent grid from `_tiling` (knob-driven-tiling, i.e. the user's `knob(x).tile_op(...)`), the
        ring depth from `_stages` (insert-spill-reload, which shrinks it to the shared-memory budget), and the
        elementwise epilogue chain from knob-driven-fusion (`epilogue`), which is compiled into a functor
        that the GEMM applies to the fp32 accumulator before its single store."""
        (am, ak), (bk, bn) = a_ms, b_ks
        if not (bk[1] == 1 and bn[1] % 8 == 0 and bv.offset % 8 == 0):
            tmp = self.new_buffer((N, K), bfloat16)
            tv = self.contiguous_view(tmp, (N, K), bfloat16)
            src = View(bv.buffer, (N, K), (bn[1], bk[1]), bv.offset, bv.dtype)
            self.emit_pointwise([("copy", [("in", src)], {}, bfloat16)], [tv], (N, K), loc=n.loc)
            bv, ldb = tv, K
        else:
            ldb = bn[1]
        self.uses_tcgen05 = True
        name = self.kname("gemm_tcgen05")
        bn_tile = 256 if N >= 256 else (128 if N > 64 else 64 if N > 32 else 32)
        tiling = n.attrs.get("_tiling") or {}
        cta = tiling.get("cta_tile")
        if cta and len(cta) >= 2 and int(cta[1]) in (32, 64, 128, 256):
            bn_tile = int(cta[1])
        stage_bytes = 128 * 64 * 2 + bn_tile * 64 * 2
        max_stages = min(12, (232448 - 1024 - 512 - 64) // stage_bytes)
        stages = max_stages
        want_stages = n.attrs.get("_stages", tiling.get("stages"))
        if want_stages:
            stages = max(2, min(int(want_stages), max_stages))
        smem = stages * stage_bytes + 1024 + 512 + 64
        tiles = ((M + 127) // 128) * ((N + bn_tile - 1) // bn_tile)
        grid = min(tiles, 148)
        if tiling.get("grid"):
            grid = max(1, min(int(tiling["grid"]), tiles, 148))
        extra_params, extra_args, functor = "", [], ""
        ee_type, ee_make = "nkb::NoElemEpi", ""
        if epilogue:
            functor, ptr_params, extra_args, ee_type = self._epilogue_functor(name, n, epilogue)
            extra_params = "".join(f", {p}" for p in ptr_params)
            ee_make = f"  const {ee_type} ee{{{', '.join(f'p{i}' for i in range(len(ptr_params)))}}};\n"
            last = epilogue[-1].outputs[0]
            self.views[last.id] = self.contiguous_view(out_buf, last.shape, last.dtype)
        body_call = (f"  nkb::gemm_bf16_body<{bn_tile}, false, false, nkb::NoFix, {ee_type}>(tmA, tmB, args, "
                     f"nkb::PushArgs{{}}, nkb::GroupArgs{{}}, nkb::NoFix::Args{{}}"
                     + (", ee" if epilogue else f", {ee_type}{{}}") + ");")
        self.kernels.append(functor + f"""extern "C" __global__ void __launch_bounds__(nkb::kGemmThreads, 1)
{name}(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const nkb::GemmArgs args,
       const nkb::PushArgs{extra_params}) {{
{ee_make}{body_call}
}}
""")
        self.launches.append(Launch(name, (grid, 1, 1), (192, 1, 1), smem, [
            {"tensormap": {"buffer": av.buffer, "offset": av.offset * 2, "dims": [K, M], "strides": [am[1] * 2],
                           "box": [64, 128]}},
            {"tensormap": {"buffer": bv.buffer, "offset": bv.offset * 2, "dims": [K, N], "strides": [ldb * 2],
                           "box": [64, bn_tile]}},
            {"gemm_args": {"rows": M, "cols": N, "k": K, "block_n": bn_tile, "stages": stages, "ldo": N,
                           "out_buffer": out_buf, "out_offset": 0,
                           "fused_epilogue": [c.opcode for c in epilogue] if epilogue else []}}] + extra_args,
            f"{n.loc[0]}:{n.loc[1]}" if n.loc else None))

    def _epilogue_functor(self, kname: str, dot: Node, chain: List[Node]):
        """C++ functor `float operator()(float acc, long long i0, long long i1)` for an elementwise chain rooted
        at the dot's result; operands that are not chain values are read through their [M, N] views."""
        shape = tuple(dot.outputs[0].shape)
        params: List[str] = []
        args: List[Dict[str, Any]] = []
        loads: Dict[Tuple, str] = {}
        body: List[str] = []
        inside = {dot.outputs[0].id} | {c.outputs[0].id for c in chain}

        def index_expr(vw: View) -> str:
            if len(vw.shape) != 2:
                raise CodegenError("epilogue operand is not two-dimensional")
            terms = [f"i{d} * {s}LL" for d, s in enumerate(vw.strides) if s != 0 and shape[d] != 1]
            return " + ".join(terms) if terms else "0"

        def operand(val: Value, want_ctype: str) -> str:
            if val.id in inside:
                return f"v{val.id}"
            vw = self.view_of(val)
            key = (vw.buffer, vw.offset, vw.strides, want_ctype)
            if key not in loads:
                pname = f"p{len(params)}"
                params.append(f"const {ctype(vw.dtype)}* __restrict__ {pname}")
                args.append({"buffer": vw.buffer, "offset": vw.offset * vw.dtype.itemsize})
                var = f"l{len(loads)}"
                body.append(f"    const {want_ctype} {var} = ld<{want_ctype}>({pname}, {index_expr(vw)});")
                loads[key] = var
            return loads[key]

        body.append(f"    const float v{dot.outputs[0].id} = acc;")
        for c in chain:
            o = c.outputs[0]
            in_dts = [i.dtype for i in c.inputs]
            a = [operand(i, compute_type(dt)) for i, dt in zip(c.inputs, in_dts)]
            ct = compute_type(o.dtype)
            body.append(f"    const {ct} v{o.id} = {self._expr(c.opcode, a, dict(c.attrs), o.dtype, in_dts)};")
        tname = f"Epi_{kname}"
        fields = "".join(f"  {p.replace(' __restrict__', '')};\n" for p in params)
        src = (f"struct {tname} {{\n  static constexpr bool active = true;\n{fields}"
               f"  __device__ __forceinline__ float operator()(float acc, long long i0, long long i1) const {{\n"
               + "\n".join(body) + f"\n    return float(v{chain[-1].outputs[0].id});\n  }}\n}};\n")
        return src, params, args, tname

    # -- gathers / scatters -----------------------------------------------------------
    def _simple(self, name_base, n, params: List[Tuple[str, View, bool]], body_lines: List[str], total: int):
        name = self.kname(name_base)
        sig = ", ".join(f"{'const ' if c else ''}{ctype(v.dtype)}* __restrict__ {p}" for p, v, c in params)
        head = [f"  long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x;", f"  if (e >= {total}LL) return;"]
        self.kernels.append(f'extern "C" __global__ void {name}({sig}) {{\n' + "\n".join(head + body_lines) + "\n}\n")
        self.launches.append(Launch(name, ((max(total, 1) + 255) // 256, 1, 1), (256, 1, 1), 0, [
            {"buffer": v.buffer, "offset": v.offset * v.dtype.itemsize} for _, v, _ in params],
            f"{n.loc[0]}:{n.loc[1]}" if n.loc else None))

    def _out(self, o: Value) -> View:
        buf = self.new_buffer(o.shape, o.dtype)
        vw = self.contiguous_view(buf, o.shape, o.dtype)
        self.views[o.id] = vw
        return vw

    def lower_take(self, n):
        x, idx = n.inputs
        o = n.outputs[0]
        xv, iv = self.view_of(x), self.materialize(idx)
        axis = n.attrs["axis"]
        post = int(np.prod(x.shape[axis + 1:], dtype=np.int64))
        cnt = max(idx.size, 1)
        ov = self._out(o)
        lines = [f"  const long long post = e % {post}LL; long long r = e / {post}LL;",
                 f"  const long long k = r % {cnt}LL; long long pre = r / {cnt}LL;",
                 f"  long long j = (long long)idx[k]; if (j < 0) j += {x.shape[axis]}; "
                 f"j = j < 0 ? 0 : (j >= {x.shape[axis]} ? {x.shape[axis] - 1} : j);",
                 f"  long long off = j * {xv.strides[axis]}LL;"]
        lines.append("  { long long q = post;")
        for d in range(len(x.shape) - 1, axis, -1):
            lines.append(f"    off += (q % {x.shape[d]}) * {xv.strides[d]}LL; q /= {x.shape[d]};")
        lines.append("    q = pre;")
        for d in range(axis - 1, -1, -1):
            lines.append(f"    off += (q % {x.shape[d]}) * {xv.strides[d]}LL; q /= {x.shape[d]};")
        lines.append("  }")
        lines.append("  out[e] = x[off];")
        if o.size:
            self._simple("take", n, [("x", xv, True), ("idx", iv, True), ("out", ov, False)], lines, o.size)

    def lower_take_along_axis(self, n):
        x, idx = n.inputs
        o = n.outputs[0]
        xv, iv = self.view_of(x), self.view_of(idx)
        axis = n.attrs["axis"]
        ov = self._out(o)
        lines = ["  long long r = e, xo = 0, io = 0, j = 0;"]
        for d in range(len(o.shape) - 1, -1, -1):
            lines.append(f"  {{ const long long i = r % {o.shape[d]}; r /= {o.shape[d]}; io += i * {iv.strides[d]}LL;"
                         + (f" xo += i * {xv.strides[d]}LL; }}" if d != axis else " }"))
        lines.append(f"  j = (long long)idx[io]; if (j < 0) j += {x.shape[axis]}; "
                     f"j = j < 0 ? 0 : (j >= {x.shape[axis]} ? {x.shape[axis] - 1} : j);")
        lines.append(f"  out[e] = x[xo + j * {xv.strides[axis]}LL];")
        if o.size:
            self._simple("take_along", n, [("x", xv, True), ("idx", iv, True), ("out", ov, False)], lines, o.size)

    def _copy_into_new(self, x: Value, o: Value, n) -> View:
        ov = self._out(o)
        self.emit_pointwise([("copy", [("in", self.view_of(x))], {}, o.dtype)], [ov], o.shape, loc=n.loc)
        return ov

    def lower_put_along_axis(self, n):
        x, idx, upd = n.inputs
        o = n.outputs[0]
        ov = self._copy_into_new(x, o, n)
        iv, uv = self.view_of(idx), self.view_of(upd)
        axis = n.attrs["axis"]
        lines = ["  long long r = e, oo = 0, io = 0, uo = 0;"]
        ost = _contig_strides(o.shape)
        for d in range(len(idx.shape) - 1, -1, -1):
            lines.append(f"  {{ const long long i = r % {idx.shape[d]}; r /= {idx.shape[d]}; io += i * {iv.strides[d]}LL; "
                         f"uo += i * {uv.strides[d]}LL;" + (f" oo += i * {ost[d]}LL; }}" if d != axis else " }"))
        lines.append(f"  long long j = (long long)idx[io]; if (j < 0) j += {o.shape[axis]};")
        lines.append(f"  if (j >= 0 && j < {o.shape[axis]}) out[oo + j * {ost[axis]}LL] = upd[uo];")
        if idx.size:
            self._simple("put_along", n, [("idx", iv, True), ("upd", uv, True), ("out", ov, False)], lines, idx.size)

    def lower_scatter_along_axis(self, n):
        x, idx, upd = n.inputs
        o = n.outputs[0]
        ov = self._copy_into_new(x, o, n)
        iv, uv = self.view_of(idx), self.view_of(upd)
        axis = n.attrs["axis"]
        ost = _contig_strides(o.shape)
        lines = ["  long long r = e, oo = 0, uo = 0, k = 0;"]
        for d in range(len(upd.shape) - 1, -1, -1):
            lines.append(f"  {{ const long long i = r % {upd.shape[d]}; r /= {upd.shape[d]}; uo += i * {uv.strides[d]}LL;"
                         + (f" oo += i * {ost[d]}LL; }}" if d != axis else " k = i; }"))
        lines.append(f"  long long j = (long long)idx[k * {iv.strides[0]}LL]; if (j < 0) j += {o.shape[axis]};")
        lines.append(f"  if (j >= 0 && j < {o.shape[axis]}) out[oo + j * {ost[axis]}LL] = upd[uo];")
        if upd.size:
            self._simple("scatter_axis", n, [("idx", iv, True), ("upd", uv, True), ("out", ov, False)], lines, upd.size)

    def lower_update_slice(self, n):
        x, upd = n.inputs
        o = n.outputs[0]
        ov = self._copy_into_new(x, o, n)
        ost = _contig_strides(o.shape)
        off = sum(s * st for s, st in zip(n.attrs["start"], ost))
        dst = View(ov.buffer, upd.shape, tuple(st * k for st, k in zip(ost, n.attrs["stride"])), off, o.dtype)
        self.emit_pointwise([("copy", [("in", self.view_of(upd))], {}, o.dtype)], [dst], upd.shape, loc=n.loc)

    def lower_dynamic_update_slice(self, n):
        x, upd = n.inputs[0], n.inputs[1]
        starts = n.inputs[2:]
        o = n.outputs[0]
        ov = self._copy_into_new(x, o, n)
        uv = self.view_of(upd)
        ost = _contig_strides(o.shape)
        params = [("upd", uv, True), ("out", ov, False)]
        lines = ["  long long r = e, oo = 0, uo = 0;"]
        for d in range(len(upd.shape) - 1, -1, -1):
            sv = self.view_of(starts[d])
            params.append((f"s{d}", sv, True))
            lines.append(f"  {{ const long long i = r % {upd.shape[d]}; r /= {upd.shape[d]}; long long s = (long long)s{d}[0];"
                         f" s = s < 0 ? 0 : (s > {o.shape[d] - upd.shape[d]} ? {o.shape[d] - upd.shape[d]} : s);"
                         f" oo += (s + i) * {ost[d]}LL; uo += i * {uv.strides[d]}LL; }}")
        lines.append("  out[oo] = upd[uo];")
        if upd.size:
            self._simple("dyn_update", n, params, lines, upd.size)

    def lower_dynamic_slice(self, n):
        x = n.inputs[0]
        starts = n.inputs[1:]
        o = n.outputs[0]
        xv = self.view_of(x)
        ov = self._out(o)
        params = [("x", xv, True), ("out", ov, False)]
        lines = ["  long long r = e, xo = 0;"]
        for d in range(len(o.shape) - 1, -1, -1):
            sv = self.view_of(starts[d])
            params.append((f"s{d}", sv, True))
            lines.append(f"  {{ const long long i = r % {o.shape[d]}; r /= {o.shape[d]}; long long s = (long long)s{d}[0];"
                         f" s = s < 0 ? 0 : (s > {x.shape[d] - o.shape[d]} ? {x.shape[d] - o.shape[d]} : s);"
                         f" xo += (s + i) * {xv.strides[d]}LL; }}")
        lines.append("  out[e] = x[xo];")
        if o.size:
            self._simple("dyn_slice", n, params, lines, o.size)

    def lower_topk(self, n):
        x = n.inputs[0]
        vals, idx = n.outputs
        xv = self.materialize(x)
        k, width = n.attrs["k"], x.shape[-1]
        rows = x.size // max(width, 1)
        vv, iv = self._out(vals), self._out(idx)
        name = self.kname("topk")
        t = ctype(x.dtype)
        # one warp per row; k rounds of (max value, lowest index) selection, previous winners excluded
        self.kernels.append(f"""extern "C" __global__ void {name}(const {t}* __restrict__ x, {t}* __restrict__ vals, unsigned int* __restrict__ idx) {{
  const int lane = threadIdx.x & 31;
  const long long row = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  if (row >= {rows}LL) return;
  const {t}* xr = x + row * {width}LL;
  float prev_v = INFINITY; int prev_i = -1;
  for (int r = 0; r < {k}; ++r) {{
    float best = -INFINITY; int bi = 0x7fffffff;
    for (int j = lane; j < {width}; j += 32) {{
      const float v = ld<float>(xr, j);
      const bool after = (v < prev_v) || (v == prev_v && j > prev_i);
      if (after && (v > best || (v == best && j < bi))) {{ best = v; bi = j; }}
    }}
    for (int o = 16; o; o >>= 1) {{
      const float ov = __shfl_xor_sync(~0u, best, o); const int oi = __shfl_xor_sync(~0u, bi, o);
      if (ov > best || (ov == best && oi < bi)) {{ best = ov; bi = oi; }}
    }}
    if (lane == 0) {{ vals[row * {k}LL + r] = xr[bi < {width} ? bi : 0]; idx[row * {k}LL + r] = (unsigned int)bi; }}
    prev_v = best; prev_i = bi;
  }}
}}
""")
        self.launches.append(Launch(name, ((rows * 32 + 127) // 128, 1, 1), (128, 1, 1), 0, [
            {"buffer": xv.buffer, "offset": 0}, {"buffer": vv.buffer, "offset": 0}, {"buffer": iv.buffer, "offset": 0}]))

    def lower_conv(self, n):
        x, w = n.inputs[0], n.inputs[1]
        b = n.inputs[2] if len(n.inputs) > 2 else None
        o = n.outputs[0]
        xv, wv = self.materialize(x), self.materialize(w)
        ov = self._out(o)
        nsp = len(x.shape) - 2
        at = n.attrs
        C, O = x.shape[1], w.shape[0]
        cg, og = C // at["groups"], O // at["groups"]
        params = [("x", xv, True), ("w", wv, True), ("out", ov, False)]
        if b is not None:
            params.append(("bias", self.materialize(b), True))
        lines = ["  long long r = e;"]
        for d in range(nsp - 1, -1, -1):
            lines.append(f"  const long long o{d} = r % {o.shape[2 + d]}; r /= {o.shape[2 + d]};")
        lines.append(f"  const long long oc = r % {O}; const long long nb = r / {O}; const long long g = oc / {og};")
        lines.append("  float acc = 0.f;")
        lines.append(f"  for (long long c = 0; c < {cg}; ++c) {{")
        for d in range(nsp):
            lines.append(f"  for (long long k{d} = 0; k{d} < {w.shape[2 + d]}; ++k{d}) {{ const long long p{d} = o{d} * "
                         f"{at['stride'][d]} - {at['padding'][d]} + k{d} * {at['dilation'][d]}; "
                         f"if (p{d} < 0 || p{d} >= {x.shape[2 + d]}) continue;")
        xs, ws = _contig_strides(x.shape), _contig_strides(w.shape)
        xoff = f"nb * {xs[0]}LL + (g * {cg} + c) * {xs[1]}LL" + "".join(f" + p{d} * {xs[2 + d]}LL" for d in range(nsp))
        woff = f"oc * {ws[0]}LL + c * {ws[1]}LL" + "".join(f" + k{d} * {ws[2 + d]}LL" for d in range(nsp))
        lines.append(f"    acc += ld<float>(x, {xoff}) * ld<float>(w, {woff});")
        lines.append("  " + "}" * nsp + " }")
        if b is not None:
            lines.append("  acc += ld<float>(bias, oc);")
        lines.append("  st(out, e, acc);")
        if o.size:
            self._simple("conv", n, params, lines, o.size)

    # ------------------------------------------------------------------ row operations (one warp per row)
    def _row_kernel(self, n, base: str, body: List[str], extra_params: List[Tuple[str, View]] = ()):
        """Emit a kernel in which one warp owns one row of the (dense) input over its last axis: `L` is the row
        length, `x` / `out` point at the row, `lane` is the lane; fp32 arithmetic, shuffles for the row sums."""
        x, o = n.inputs[0], n.outputs[0]
        xv = self.materialize(x)
        ov = self._out(o)
        L = x.shape[-1]
        rows = max(x.size // max(L, 1), 1)
        ct = ctype(x.dtype)
        name = self.kname(base)
        sig = f"const {ct}* __restrict__ xin, {ct}* __restrict__ oout" + "".join(
            f", const {ctype(v.dtype)}* __restrict__ {p}" for p, v in extra_params)
        head = [f"  const long long row = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;",
                f"  const int lane = threadIdx.x & 31;",
                f"  if (row >= {rows}LL) return;",
                f"  const {ct}* x = xin + row * {L}LL; {ct}* out = oout + row * {L}LL;",
                f"  const int L = {L};"]
        self.kernels.append(f'extern "C" __global__ void {name}({sig}) {{\n' + "\n".join(head + body) + "\n}\n")
        self.launches.append(Launch(name, ((rows * 32 + 255) // 256, 1, 1), (256, 1, 1), 0,
                                    [{"buffer": xv.buffer, "offset": xv.offset * x.dtype.itemsize},
                                     {"buffer": ov.buffer, "offset": 0}]
                                    + [{"buffer": v.buffer, "offset": v.offset * v.dtype.itemsize} for _, v in extra_params],
                                    f"{n.loc[0]}:{n.loc[1]}" if n.loc else None))

    def lower_softmax(self, n):
        """softmax over the last axis in one launch: running maximum, exponentials and their sum per warp."""
        body = ["  float m = -INFINITY;",
                "  for (int i = lane; i < L; i += 32) m = fmaxf(m, ld<float>(x, i));",
                "  for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(~0u, m, o));",
                "  float s = 0.f;",
                "  for (int i = lane; i < L; i += 32) s += expf(ld<float>(x, i) - m);",
                "  s = warp_reduce_sum(s);",
                "  const float inv = 1.f / s;",
                "  for (int i = lane; i < L; i += 32) st(out, i, expf(ld<float>(x, i) - m) * inv);"]
        if n.outputs[0].size:
            self._row_kernel(n, "softmax", body)
        else:
            self._out(n.outputs[0])

    def lower_rms_norm(self, n):
        """RMSNorm over the last axis in one launch (fp32 statistics, eps inside the root, optional weight)."""
        eps = float(n.attrs["eps"])
        has_w = len(n.inputs) > 1
        body = ["  float ss = 0.f;",
                "  for (int i = lane; i < L; i += 32) { const float v = ld<float>(x, i); ss += v * v; }",
                "  ss = warp_reduce_sum(ss);",
                f"  const float inv = 1.f / sqrtf(ss / float(L) + {eps!r}f);",
                "  for (int i = lane; i < L; i += 32) st(out, i, ld<float>(x, i) * inv"
                + (" * ld<float>(w, i));" if has_w else ");")]
        extra = [("w", self.materialize(n.inputs[1]))] if has_w else []
        if n.outputs[0].size:
            self._row_kernel(n, "rms_norm", body, extra)
        else:
            self._out(n.outputs[0])

    def _collective(self, n):
        """A collective as two kernels of the module itself: every rank stores its operand into slot [rank] of
        all ranks' symmetric workspace (`cc_push`), then builds the result from the slots (`cc_consume`):
        a reduction over the slots (all_reduce, reduce_scatter) or a re-indexing of them (all_gather,
        all_to_all).  The runtime supplies the workspace and the peer table when the module is loaded with
        collectives enabled (reference: spike/src/model.cpp:38-46 loads collectives with the program)."""
        x, o = n.inputs[0], n.outputs[0]
        at = n.attrs
        groups = at.get("replica_groups") or [[0]]
        world = len(groups[0])
        if any(len(g) != world for g in groups):
            raise CodegenError("replica groups of different sizes")
        if world > 8:
            raise CodegenError("collectives inside a module support up to 8 ranks (one NVSwitch domain)")
        xv = self.materialize(x)
        ov = self._out(o)
        ct = ctype(x.dtype)
        acc = compute_type(x.dtype)
        nelem = max(x.size, 1)
        self.cc_world = max(getattr(self, "cc_world", 1), world)
        self.cc_half_bytes = max(getattr(self, "cc_half_bytes", 0), world * nelem * x.dtype.itemsize)
        loc = f"{n.loc[0]}:{n.loc[1]}" if n.loc else None
        push = self.kname("cc_push")
        self.kernels.append(f'extern "C" __global__ void {push}(const {ct}* __restrict__ in, const CcTable* __restrict__ t) '
                            f'{{\n  cc_push<{ct}>(in, {nelem}LL, *t);\n}}\n')
        grid = min(max((nelem + 255) // 256, 1), 296)
        self.launches.append(Launch(push, (grid, 1, 1), (256, 1, 1), 0,
                                    [{"buffer": xv.buffer, "offset": xv.offset * x.dtype.itemsize}, {"cc": "table"}], loc))
        # consumer: output element e -> source slot(s) and element
        shape_in, shape_out = list(x.shape), list(o.shape)
        strides_in = _contig_strides(shape_in)
        red = {"add": "a + b", "multiply": "a * b", "maximum": "(a > b ? a : b)", "minimum": "(a < b ? a : b)"}
        lines = [f"  const unsigned int use = *reinterpret_cast<volatile unsigned int*>(t->seen);",
                 f"  const bool ok = cc_wait(*t, use);",
                 f"  const {ct}* slots = reinterpret_cast<const {ct}*>(t->local_ws + kCcFlagBytes + "
                 f"(long long)(use & 1u) * t->half_bytes);",
                 f"  for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; ok && e < {max(o.size, 1)}LL; "
                 f"e += (long long)gridDim.x * blockDim.x) {{"]
        op = n.opcode
        if op == "all_reduce":
            lines += [f"    {acc} a = ld<{acc}>(slots, e);",
                      f"    for (int s = 1; s < {world}; ++s) {{ const {acc} b = ld<{acc}>(slots, (long long)s * {nelem}LL + e); "
                      f"a = {red[at.get('op', 'add')]}; }}",
                      f"    st(out, e, a);"]
        else:
            # coordinates of the output element
            lines.append("    long long r = e, src = 0; int slot = 0;")
            dims = {"all_gather": (at.get("dim"), None), "reduce_scatter": (at.get("dim"), None),
                    "all_to_all": (at.get("concat_dim"), at.get("split_dim"))}[op]
            for d in range(len(shape_out) - 1, -1, -1):
                lines.append(f"    {{ long long c = r % {shape_out[d]}; r /= {shape_out[d]};")
                if op == "all_gather" and d == dims[0]:
                    lines.append(f"      slot = int(c / {shape_in[d]}); c = c % {shape_in[d]};")
                elif op == "reduce_scatter" and d == dims[0]:
                    lines.append(f"      c += (long long)t->rank * {shape_out[d]};")
                elif op == "all_to_all" and d == dims[0] and d == dims[1]:
                    # split and concatenation on the same axis: block j of the result is block `rank` of rank j
                    lines.append(f"      slot = int(c / {shape_out[d] // world}); "
                                 f"c = c % {shape_out[d] // world} + (long long)t->rank * {shape_in[d] // world};")
                elif op == "all_to_all" and d == dims[0]:
                    lines.append(f"      slot = int(c / {shape_in[d]}); c = c % {shape_in[d]};")
                elif op == "all_to_all" and d == dims[1]:
                    lines.append(f"      c += (long long)t->rank * {shape_out[d]};")
                lines.append(f"      src += c * {strides_in[d]}LL; }}")
            if op == "reduce_scatter":
                lines += [f"    {acc} a = ld<{acc}>(slots, src);",
                          f"    for (int s = 1; s < {world}; ++s) {{ const {acc} b = ld<{acc}>(slots, (long long)s * {nelem}LL + src); "
                          f"a = {red[at.get('op', 'add')]}; }}",
                          f"    st(out, e, a);"]
            else:
                lines.append(f"    out[e] = slots[(long long)slot * {nelem}LL + src];")
        lines += ["  }", "  cc_finish(*t, use, ok);"]
        cons = self.kname("cc_" + op)
        self.kernels.append(f'extern "C" __global__ void {cons}({ct}* __restrict__ out, const CcTable* __restrict__ t) {{\n'
                            + "\n".join(lines) + "\n}\n")
        grid = min(max((max(o.size, 1) + 255) // 256, 1), 296)
        self.launches.append(Launch(cons, (grid, 1, 1), (256, 1, 1), 0,
                                    [{"buffer": ov.buffer, "offset": 0}, {"cc": "table"}], loc))

    lower_all_gather = lower_all_reduce = lower_reduce_scatter = lower_all_to_all = _collective

    def lower_custom_call(self, n):
        """Hand-written kernel: its source is emitted verbatim; arguments are the operand
        pointers followed by the output pointers.  An output aliased to an operand starts as
        a copy of that operand (the kernel updates it in place)."""
        at = n.attrs
        if at["source"] not in self.kernels:
            self.kernels.append(at["source"])
        args = []
        for x in n.inputs:
            vw = self.materialize(x)
            args.append({"buffer": vw.buffer, "offset": 0})
        aliases = {int(k): int(v) for k, v in (at.get("aliases") or {}).items()}
        for i, o in enumerate(n.outputs):
            if i in aliases:
                ov = self._copy_into_new(n.inputs[aliases[i]], o, n)
            else:
                ov = self._out(o)
            args.append({"buffer": ov.buffer, "offset": 0})
        self.launches.append(Launch(at["entry"], tuple(at["grid"]), tuple(at["block"]), int(at.get("smem", 0)), args,
                                    f"{n.loc[0]}:{n.loc[1]}" if n.loc else None))


def _int_min(dt) -> str:
    return str(np.iinfo(np.dtype(dt)).min) if np.dtype(dt).kind in "iu" else "0"


def _int_max(dt) -> str:
    return str(np.iinfo(np.dtype(dt)).max) if np.dtype(dt).kind in "iu" else "1"


def generate(graph: Graph, use_tcgen05: bool = True) -> Program:
    return Generator(graph, use_tcgen05).run()


def lower_to_cuda(graph: Graph, use_tcgen05: bool = True) -> str:
    """CUDA C++ source generated for a traced graph."""
    return generate(graph, use_tcgen05).source
