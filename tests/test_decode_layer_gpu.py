"""The persistent decode-layer kernel (csrc/kernels/decode_layer.cu) against an fp32 PyTorch oracle of the
same chain written here: o_proj -> sum + residual + RMSNorm -> gate/up + SwiGLU -> down -> sum + residual +
RMSNorm -> QKV of the next layer -> bias, QK-norm, RoPE, cache append.  Single GPU (split-K partials summed
locally), one rank through the tensor-parallel push path, and 2+ ranks as child processes."""
import os
import socket
import sys

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEV = "cuda"
EPS = 1e-5


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def bf(t):
    return t.to(torch.bfloat16)


def rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-9)).item()


def check(out, ref, tol=1.5e-2):
    assert out.shape == ref.shape
    assert torch.isfinite(out.float()).all()
    assert rel(out, ref) < tol, rel(out, ref)
    scale = ref.float().abs().max().item() + 1e-6
    assert (out.float() - ref.float()).abs().max().item() < 0.06 * scale
    # every block of 8 rows x 128 columns on its own: one wrong tile or token slice cannot hide
    o, r = out.float().reshape(out.shape[0], -1), ref.float().reshape(ref.shape[0], -1)
    for c in range(0, o.shape[1], 128):
        for t in range(0, o.shape[0], 8):
            ob, rb = o[t:t + 8, c:c + 128], r[t:t + 8, c:c + 128]
            e = ((ob - rb).norm() / (rb.norm() + 1e-3 * scale * rb.numel() ** 0.5)).item()
            assert e < 4 * tol, (t, c, e)


class Case:
    """Random weights and inputs of one layer boundary, and the fp32 oracle."""

    def __init__(self, T, H, k_o, inter, nq, nkv, D, seed=0, biases=False, qk_norm=False, limit=0.0, dev=DEV,
                 ranks=1, rank=0):
        g = torch.Generator(device="cpu").manual_seed(seed)

        def rn(*shape, scale=1.0):
            return bf(torch.randn(*shape, generator=g) * scale)

        self.T, self.H, self.inter, self.nq, self.nkv, self.D, self.limit = T, H, inter, nq, nkv, D, limit
        self.ranks = ranks
        # full (unsharded) tensors; rank r takes its slice of the contraction of the two row-parallel GEMMs
        self.attn_full = rn(T, k_o * ranks)
        self.w_o_full = rn(H, k_o * ranks, scale=0.05)
        self.w_gu_full = rn(2 * inter * ranks, H, scale=0.05)       # [gate(all ranks) ; up(all ranks)]
        self.w_down_full = rn(H, inter * ranks, scale=0.05)
        self.w_qkv = rn((nq + 2 * nkv) * D, H, scale=0.05)
        self.resid = rn(T, H)
        self.n1, self.n2 = bf(1 + 0.1 * torch.randn(H, generator=g)), bf(1 + 0.1 * torch.randn(H, generator=g))
        self.bias_o = rn(H) if biases else None
        self.bias_gu_full = rn(2 * inter * ranks) if biases else None
        self.bias_down = rn(H) if biases else None
        self.bias_qkv = rn((nq + 2 * nkv) * D) if biases else None
        self.qn = bf(1 + 0.1 * torch.randn(D, generator=g)) if qk_norm else None
        self.kn = bf(1 + 0.1 * torch.randn(D, generator=g)) if qk_norm else None
        self.max_pos, self.bs, self.nblocks = 256, 32, 8
        self.pos = torch.randint(0, self.max_pos, (T,), generator=g, dtype=torch.int32)
        self.slots = torch.randperm(self.nblocks * self.bs, generator=g)[:T].to(torch.int32)
        if T > 2:
            self.slots[T // 2] = -1
        self.k_o = k_o
        self.dev = dev
        self.rank = rank

    # ---- this rank's shards on the device
    def shard(self):
        r, n, I, ko = self.rank, self.ranks, self.inter, self.k_o
        d = lambda t: None if t is None else t.to(self.dev).contiguous()  # noqa: E731
        gate = self.w_gu_full[:I * n][r * I:(r + 1) * I]
        up = self.w_gu_full[I * n:][r * I:(r + 1) * I]
        out = dict(attn=d(self.attn_full[:, r * ko:(r + 1) * ko]), w_o=d(self.w_o_full[:, r * ko:(r + 1) * ko]),
                   w_gu=d(torch.cat([gate, up])), w_down=d(self.w_down_full[:, r * I:(r + 1) * I]),
                   w_qkv=d(self.w_qkv), resid=d(self.resid), n1=d(self.n1), n2=d(self.n2),
                   bias_o=d(self.bias_o) if r == 0 else (None if self.bias_o is None else d(torch.zeros_like(self.bias_o))),
                   bias_down=d(self.bias_down) if r == 0 else (None if self.bias_down is None else d(torch.zeros_like(self.bias_down))),
                   bias_qkv=d(self.bias_qkv), qn=d(self.qn), kn=d(self.kn), pos=d(self.pos), slots=d(self.slots))
        if self.bias_gu_full is not None:
            bg = self.bias_gu_full[:I * n][r * I:(r + 1) * I]
            bu = self.bias_gu_full[I * n:][r * I:(r + 1) * I]
            out["bias_gu"] = d(torch.cat([bg, bu]))
        else:
            out["bias_gu"] = None
        return out

    # ---- fp32 oracle of the whole chain (all ranks together)
    def oracle(self, cos_sin):
        f = lambda t: t.float()  # noqa: E731
        n, I = self.ranks, self.inter

        def norm(h, w):
            return h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + EPS) * f(w)

        y = f(self.attn_full) @ f(self.w_o_full).T
        if self.bias_o is not None:
            y = y + f(self.bias_o)
        resid_mid = bf(y + f(self.resid)).float()
        normed_mid = bf(norm(resid_mid, self.n1)).float()
        gu = normed_mid @ f(self.w_gu_full).T
        if self.bias_gu_full is not None:
            gu = gu + f(self.bias_gu_full)
        gate, up = gu[:, :I * n], gu[:, I * n:]
        if self.limit > 0:
            gate, up = gate.clamp(max=self.limit), up.clamp(-self.limit, self.limit)
            act = (up + 1) * gate * torch.sigmoid(1.702 * gate)
        else:
            act = torch.nn.functional.silu(gate) * up
        act = bf(act).float()
        z = act @ f(self.w_down_full).T
        if self.bias_down is not None:
            z = z + f(self.bias_down)
        resid_out = bf(z + resid_mid).float()
        normed_out = bf(norm(resid_out, self.n2)).float()
        qkv = normed_out @ f(self.w_qkv).T
        if self.bias_qkv is not None:
            qkv = qkv + f(self.bias_qkv)
        T, D, nq, nkv = self.T, self.D, self.nq, self.nkv
        qkv = qkv.reshape(T, nq + 2 * nkv, D)
        q, k, v = qkv[:, :nq], qkv[:, nq:nq + nkv], qkv[:, nq + nkv:]

        def hn(t, w):
            if w is None:
                return t
            return bf(t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + EPS) * f(w)).float()

        q, k = hn(q, self.qn), hn(k, self.kn)
        cs = cos_sin.cpu()[self.pos.long()]
        c, s = cs[:, None, :D // 2], cs[:, None, D // 2:]

        def rot(t):
            a, b = t[..., :D // 2], t[..., D // 2:]
            return torch.cat([a * c - b * s, b * c + a * s], dim=-1)

        return dict(resid_mid=resid_mid, normed_mid=normed_mid, act=act, resid_out=resid_out, normed_out=normed_out,
                    q=rot(q), k=rot(k), v=v)


def run_case(case, splits=(2, 2, 2, 2), fused_gate=False, tp_buffers=None, mask=None, cos_sin=None, sh=None):
    from nkipy_b200 import ops
    from nkipy_b200.ops import decode_layer as DL

    T, H, I, D = case.T, case.H, case.inter, case.D
    dev = case.dev
    sh = case.shard() if sh is None else sh
    if cos_sin is None:
        cos_sin = ops.rope_table(D, case.max_pos, theta=10000.0, device=dev)
    e = lambda *s: torch.zeros(*s, dtype=torch.bfloat16, device=dev)  # noqa: E731
    out = dict(resid_mid=e(T, H), normed_mid=e(T, H), act=e(T, I), resid_out=e(T, H), normed_out=e(T, H),
               q=e(T, case.nq * D), kc=e(case.nblocks, case.nkv, case.bs, D), vc=e(case.nblocks, case.nkv, case.bs, D))
    qkv_w = sh["w_qkv"].shape[0]
    scratch = DL.layer_scratch(dev, DL.scratch_floats(DL.block_n_for(T), [
        (H, splits[0]), (2 * I, splits[1]), (H, splits[2]), (qkv_w, splits[3])]))
    if mask is None:
        mask = DL.ST_ALL if not fused_gate else DL.ST_ALL & ~DL.ST_SILU
    DL.decode_layer(mask, T, H, EPS, scratch, w_o=sh["w_o"], attn=sh["attn"], splits_o=splits[0], bias_o=sh["bias_o"],
                    resid_in=sh["resid"], norm1_w=sh["n1"], resid_mid=out["resid_mid"], normed_mid=out["normed_mid"],
                    w_gu=sh["w_gu"], inter=I, splits_gu=splits[1], fused_gate=fused_gate, bias_gu=sh["bias_gu"],
                    act_limit=case.limit, act=out["act"], w_down=sh["w_down"], splits_down=splits[2],
                    bias_down=sh["bias_down"], norm2_w=sh["n2"], resid_out=out["resid_out"],
                    normed_out=out["normed_out"], w_qkv=sh["w_qkv"], splits_qkv=splits[3], nq=case.nq, nkv=case.nkv,
                    head_dim=D, bias_qkv=sh["bias_qkv"], positions=sh["pos"], slots=sh["slots"], cos_sin=cos_sin,
                    q_norm_w=sh["qn"], k_norm_w=sh["kn"], q_out=out["q"], k_cache=out["kc"], v_cache=out["vc"],
                    tp_buffers=tp_buffers)
    torch.cuda.synchronize()
    return out, cos_sin


def compare(case, out, cos_sin, check_act=True):
    ref = case.oracle(cos_sin)
    T, D = case.T, case.D
    c = lambda k: out[k].cpu()  # noqa: E731
    check(c("resid_mid"), ref["resid_mid"])
    check(c("normed_mid"), ref["normed_mid"])
    if check_act:
        check(c("act"), ref["act"], tol=2e-2)
    check(c("resid_out"), ref["resid_out"])
    check(c("normed_out"), ref["normed_out"])
    check(c("q").reshape(T, case.nq, D), ref["q"], tol=2e-2)
    keep = case.slots >= 0
    blk, off = (case.slots[keep] // case.bs).long(), (case.slots[keep] % case.bs).long()
    kc, vc = c("kc"), c("vc")
    check(kc[blk, :, off], ref["k"][keep], tol=2e-2)
    check(vc[blk, :, off], ref["v"][keep], tol=2e-2)
    untouched = torch.ones(case.nblocks, case.bs, dtype=torch.bool)
    untouched[blk, off] = False
    assert kc.permute(0, 2, 1, 3)[untouched].abs().sum().item() == 0
    assert vc.permute(0, 2, 1, 3)[untouched].abs().sum().item() == 0


@pytest.mark.parametrize("T", [1, 17, 64, 100])
@pytest.mark.parametrize("fused_gate", [False, True])
def test_layer_chain_matches_fp32(T, fused_gate):
    from nkipy_b200 import ops

    case = Case(T, H=512, k_o=384, inter=384, nq=4, nkv=2, D=64, seed=T)
    out, cs = run_case(case, splits=(2, 1 if fused_gate else 3, 2, 2), fused_gate=fused_gate)
    compare(case, out, cs)
    assert ops.device_status() == 0


def test_layer_chain_biases_qk_norm_head_dim_128_clamped():
    from nkipy_b200 import ops

    case = Case(48, H=1024, k_o=512, inter=640, nq=4, nkv=1, D=128, seed=7, biases=True, qk_norm=True, limit=7.0)
    out, cs = run_case(case, splits=(4, 4, 5, 3))
    compare(case, out, cs)
    assert ops.device_status() == 0


def test_layer_chain_llama_shard_shapes_and_many_splits():
    """Llama-3-8B's per-rank shapes at 8 ranks (hidden 4096, 512-wide attention slice, 1792-wide FFN slice)."""
    from nkipy_b200 import ops

    case = Case(64, H=4096, k_o=512, inter=1792, nq=4, nkv=1, D=128, seed=3)
    out, cs = run_case(case, splits=(2, 5, 4, 8))
    compare(case, out, cs)
    assert ops.device_status() == 0


def test_back_to_back_launches_and_graph_replay():
    """The barrier words and the scratch are shared by consecutive launches; a captured graph replays them."""
    from nkipy_b200 import ops

    cases = [Case(32, H=512, k_o=256, inter=256, nq=4, nkv=2, D=64, seed=20 + i) for i in range(3)]
    outs = [run_case(c, splits=(2, 2, 2, 2)) for c in cases]
    for c, (o, cs) in zip(cases, outs):
        compare(c, o, cs)
    case, cs, sh = cases[0], outs[0][1], cases[0].shard()       # no host-to-device copies inside the capture
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        run_case(case, cos_sin=cs, sh=sh)
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    box = {}
    with torch.cuda.graph(graph):
        for _ in range(4):
            box["out"] = _launch_only(case, cs, sh)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    compare(case, box["out"][0], box["out"][1])
    assert ops.device_status() == 0


def _launch_only(case, cos_sin, sh):
    """run_case without the synchronize (stream capture forbids it)."""
    import unittest.mock as mock

    with mock.patch.object(torch.cuda, "synchronize", lambda *a, **k: None):
        return run_case(case, cos_sin=cos_sin, sh=sh)


def test_sub_chains_first_and_last_layer_masks():
    """QKV + RoPE alone (first layer of a step) and the chain without them (last layer)."""
    from nkipy_b200 import ops
    from nkipy_b200.ops import decode_layer as DL

    case = Case(40, H=512, k_o=256, inter=384, nq=4, nkv=2, D=64, seed=11)
    full, cs = run_case(case)
    compare(case, full, cs)
    head, _ = run_case(case, mask=DL.ST_ALL & ~(DL.ST_QKV | DL.ST_ROPE))
    assert torch.equal(head["normed_out"], full["normed_out"]) and head["q"].abs().sum().item() == 0
    # the tail alone, fed with the normed hidden state of the full run
    T, H, D = case.T, case.H, case.D
    sh = case.shard()
    q = torch.zeros(T, case.nq * D, dtype=torch.bfloat16, device=DEV)
    kc = torch.zeros(case.nblocks, case.nkv, case.bs, D, dtype=torch.bfloat16, device=DEV)
    vc = torch.zeros_like(kc)
    scratch = DL.layer_scratch(DEV, DL.scratch_floats(DL.block_n_for(T), [(sh["w_qkv"].shape[0], 2)]))
    DL.decode_layer(DL.ST_QKV | DL.ST_ROPE, T, H, EPS, scratch, normed_out=full["normed_out"], w_qkv=sh["w_qkv"],
                    splits_qkv=2, nq=case.nq, nkv=case.nkv, head_dim=D, positions=sh["pos"], slots=sh["slots"],
                    cos_sin=cs, q_out=q, k_cache=kc, v_cache=vc)
    torch.cuda.synchronize()
    assert torch.equal(q, full["q"]) and torch.equal(kc, full["kc"]) and torch.equal(vc, full["vc"])
    assert ops.device_status() == 0


def test_bad_arguments_are_rejected_before_launch():
    from nkipy_b200.ops import _lib
    from nkipy_b200.ops import decode_layer as DL

    case = Case(8, H=512, k_o=256, inter=256, nq=4, nkv=2, D=64)
    with pytest.raises(ValueError):
        DL.block_n_for(129)
    small = DL.DecodeLayerScratch(DEV, 16)                     # far too small for any stage
    sh = case.shard()
    with pytest.raises(_lib.KernelLibraryError):
        DL.decode_layer(DL.ST_O | DL.ST_RED1, 8, 512, EPS, small, w_o=sh["w_o"], attn=sh["attn"], splits_o=2,
                        resid_in=sh["resid"], norm1_w=sh["n1"],
                        resid_mid=torch.empty(8, 512, dtype=torch.bfloat16, device=DEV),
                        normed_mid=torch.empty(8, 512, dtype=torch.bfloat16, device=DEV))


def test_one_rank_through_the_push_path():
    """FusedTP on a single rank: the row-parallel stages store their partials into the (local) symmetric buffer
    and the reducing stages wait for the arrival counters -- the code path of tensor parallelism."""
    from nkipy_b200 import ops
    from nkipy_b200.parallel.comm import TPGroup
    from nkipy_b200.parallel.symm import FusedTP

    tp = TPGroup.single(torch.device("cuda:0"))
    case = Case(64, H=1024, k_o=512, inter=768, nq=4, nkv=2, D=64, seed=5)
    fused = FusedTP(tp, 64, 1024)
    try:
        for _ in range(3):                                      # counters and buffer parity carry over
            fused.begin_step()
            out, cs = run_case(case, splits=(2, 3, 4, 2), tp_buffers=fused.layer_buffers(64, 1024))
            compare(case, out, cs)
        assert ops.device_status() == 0
    finally:
        fused.close()


# ----------------------------------------------------------------------------- several ranks
def _rank_worker(rank, world, port, q, mode):
    sys.path.insert(0, ROOT)
    from test_fused_tp_gpu import MODES

    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0", **MODES[mode])
    import torch.distributed as dist

    from nkipy_b200 import ops
    from nkipy_b200.parallel.comm import TPGroup
    from nkipy_b200.parallel.symm import FusedTP

    tp = TPGroup.from_env()
    T, H = 64, 1024
    fused = FusedTP(tp, T, H)
    errs = []
    try:
        for it in range(3):
            case = Case(T, H=H, k_o=256, inter=384, nq=4, nkv=2, D=64, seed=40 + it, biases=(it == 1),
                        dev=tp.device, ranks=world, rank=rank)
            fused.begin_step()
            out, cs = run_case(case, splits=(2, 2, 3, 2), tp_buffers=fused.layer_buffers(T, H))
            try:
                compare(case, out, cs, check_act=False)         # act is this rank's slice only
                errs.append(0)
            except AssertionError as e:
                errs.append(str(e)[:200])
        status = ops.device_status()
        tp.barrier()
    finally:
        fused.close()
    q.put((rank, errs, status, bool(fused.mem.mc_ptr)))
    dist.destroy_process_group()


def _worlds():
    n = torch.cuda.device_count()
    return [w for w in (2, 4, 8) if w <= n] or [2]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("mode", ["vmm", "nvls"])
@pytest.mark.parametrize("world", _worlds())
def test_layer_chain_ranks(world, mode):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_worker, args=(r, world, port, q, mode)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=240) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, errs, status, _ in res:
        assert status == 0, (rank, status)
        assert errs == [0, 0, 0], (rank, errs)
