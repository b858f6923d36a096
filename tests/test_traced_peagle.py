"""The P-EAGLE drafter as NumPy kernel functions (examples/models/gpt_oss/peagle/peagle_kernels): a prefill-like
step at position 0 followed by a drafting step at a later position, direct and traced + interpreted, against a
per-head fp32 restatement in PyTorch written here."""
import math
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "examples", "models", "llama"))
sys.path.insert(0, os.path.join(ROOT, "examples", "models", "gpt_oss", "peagle"))

from peagle_kernels import draft_tokens, drafter_layer, fuse_inputs, fusion_layer  # noqa: E402

from nkipy_b200.core.compile import trace  # noqa: E402
from nkipy_b200.core.interp import evaluate  # noqa: E402

B, W, H, TH, NQ, NKV, D, I, S, V, VD = 2, 4, 64, 48, 2, 1, 32, 96, 24, 80, 50
EPS, THETA = 1e-5, 10000.0
SC = dict(n_heads=NQ, n_kv_heads=NKV, head_dim=D, rope_theta=THETA, norm_eps=EPS)


def _weights(seed=0):
    g = np.random.default_rng(seed)
    r = lambda *s: (g.standard_normal(s) * 0.2).astype(np.float32)
    w = dict(embed_tokens=r(V, H), fc=r(3 * TH, H), mask_hidden=r(3 * TH), embed_norm=1 + 0.1 * r(H), hidden_norm=1 + 0.1 * r(H),
             final_norm=1 + 0.1 * r(H), lm_head=r(H, VD), d2t=g.integers(0, V - VD, VD).astype(np.int32))
    for l, win in ((0, 2 * H), (1, H)):
        w[f"qkv{l}"], w[f"o{l}"] = r(win, (NQ + 2 * NKV) * D), r(NQ * D, H)
        w[f"gu{l}"], w[f"dn{l}"] = r(H, 2 * I), r(I, H)
        w[f"post{l}"] = 1 + 0.1 * r(H)
    w["in1"] = 1 + 0.1 * r(H)
    return w


def _step(w, caches, ids, hidden3, is_mask, start, run):
    """One drafter pass through the kernel functions; `run(fn, args, scalars)` calls them directly or traced."""
    pos = np.array([start], np.int32)
    hid, fused = run(fuse_inputs, [ids, hidden3, is_mask, w["embed_tokens"], w["fc"], w["mask_hidden"], w["embed_norm"],
                                   w["hidden_norm"]], dict(norm_eps=EPS))
    x = run(fusion_layer, [hid, fused, pos, w["qkv0"], w["o0"], w["gu0"], w["dn0"], w["post0"], caches[0], caches[1]], SC,
            caches=(0, 1))
    x = run(drafter_layer, [x, pos, w["qkv1"], w["o1"], w["gu1"], w["dn1"], w["in1"], w["post1"], caches[2], caches[3]], SC,
            caches=(2, 3))
    return run(draft_tokens, [x, w["final_norm"], w["lm_head"], w["d2t"]], dict(norm_eps=EPS))


def _direct(caches):
    def run(fn, args, scalars, caches=None):
        return fn(*args, **scalars)                      # cache arguments are updated in place
    return run


def _traced(store):
    graphs = {}

    def run(fn, args, scalars, caches=None):
        key = fn.__name__
        if key not in graphs:
            graphs[key] = trace(fn).specialize(*[a.copy() for a in args], **scalars)
        g = graphs[key]
        out = evaluate(g, list(args))
        names = [o.name for o in g.outputs]
        if caches:
            store[caches[0]][...] = np.asarray(out[names.index("cache_k")])
            store[caches[1]][...] = np.asarray(out[names.index("cache_v")])
        res = [np.asarray(out[i]) for i, n in enumerate(names) if n.startswith("output")]
        return res[0] if len(res) == 1 else tuple(res)
    return run


# ---- fp32 restatement ------------------------------------------------------------------------------
def _rms(x, w):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + EPS) * w


def _rope(t, pos):
    half = D // 2
    inv = 1.0 / (THETA ** (torch.arange(0, D, 2, dtype=torch.float64) / D))
    ang = pos.double()[:, None] * inv[None, :]
    c, s = ang.cos().float()[None, :, None, :], ang.sin().float()[None, :, None, :]
    a, b = t[..., :half], t[..., half:]
    return torch.cat([a * c - b * s, b * c + a * s], -1)


class Oracle:
    def __init__(self, w):
        self.w = {k: torch.from_numpy(np.asarray(v)) for k, v in w.items()}
        self.k = [torch.zeros(B, 0, NKV, D), torch.zeros(B, 0, NKV, D)]
        self.v = [torch.zeros(B, 0, NKV, D), torch.zeros(B, 0, NKV, D)]

    def _attn(self, l, h, start):
        w = self.w
        qkv = h @ w[f"qkv{l}"]
        q, k, v = qkv.split([NQ * D, NKV * D, NKV * D], -1)
        pos = torch.arange(start, start + W)
        q, k = _rope(q.reshape(B, W, NQ, D), pos), _rope(k.reshape(B, W, NKV, D), pos)
        self.k[l] = torch.cat([self.k[l][:, :start], k], 1)          # rows from `start` on are overwritten
        self.v[l] = torch.cat([self.v[l][:, :start], v.reshape(B, W, NKV, D)], 1)
        out = torch.zeros(B, W, NQ, D)
        for hq in range(NQ):
            kk, vv = self.k[l][:, :, hq // (NQ // NKV)], self.v[l][:, :, hq // (NQ // NKV)]
            s = torch.einsum("bqd,bkd->bqk", q[:, :, hq], kk) / math.sqrt(D)
            mask = torch.arange(kk.shape[1])[None, :] <= pos[:, None]
            s = s.masked_fill(~mask[None], float("-inf"))
            out[:, :, hq] = torch.softmax(s, -1) @ vv
        return out.reshape(B, W, NQ * D) @ w[f"o{l}"]

    def step(self, ids, hidden3, is_mask, start):
        w = self.w
        emb = w["embed_tokens"][torch.from_numpy(ids).long()]
        h3 = torch.where(torch.from_numpy(is_mask)[..., None] != 0, w["mask_hidden"][None, None], torch.from_numpy(hidden3))
        hid = h3 @ w["fc"]
        fused = torch.cat([_rms(emb, w["embed_norm"]), _rms(hid, w["hidden_norm"])], -1)
        x = hid + self._attn(0, fused, start)
        gu = _rms(x, w["post0"]) @ w["gu0"]
        x = x + (torch.nn.functional.silu(gu[..., :I]) * gu[..., I:]) @ w["dn0"]
        x = x + self._attn(1, _rms(x, w["in1"]), start)
        gu = _rms(x, w["post1"]) @ w["gu1"]
        x = x + (torch.nn.functional.silu(gu[..., :I]) * gu[..., I:]) @ w["dn1"]
        idx = (_rms(x, w["final_norm"]) @ w["lm_head"]).argmax(-1)
        return (idx + w["d2t"].long()[idx]).int().numpy()


def _inputs(seed):
    g = np.random.default_rng(seed)
    ids = g.integers(0, V, (B, W)).astype(np.int32)
    hidden3 = g.standard_normal((B, W, 3 * TH)).astype(np.float32)
    return ids, hidden3


def test_two_drafter_steps_match_the_restatement_direct_and_traced():
    w = _weights()
    ids0, h0 = _inputs(1)
    ids1, h1 = _inputs(2)
    none, tail = np.zeros((B, W), np.int32), np.array([[0, 0, 1, 1]] * B, np.int32)     # last two rows are placeholders
    oracle = Oracle(w)
    want0 = oracle.step(ids0, h0, none, 0)
    want1 = oracle.step(ids1, h1, tail, 3)           # overlaps row 3 of the first step: that row is overwritten
    for make in (_direct, _traced):
        caches = [np.zeros((B, S, NKV, D), np.float32) for _ in range(4)]
        run = make(caches)
        got0 = _step(w, caches, ids0, h0, none, 0, run)
        got1 = _step(w, caches, ids1, h1, tail, 3, run)
        assert got0.dtype == np.int32 and np.array_equal(got0, want0), make.__name__
        assert np.array_equal(got1, want1), make.__name__
