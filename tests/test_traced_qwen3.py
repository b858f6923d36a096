"""Qwen3-MoE as NumPy kernel functions (examples/models/qwen3/qwen3_kernels): called directly and traced +
interpreted, both against the eager fp32 model with the same weights; the routed feed-forward alone against a
per-token, per-expert restatement written here."""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "examples", "models", "llama"))
sys.path.insert(0, os.path.join(ROOT, "examples", "models", "qwen3"))

from qwen3_kernels import moe_ffn, prefill_layer  # noqa: E402
from qwen3_traced import TracedQwen3  # noqa: E402

from nkipy_b200.core.compile import trace  # noqa: E402
from nkipy_b200.core.interp import evaluate  # noqa: E402
from nkipy_b200.models import config as C  # noqa: E402
from nkipy_b200.models.reference import EagerTransformer  # noqa: E402
from nkipy_b200.models.weights import random_weights  # noqa: E402


def _setup(layers=2, B=2, T=7, new=5):
    cfg = C.tiny(hidden_size=128, head_dim=64, num_heads=2, num_kv_heads=1, vocab_size=384, num_layers=layers,
                 qk_norm=True, num_experts=6, top_k=2, moe_intermediate_size=64, intermediate_size=0, rms_eps=1e-6)
    w = random_weights(cfg, seed=7, std=0.08, dtype=torch.float32)
    for i in range(layers):                                   # QK-norm weights that are not all ones
        g = torch.Generator().manual_seed(100 + i)
        w[f"layers.{i}.q_norm_weight"] = 1.0 + 0.2 * torch.randn(64, generator=g)
        w[f"layers.{i}.k_norm_weight"] = 1.0 + 0.2 * torch.randn(64, generator=g)
    g = torch.Generator().manual_seed(2)
    prompts = torch.randint(0, cfg.vocab_size, (B, T), generator=g)
    expect = EagerTransformer(cfg, w, dtype=torch.float32).generate(prompts, new).tolist()
    return cfg, w, prompts.numpy(), expect


def test_routed_feed_forward_matches_a_per_token_restatement():
    rng = np.random.default_rng(0)
    B, T, H, E, I, K = 2, 5, 32, 7, 16, 3
    x = rng.standard_normal((B, T, H)).astype(np.float32)
    rw = rng.standard_normal((H, E)).astype(np.float32)
    gu = (rng.standard_normal((E, H, 2 * I)) * 0.2).astype(np.float32)
    dn = (rng.standard_normal((E, I, H)) * 0.2).astype(np.float32)
    got = moe_ffn(x, rw, gu, dn, K)
    xt = x.reshape(-1, H).astype(np.float64)
    logits = xt @ rw
    p = np.exp(logits - logits.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    want = np.zeros_like(xt)
    for n in range(xt.shape[0]):
        top = np.argsort(-p[n])[:K]
        wt = p[n, top] / p[n, top].sum()
        for e, we in zip(top, wt):
            h = xt[n] @ gu[e]
            g_, u_ = h[:I], h[I:]
            want[n] += we * ((g_ / (1 + np.exp(-g_)) * u_) @ dn[e])
    np.testing.assert_allclose(got.reshape(-1, H), want, rtol=1e-4, atol=1e-5)
    graph = trace(moe_ffn).specialize(x, rw, gu, dn, top_k=K)
    ops = {n.opcode for n in graph.nodes}
    assert {"softmax", "topk", "take", "dot"} <= ops
    assert len(graph.nodes) < 80                       # one batched graph, not B x T x top_k unrolled experts
    np.testing.assert_allclose(np.asarray(evaluate(graph, [x, rw, gu, dn])[0]), got, rtol=1e-5, atol=1e-6)


def test_direct_mode_generates_the_oracle_tokens():
    cfg, w, prompts, expect = _setup()
    model = TracedQwen3(cfg, w, prompts.shape[0], prompts.shape[1], 16, backend="numpy")
    assert model.generate(prompts, 5) == expect


def test_traced_graphs_generate_the_oracle_tokens():
    cfg, w, prompts, expect = _setup()
    model = TracedQwen3(cfg, w, prompts.shape[0], prompts.shape[1], 16, backend="traced")
    assert model.generate(prompts, 5) == expect
    assert set(model.graphs) >= {"prefill", "decode"}          # one graph per kernel function and shape, reused per step
    outs = [o.name for o in model.graphs["decode"].outputs]
    assert outs == ["output0", "cache_k", "cache_v"]           # the caches are written through


def test_traced_prefill_layer_equals_direct_mode():
    cfg, w, prompts, _ = _setup(layers=1)
    model = TracedQwen3(cfg, w, prompts.shape[0], prompts.shape[1], 16, backend="numpy")
    from llama import embed
    from qwen3_traced import _ORDER

    lw = model.layers[0]
    x = embed(prompts, model.host["table"])
    args = [lw[k].copy() for k in _ORDER]
    want = prefill_layer(x, *[a.copy() for a in args], **model.scalars)
    g = trace(prefill_layer).specialize(x, *[a.copy() for a in args], **model.scalars)
    got = evaluate(g, [x] + [a.copy() for a in args])
    np.testing.assert_allclose(np.asarray(got[0]), want, rtol=1e-4, atol=1e-4)


def test_traced_layers_lower_to_cuda_that_compiles_for_sm_100a(tmp_path):
    """The code generator covers everything the routed layer needs (softmax, top-k, gather of expert weights,
    batched products, cache write-through): both layer graphs become CUDA source that nvcc accepts.  Compiling needs
    no GPU."""
    import shutil
    import subprocess

    import pytest

    from llama import embed
    from qwen3_kernels import decode_layer
    from qwen3_traced import _ORDER

    from nkipy_b200.compiler.codegen import generate

    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc not installed")
    cfg, w, prompts, _ = _setup(layers=1)
    model = TracedQwen3(cfg, w, prompts.shape[0], prompts.shape[1], 16, backend="numpy")
    lw = model.layers[0]
    x = embed(prompts, model.host["table"])
    cases = (("prefill", prefill_layer, [x]), ("decode", decode_layer, [x[:, :1], np.array([7], np.int32)]))
    for name, fn, lead in cases:
        g = trace(fn).specialize(*lead, *[lw[k].copy() for k in _ORDER], **model.scalars)
        prog = generate(g)
        assert len(prog.launches) < 120
        src = tmp_path / f"{name}.cu"
        src.write_text(prog.source)
        r = subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O1", "-cubin", "-I",
                            os.path.join(ROOT, "csrc", "kernels"), "-o", str(tmp_path / f"{name}.cubin"), str(src)],
                           capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
