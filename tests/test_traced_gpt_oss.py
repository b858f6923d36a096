"""gpt-oss as NumPy kernel functions (examples/models/gpt_oss/gpt_oss_kernels): direct mode and traced +
interpreted, both against the eager fp32 model with the same weights (biases, a sliding window on alternating
layers, sink logits, YaRN-scaled RoPE, top-k-then-softmax routing, clamped activation)."""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "examples", "models", "llama"))
sys.path.insert(0, os.path.join(ROOT, "examples", "models", "gpt_oss"))

from gpt_oss_kernels import moe_ffn  # noqa: E402
from gpt_oss_traced import TracedGptOss, tiny_config  # noqa: E402

from nkipy_b200.core.compile import trace  # noqa: E402
from nkipy_b200.core.interp import evaluate  # noqa: E402
from nkipy_b200.models.reference import EagerTransformer  # noqa: E402
from nkipy_b200.models.weights import random_weights  # noqa: E402


def _setup(layers=2, B=2, T=9, new=6):
    cfg = tiny_config(layers=layers, window=4)             # the window is shorter than the prompt: it matters
    w = random_weights(cfg, seed=11, std=0.08, dtype=torch.float32)
    g = torch.Generator().manual_seed(3)
    prompts = torch.randint(0, cfg.vocab_size, (B, T), generator=g)
    expect = EagerTransformer(cfg, w, dtype=torch.float32).generate(prompts, new).tolist()
    return cfg, w, prompts.numpy(), expect


def test_direct_mode_generates_the_oracle_tokens():
    cfg, w, prompts, expect = _setup()
    model = TracedGptOss(cfg, w, prompts.shape[0], prompts.shape[1], 16, backend="numpy")
    assert model.windows == [4, 0]
    assert model.generate(prompts, 6) == expect


def test_traced_graphs_generate_the_oracle_tokens():
    cfg, w, prompts, expect = _setup()
    model = TracedGptOss(cfg, w, prompts.shape[0], prompts.shape[1], 16, backend="traced")
    assert model.generate(prompts, 6) == expect
    # one graph per kernel function and layer type: sliding and full attention, prefill and decode
    assert set(model.graphs) == {("prefill", 4), ("prefill", 0), ("decode", 4), ("decode", 0)}


def test_the_window_and_the_sinks_change_the_result():
    """The oracle comparison has teeth: without the window, or with the sinks zeroed out of the softmax (a very
    negative logit), other tokens come out."""
    cfg, w, prompts, expect = _setup()
    model = TracedGptOss(cfg, w, prompts.shape[0], prompts.shape[1], 16, backend="numpy")
    model.windows = [0, 0]
    no_window = model.generate(prompts, 6)
    model = TracedGptOss(cfg, w, prompts.shape[0], prompts.shape[1], 16, backend="numpy")
    for lw in model.layers:
        lw["sinks"] = np.full_like(lw["sinks"], -1e4)
    no_sinks = model.generate(prompts, 6)
    assert no_window != expect or no_sinks != expect


def test_routed_feed_forward_matches_a_per_token_restatement():
    rng = np.random.default_rng(1)
    B, T, H, E, I, K = 2, 4, 32, 6, 16, 3
    x = rng.standard_normal((B, T, H)).astype(np.float32)
    rw, rb = rng.standard_normal((H, E)).astype(np.float32), rng.standard_normal(E).astype(np.float32)
    gu, bgu = (rng.standard_normal((E, H, 2 * I)) * 0.3).astype(np.float32), rng.standard_normal((E, 2 * I)).astype(np.float32)
    dn, bdn = (rng.standard_normal((E, I, H)) * 0.3).astype(np.float32), rng.standard_normal((E, H)).astype(np.float32)
    limit, alpha = 1.5, 1.702                              # a limit the data reaches
    got = moe_ffn(x, rw, rb, gu, bgu, dn, bdn, K, limit, alpha)
    xt = x.reshape(-1, H).astype(np.float64)
    logits = xt @ rw + rb
    want = np.zeros_like(xt)
    for n in range(xt.shape[0]):
        top = np.argsort(-logits[n])[:K]
        wt = np.exp(logits[n, top] - logits[n, top].max())
        wt /= wt.sum()
        for e, we in zip(top, wt):
            h = xt[n] @ gu[e] + bgu[e]
            g_, u_ = np.minimum(h[:I], limit), np.clip(h[I:], -limit, limit)
            want[n] += we * (((u_ + 1) * g_ / (1 + np.exp(-alpha * g_))) @ dn[e] + bdn[e])
    np.testing.assert_allclose(got.reshape(-1, H), want, rtol=2e-4, atol=2e-5)
    graph = trace(moe_ffn).specialize(x, rw, rb, gu, bgu, dn, bdn, top_k=K, limit=limit, alpha=alpha)
    np.testing.assert_allclose(np.asarray(evaluate(graph, [x, rw, rb, gu, bgu, dn, bdn])[0]), got, rtol=1e-5, atol=1e-6)


def test_traced_layers_lower_to_cuda_that_compiles_for_sm_100a(tmp_path):
    import shutil
    import subprocess

    import pytest

    from gpt_oss_kernels import decode_layer, prefill_layer
    from gpt_oss_traced import _ORDER
    from llama import embed

    from nkipy_b200.compiler.codegen import generate

    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc not installed")
    cfg, w, prompts, _ = _setup(layers=1)
    model = TracedGptOss(cfg, w, prompts.shape[0], prompts.shape[1], 16, backend="numpy")
    lw = model.layers[0]
    x = embed(prompts, model.host["table"])
    cases = (("prefill", prefill_layer, [x]), ("decode", decode_layer, [x[:, :1], np.array([9], np.int32)]))
    for name, fn, lead in cases:
        g = trace(fn).specialize(*lead, *[lw[k].copy() for k in _ORDER], window=4, **model.scalars)
        prog = generate(g)
        src = tmp_path / f"{name}.cu"
        src.write_text(prog.source)
        r = subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O1", "-cubin", "-I",
                            os.path.join(ROOT, "csrc", "kernels"), "-o", str(tmp_path / f"{name}.cubin"), str(src)],
                           capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]


def test_verify_kernel_and_acceptance():
    """The speculative-decoding verification as a kernel function: greedy target tokens at K + 1 positions, direct
    and traced, and the host-side acceptance rule (longest matching prefix plus the target's own token)."""
    from gpt_oss_kernels import accept, verify_tokens

    rng = np.random.default_rng(5)
    B, S, H, V = 3, 4, 32, 97
    h = rng.standard_normal((B, S, H)).astype(np.float32)
    norm = (1.0 + 0.1 * rng.standard_normal(H)).astype(np.float32)
    head = rng.standard_normal((H, V)).astype(np.float32)
    got = verify_tokens(h, norm, head, 1e-5)
    hn = h / np.sqrt((h * h).mean(-1, keepdims=True) + 1e-5) * norm
    want = np.argmax(hn @ head, axis=-1)
    assert got.dtype == np.int32 and np.array_equal(got, want)
    g = trace(verify_tokens).specialize(h, norm, head, norm_eps=1e-5)
    assert np.array_equal(np.asarray(evaluate(g, [h, norm, head])[0]), want)
    # vocabulary-parallel form: in one process the gather replicates this rank's winners, rank 0 wins every tie,
    # so the global id is the local one -- the reshapes, the winner selection and the id arithmetic all run
    assert np.array_equal(verify_tokens(h, norm, head, 1e-5, world_size=2), want)
    g2 = trace(verify_tokens).specialize(h, norm, head, norm_eps=1e-5, world_size=2)
    assert any(n.opcode == "all_gather" for n in g2.nodes)
    target = np.array([[5, 6, 7, 8], [5, 6, 7, 8], [1, 2, 3, 4]])
    drafts = np.array([[5, 6, 7], [5, 9, 7], [0, 2, 3]])
    n, out = accept(drafts, target)
    assert n.tolist() == [3, 1, 0]
    assert out == [[5, 6, 7, 8], [5, 6], [1]]
