"""Whole model graphs through the native pass pipeline: every graph the traced Qwen3-MoE and gpt-oss examples build
(prefill and decode layers, both attention types, the sampler) is lowered by all 21 passes, by the regular build and by
the one under AddressSanitizer + UBSan, and the lowered graph must give the results of the traced graph on random
inputs.  The rewriting passes thus meet attention with windows and sinks, rotary tables, routed experts (softmax, top-k,
gathers of expert weights), cache write-through with aliased results."""
import os
import shutil
import subprocess
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
for sub in ("llama", "qwen3", "gpt_oss"):
    sys.path.insert(0, os.path.join(ROOT, "examples", "models", sub))

from nkipy_b200.compiler import native  # noqa: E402
from nkipy_b200.core.interp import evaluate  # noqa: E402
from nkipy_b200.core.ir import Graph  # noqa: E402
from nkipy_b200.models import config as C  # noqa: E402
from nkipy_b200.models.weights import random_weights  # noqa: E402
from nkipy_b200.nkigen import transforms as T  # noqa: E402


def _qwen3_graphs():
    from qwen3_traced import TracedQwen3

    cfg = C.tiny(hidden_size=128, head_dim=64, num_heads=2, num_kv_heads=1, vocab_size=384, num_layers=1, qk_norm=True,
                 num_experts=6, top_k=2, moe_intermediate_size=64, intermediate_size=0, rms_eps=1e-6)
    w = random_weights(cfg, seed=7, std=0.08, dtype=torch.float32)
    prompts = torch.randint(0, cfg.vocab_size, (2, 7), generator=torch.Generator().manual_seed(2)).numpy()
    model = TracedQwen3(cfg, w, 2, 7, 16, backend="traced")
    model.generate(prompts, 2)
    return {f"qwen3/{k}": g for k, g in model.graphs.items()}


def _gpt_oss_graphs():
    from gpt_oss_traced import TracedGptOss, tiny_config

    cfg = tiny_config(layers=2, window=4)
    w = random_weights(cfg, seed=11, std=0.08, dtype=torch.float32)
    prompts = torch.randint(0, cfg.vocab_size, (2, 9), generator=torch.Generator().manual_seed(3)).numpy()
    model = TracedGptOss(cfg, w, 2, 9, 16, backend="traced")
    model.generate(prompts, 2)
    return {f"gpt_oss/{k}": g for k, g in model.graphs.items()}


@pytest.fixture(scope="module")
def graphs():
    out = {}
    out.update(_qwen3_graphs())
    out.update(_gpt_oss_graphs())
    assert len(out) >= 6
    return out


def _random_inputs(g, seed):
    rng = np.random.default_rng(seed)
    args = []
    for p in g.params:
        dt = np.dtype(p.dtype)
        if dt.kind == "f":
            args.append((rng.standard_normal(p.shape) * 0.3).astype(dt))
        elif dt.kind in "iu":
            args.append(rng.integers(0, 4, p.shape).astype(dt))          # positions / token ids: small and valid
        else:
            args.append(rng.random(p.shape) > 0.5)
    return args


def _same_results(g, lowered_text, seed):
    args = _random_inputs(g, seed)
    want = evaluate(g, [a.copy() for a in args])
    got = evaluate(Graph.from_text(lowered_text), [a.copy() for a in args])
    assert len(got) == len(want)
    for o, e in zip(got, want):
        np.testing.assert_allclose(np.asarray(o, np.float64), np.asarray(e, np.float64), rtol=1e-5, atol=1e-6)


def test_lowered_model_graphs_keep_their_results(graphs):
    for i, (name, g) in enumerate(sorted(graphs.items(), key=lambda kv: str(kv[0]))):
        lowered = T.apply_complete_knob_pipeline(g.to_text())
        _same_results(g, lowered, seed=i)
        after = Graph.from_text(lowered)
        assert len(after.nodes) <= len(g.nodes), name                     # the pipeline never grows a graph
        assert [(a.output_index, a.param_index) for a in after.aliases] == [(a.output_index, a.param_index) for a in g.aliases]


@pytest.mark.skipif(shutil.which("g++") is None, reason="no host compiler")
def test_model_graphs_are_clean_under_the_sanitizers(graphs, tmp_path):
    try:
        san = native.build_sanitized()
    except RuntimeError as e:
        if "sanitize" in str(e) or "asan" in str(e):
            pytest.skip("sanitizer runtime not installed")
        raise
    for name, g in graphs.items():
        text = g.to_text()
        res = subprocess.run([str(san), "--pipeline", "-"], input=text, capture_output=True, text=True, timeout=300)
        assert res.returncode == 0 and "Sanitizer" not in res.stderr and "runtime error" not in res.stderr, \
            (name, res.stderr[-3000:])
        assert res.stdout == T.apply_complete_knob_pipeline(text), name
