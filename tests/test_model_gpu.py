"""End-to-end model checks on a B200: native kernels vs the fp32 eager oracle."""
import math

import pytest
import torch

from nkipy_b200 import ops
from nkipy_b200.models import config as C
from nkipy_b200.models.engine import GenerationEngine
from nkipy_b200.models.reference import EagerTransformer
from nkipy_b200.models.transformer import TransformerLM
from nkipy_b200.models.weights import random_weights

pytestmark = pytest.mark.gpu


def _prompts(b, n, vocab, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (b, n), generator=g)


def test_llama_block_prefill_matches_fp32_reference():
    """Single Llama-style decoder block, hidden 4096, 32/8 heads, FFN 14336, causal prefill
    batch 8 x seq 2048, against the fp32 PyTorch reference (rel err < 2e-2)."""
    cfg = C.llama3_8b(num_layers=1, vocab_size=4096, max_position=4096)
    dev = torch.device("cuda")
    w = random_weights(cfg, device=dev, seed=0, std=0.02)
    model = TransformerLM(cfg, w, device=dev)
    B, S = 8, 2048
    prompts = _prompts(B, S, cfg.vocab_size)
    eng = GenerationEngine(model, max_batch=B, max_seq_len=S + 64, prefill_chunk_tokens=B * S)
    seqs = eng.add_requests(prompts.tolist())
    cache = eng.cache
    ids = prompts.reshape(-1).to(torch.int32).to(dev)
    pos = torch.arange(S, dtype=torch.int32).repeat(B).to(dev)
    slots = torch.cat([cache.slots_for(s, 0, S) for s in seqs]).to(dev)
    t = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    table = cache.block_table[torch.tensor([s.slot for s in seqs], device=dev)]
    hidden = model.prefill(ids, pos, slots, cache, table, t([i * S for i in range(B)]), t([S] * B), t([S] * B), S)
    torch.cuda.synchronize()
    ops.raise_on_device_error()
    ref = EagerTransformer(cfg, w, device=dev, dtype=torch.float32)
    expect = torch.cat([ref_forward(ref, prompts[b:b + 1].to(dev)) for b in range(B)])
    err = ((hidden.float() - expect).norm() / expect.norm()).item()
    assert err < 2e-2, err


def ref_forward(ref, ids):
    ref.reset()
    return ref.forward(ids, 0).reshape(-1, ref.cfg.hidden_size)


@pytest.fixture(params=["chain", "persistent"])
def layer_impl(request, monkeypatch):
    """Both ways of running a decode step: one launch per operation, and the persistent layer kernel."""
    monkeypatch.setattr(ops, "DECODE_LAYER_IMPL", request.param)
    return request.param


@pytest.mark.parametrize("graph", [False, True])
def test_tiny_generate_matches_oracle_tokens(graph, layer_impl):
    cfg = C.tiny(hidden_size=512, head_dim=128, num_heads=4, num_kv_heads=2, intermediate_size=1024,
                 vocab_size=2048, num_layers=3)
    dev = torch.device("cuda")
    w = random_weights(cfg, device=dev, seed=3, std=0.05)
    model = TransformerLM(cfg, w, device=dev)
    eng = GenerationEngine(model, max_batch=4, max_seq_len=256, use_cuda_graph=graph)
    prompts = _prompts(3, 70, cfg.vocab_size, 5)
    outs = eng.generate(prompts.tolist(), 12)
    ref = EagerTransformer(cfg, w, device=dev, dtype=torch.float32)
    expect = ref.generate(prompts.to(dev), 12).tolist()
    assert [o[0] for o in outs] == [e[0] for e in expect]
    # Greedy decoding follows whichever token wins a near-tie, so after one flipped tie two correct
    # implementations produce different continuations.  Judge every generated token on its own instead: given the
    # tokens generated so far it must be (nearly) the oracle's best choice.
    agree = sum(int(a == b) for o, e in zip(outs, expect) for a, b in zip(o, e))
    assert agree >= 18, (outs, expect)
    for b in range(len(outs)):
        seq = prompts[b].tolist()
        for tok in outs[b]:
            ref.reset()
            h = ref.forward(torch.tensor([seq], device=dev))[:, -1]
            logits = (h @ ref.w["lm_head_weight"].float()).float()[0]
            assert logits[tok] >= logits.max() - 0.05 * logits.std(), (b, tok, int(logits.argmax()))
            seq.append(tok)


def test_decode_hidden_matches_oracle(layer_impl):
    cfg = C.llama3_8b(num_layers=2, vocab_size=4096, max_position=2048)
    dev = torch.device("cuda")
    w = random_weights(cfg, device=dev, seed=1, std=0.02)
    model = TransformerLM(cfg, w, device=dev)
    B, S = 5, 300
    prompts = _prompts(B, S, cfg.vocab_size, 2)
    eng = GenerationEngine(model, max_batch=B, max_seq_len=512, use_cuda_graph=False)
    seqs = eng.add_requests(prompts.tolist())
    first = eng.prefill(seqs)
    eng.prepare_decode(4)
    ops.decode_advance(eng.context_lens, eng.cache.block_table, eng.positions, eng.slots)
    hidden = model.decode_step(eng.ids, eng.positions, eng.slots, eng.cache, eng.cache.block_table, eng.context_lens)
    torch.cuda.synchronize()
    ref = EagerTransformer(cfg, w, device=dev, dtype=torch.float32)
    ref.forward(prompts.to(dev), 0)
    expect = ref.forward(first.long()[:, None], S)[:, 0]
    err = ((hidden.float() - expect).norm() / expect.norm()).item()
    assert err < 2e-2, err


def test_moe_model_prefill_and_decode_match_oracle(layer_impl):
    cfg = C.tiny(name="tiny-qwen3-moe", hidden_size=512, head_dim=128, num_heads=4, num_kv_heads=2, qk_norm=True,
                 num_experts=16, top_k=4, moe_intermediate_size=256, intermediate_size=0, vocab_size=2048,
                 num_layers=2, rms_eps=1e-6)
    dev = torch.device("cuda")
    w = random_weights(cfg, device=dev, seed=2, std=0.05)
    model = TransformerLM(cfg, w, device=dev)
    eng = GenerationEngine(model, max_batch=4, max_seq_len=256)
    prompts = _prompts(4, 90, cfg.vocab_size, 3)
    outs = eng.generate(prompts.tolist(), 6)
    ref = EagerTransformer(cfg, w, device=dev, dtype=torch.float32)
    expect = ref.generate(prompts.to(dev), 6).tolist()
    assert [o[0] for o in outs] == [e[0] for e in expect]
    agree = sum(int(a == b) for o, e in zip(outs, expect) for a, b in zip(o, e))
    assert agree >= 18, (outs, expect)
