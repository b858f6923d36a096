"""Engine / paged-cache logic on CPU (PyTorch reference ops) against the eager oracle."""
import torch

from nkipy_b200.models import config as C
from nkipy_b200.models.engine import GenerationEngine, percentile
from nkipy_b200.models.kv_cache import BlockAllocator, OutOfBlocks
from nkipy_b200.models.reference import EagerTransformer
from nkipy_b200.models.transformer import TransformerLM, pick_splits
from nkipy_b200.models.weights import random_weights


def _tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def test_tiny_dense_matches_eager_oracle():
    cfg = C.tiny()
    w = random_weights(cfg, seed=1, std=0.05)
    model = TransformerLM(cfg, w, device="cpu")
    eng = GenerationEngine(model, max_batch=4, max_seq_len=128, use_cuda_graph=False)
    prompts = [_tokens(40, cfg.vocab_size, 1), _tokens(40, cfg.vocab_size, 2)]
    outs = eng.generate(prompts, max_new_tokens=6)
    ref = EagerTransformer(cfg, w, dtype=torch.float32)
    expect = ref.generate(torch.tensor(prompts), 6)
    agree = sum(int(a == b) for o, e in zip(outs, expect.tolist()) for a, b in zip(o, e))
    assert agree >= 10, (outs, expect.tolist())   # bf16 vs fp32: near ties may flip late tokens
    assert outs[0][0] == expect[0, 0].item() and outs[1][0] == expect[1, 0].item()


def test_prefix_sharing_reuses_blocks_and_keeps_results():
    cfg = C.tiny()
    w = random_weights(cfg, seed=2, std=0.05)
    model = TransformerLM(cfg, w, device="cpu")
    eng = GenerationEngine(model, max_batch=4, max_seq_len=256, use_cuda_graph=False)
    shared = _tokens(64, cfg.vocab_size, 3)
    a, b = shared + _tokens(10, cfg.vocab_size, 4), shared + _tokens(7, cfg.vocab_size, 5)
    out_a = eng.generate([a], 4)
    assert eng.stats.cached_tokens == 0
    out_b = eng.generate([b], 4)
    assert eng.stats.cached_tokens == 64          # two full blocks reused
    eng2 = GenerationEngine(model, max_batch=4, max_seq_len=256, use_cuda_graph=False, enable_prefix_sharing=False)
    assert eng2.generate([b], 4) == out_b
    both = eng.generate([a, b], 4)
    assert both[0] == out_a[0] and both[1] == out_b[0]


def test_block_allocator_refcounts_and_eviction():
    al = BlockAllocator(6, 32)
    toks = list(range(70))
    blocks, cached = al.admit(toks)
    assert len(blocks) == 3 and cached == 0
    al.publish(toks, blocks, 70)
    blocks2, cached2 = al.admit(toks[:64] + [999] * 10)
    assert cached2 == 64 and blocks2[:2] == blocks[:2] and al.ref[blocks[0]] == 2
    al.release(blocks)
    assert al.ref[blocks[0]] == 1
    al.release(blocks2)
    assert al.num_free() == 6
    # content survives release until recycled
    b3, c3 = al.admit(toks)
    assert c3 == 64
    al.release(b3)
    big, _ = al.admit(list(range(1000, 1000 + 6 * 32)))
    assert len(big) == 6
    try:
        al.admit([1] * 10)
        assert False
    except OutOfBlocks:
        pass
    al.release(big)
    _, c4 = al.admit(toks)
    assert c4 == 0                                # evicted


def test_helpers():
    assert pick_splits(4096, 4096) == 8 and pick_splits(128256, 4096) == 1 and pick_splits(6144, 4096) == 6
    assert percentile([1, 2, 3, 4], 50) == 2.5


def test_gqa_replicated_kv_and_qknorm_cpu():
    cfg = C.tiny(qk_norm=True, num_kv_heads=1, num_heads=4)
    w = random_weights(cfg, seed=5, std=0.05)
    model = TransformerLM(cfg, w, device="cpu")
    eng = GenerationEngine(model, max_batch=2, max_seq_len=96, use_cuda_graph=False)
    p = [_tokens(33, cfg.vocab_size, 7)]
    out = eng.generate(p, 3)
    ref = EagerTransformer(cfg, w, dtype=torch.float32).generate(torch.tensor(p), 3)
    assert out[0][0] == ref[0, 0].item()


def test_moe_models_match_oracle_cpu():
    """Qwen3-style (softmax -> top-k -> renorm, QK-norm) and gpt-oss-style (top-k -> softmax, biases,
    sinks, sliding window, clamped SwiGLU, YaRN) tiny MoE models against the eager oracle."""
    qwen = C.tiny(name="tiny-qwen3-moe", qk_norm=True, num_experts=8, top_k=2, moe_intermediate_size=128,
                  intermediate_size=0, rms_eps=1e-6, rope_theta=1e6)
    oss = C.tiny(name="tiny-gpt-oss", num_experts=4, top_k=2, moe_intermediate_size=128, intermediate_size=0,
                 attn_bias=True, router_mode="topk_softmax", router_bias=True, expert_bias=True, sliding_window=16,
                 layer_types=["sliding_attention", "full_attention"], attention_sinks=True, swiglu_limit=7.0,
                 rope_scaling_factor=4.0, rope_original_max_position=64, rope_theta=150000.0)
    for cfg in (qwen, oss):
        w = random_weights(cfg, seed=4, std=0.05)
        model = TransformerLM(cfg, w, device="cpu")
        eng = GenerationEngine(model, max_batch=2, max_seq_len=128, use_cuda_graph=False)
        prompts = [_tokens(45, cfg.vocab_size, 8), _tokens(45, cfg.vocab_size, 9)]
        seqs = eng.add_requests(prompts)
        first = eng.prefill(seqs)
        ref = EagerTransformer(cfg, w, dtype=torch.float32)
        h = ref.forward(torch.tensor(prompts))
        logits = (h[:, -1] @ ref.w["lm_head_weight"]).float()
        for b in range(2):
            assert logits[b, int(first[b])] >= logits[b].max() - 0.05 * logits[b].std(), cfg.name
        eng.release(seqs)
        out = eng.generate(prompts, 4)
        assert all(len(o) == 4 for o in out)
