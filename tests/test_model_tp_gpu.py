"""Tiny dense and MoE models on 2 GPUs (tensor-parallel attention, expert-parallel MoE) with the fused
peer-memory runtime (GEMM push all-reduce, MoE combine push, argmax exchange) inside a CUDA graph; the
tokens every rank generates must agree and be (near-)best under the fp32 eager oracle."""
import os
import socket
import sys

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _cfg(kind):
    from nkipy_b200.models import config as C

    if kind.startswith("dense"):
        return C.tiny(num_heads=4, num_kv_heads=2)
    return C.tiny(num_heads=4, num_kv_heads=2, num_experts=8, top_k=2, moe_intermediate_size=128)


def _worker(rank, world, port, q, kind):
    sys.path.insert(0, ROOT)
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                      NKIPY_B200_DECODE_LAYER="persistent" if "persistent" in kind else "chain")
    from nkipy_b200 import ops
    from nkipy_b200.models.engine import GenerationEngine
    from nkipy_b200.models.transformer import TransformerLM
    from nkipy_b200.models.weights import random_weights
    from nkipy_b200.parallel.comm import TPGroup

    tp = TPGroup.from_env()
    cfg = _cfg(kind)
    w = random_weights(cfg, rank, world, seed=11, std=0.05)
    model = TransformerLM(cfg, w, tp, device=tp.device)
    eng = GenerationEngine(model, max_batch=4, max_seq_len=128, use_cuda_graph=True)
    assert getattr(tp, "fused", None) is not None
    g = torch.Generator().manual_seed(3)
    # "_sp" kinds prefill 4 x 64 = 256 tokens: enough rows for the sequence-parallel prefill path
    prompts = torch.randint(0, cfg.vocab_size, (4, 64 if kind.endswith("_sp") else 37), generator=g).tolist()
    out = eng.generate(prompts, 8)
    if kind.endswith("_sp"):
        assert getattr(model, "_sp_ops", None), "sequence-parallel prefill was not used"
    gathered = tp.all_gather_object(out)
    status = ops.device_status()
    q.put((rank, out, all(o == gathered[0] for o in gathered), status))
    tp.barrier()
    tp.fused.close()
    torch.distributed.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("kind", ["dense", "moe", "dense_sp", "moe_sp", "dense_persistent", "moe_persistent"])
def test_tp2_fused_generation(kind):
    from nkipy_b200.models.reference import EagerTransformer
    from nkipy_b200.models.weights import random_weights

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q, kind)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in range(2)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, out, agree, status in res:
        assert status == 0, (rank, status)
        assert agree, rank
    out = res[0][1]
    cfg = _cfg(kind)
    w = random_weights(cfg, 0, 1, seed=11, std=0.05)
    ref = EagerTransformer(cfg, w, dtype=torch.float32)
    g = torch.Generator().manual_seed(3)
    prompts = torch.randint(0, cfg.vocab_size, (4, 64 if kind.endswith("_sp") else 37), generator=g).tolist()
    for b in range(4):
        seq = list(prompts[b])
        for tok in out[b]:
            ref.reset()
            h = ref.forward(torch.tensor([seq]))[:, -1]
            logits = (h @ ref.w["lm_head_weight"]).float()[0]
            assert logits[tok] >= logits.max() - 0.05 * logits.std(), (b, tok)
            seq.append(tok)
