"""Verification step of speculative decoding as kernel functions.

The target runs the K + 1 candidate tokens (the last committed token followed by K drafts) through its layers; the
kernel below turns the final hidden states into the target's greedy token at every candidate position, vocabulary
parallel when several ranks hold slices of the LM head.  Position i predicts the token after candidate i, so draft
i + 1 is accepted iff it equals the target token at position i; the target token at the first mismatch is emitted
as well (examples/models/gpt_oss/peagle/kernels/verify.py:21-59 and speculate.py in the reference, where the
comparison also runs on the host)."""
import numpy as np

from nkipy_b200.core import tensor_apis
from nkipy_b200.distributed import collectives as cc

from llama_kernels.rmsnorm import rmsnorm


def verify_tokens(h, final_norm, lm_head, norm_eps: float, world_size: int = 1):
    """h [B, S, H]; lm_head [H, V_local] (this rank's vocabulary slice).  Returns int32 [B, S]: the target's greedy
    token at each position, as a global vocabulary id."""
    B, S, _ = h.shape
    v_local = lm_head.shape[1]
    logits = np.matmul(rmsnorm(h, final_norm, norm_eps), lm_head).astype(np.float32)
    val, idx = tensor_apis.topk(logits, 1)                                   # [B, S, 1]
    val, idx = val[:, :, 0], idx[:, :, 0].astype(np.int32)
    if world_size == 1:
        return idx
    # every rank's local winner, then the winning rank per position
    groups = [list(range(world_size))]
    vals = cc.all_gather(val, all_gather_dim=0, replica_groups=groups).reshape(world_size, B, S)
    idxs = cc.all_gather(idx, all_gather_dim=0, replica_groups=groups).reshape(world_size, B, S)
    best = np.argmax(vals, axis=0).astype(np.int32)                          # [B, S]
    chosen = np.take_along_axis(idxs, best[None], axis=0)[0]
    return (best * np.int32(v_local) + chosen).astype(np.int32)


def accept(drafts, target_tokens):
    """Host side of greedy verification.  drafts [B, K] (proposed tokens), target_tokens [B, K + 1] (from
    `verify_tokens`).  Returns (accepted [B], emitted): emitted[b] is the accepted drafts followed by the target's
    token at the first mismatch (or its bonus token when every draft was accepted)."""
    drafts, target_tokens = np.asarray(drafts), np.asarray(target_tokens)
    B, K = drafts.shape
    accepted = np.zeros(B, np.int32)
    emitted = []
    for b in range(B):
        n = 0
        while n < K and drafts[b, n] == target_tokens[b, n]:
            n += 1
        accepted[b] = n
        emitted.append([int(t) for t in drafts[b, :n]] + [int(target_tokens[b, n])])
    return accepted, emitted
