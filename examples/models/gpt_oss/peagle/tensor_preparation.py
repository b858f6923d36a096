"""Convert a P-EAGLE drafter checkpoint to this package's drafter schema (one replicated shard)
(reference: examples/models/gpt_oss/peagle/tensor_preparation.py:20-113).

The drafter checkpoint stores `embed_tokens`, `fc`, `mask_hidden`, `d2t`, a fusion `midlayer`, plain
`layers.N`, `norm` and `lm_head`; every matrix is transposed into ``x @ W`` orientation and q/k/v and
gate/up are fused the way the target's layers are.
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "..", ".."))

from nkipy_b200.models.checkpoint import LazyCheckpoint  # noqa: E402
from nkipy_b200.models.weights import save_shard  # noqa: E402


def convert(sd, dtype=torch.bfloat16):
    T = lambda n: sd[n].to(dtype).t().contiguous()
    out = {"embed_tokens": sd["embed_tokens.weight"].to(dtype), "fc_weight": T("fc.weight"),
           "mask_hidden": sd["mask_hidden"].to(dtype).reshape(-1), "d2t": sd["d2t"].to(torch.int64),
           "norm_weight": sd["norm.weight"].to(dtype), "lm_head_weight": T("lm_head.weight"),
           "tok_embedding": sd["embed_tokens.weight"].to(dtype)}
    names = ["midlayer"] + sorted({k.split(".")[0] + "." + k.split(".")[1] for k in sd.keys()
                                   if k.startswith("layers.")})
    for i, src in enumerate(names):
        p = f"layers.{i}."
        out[p + "qkv_weight"] = torch.cat([T(f"{src}.self_attn.q_proj.weight"), T(f"{src}.self_attn.k_proj.weight"),
                                           T(f"{src}.self_attn.v_proj.weight")], dim=-1).contiguous()
        out[p + "o_weight"] = T(f"{src}.self_attn.o_proj.weight")
        out[p + "input_layernorm_weight"] = sd[f"{src}.input_layernorm.weight"].to(dtype)
        out[p + "post_attention_layernorm_weight"] = sd[f"{src}.post_attention_layernorm.weight"].to(dtype)
        if f"{src}.hidden_norm.weight" in sd:
            out[p + "hidden_norm_weight"] = sd[f"{src}.hidden_norm.weight"].to(dtype)
        out[p + "gate_up_weight"] = torch.cat([T(f"{src}.mlp.gate_proj.weight"), T(f"{src}.mlp.up_proj.weight")],
                                              dim=-1).contiguous()
        out[p + "down_weight"] = T(f"{src}.mlp.down_proj.weight")
    return out


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model-name", required=True)
    ap.add_argument("--output-dir", required=True)
    args = ap.parse_args()
    save_shard(convert(LazyCheckpoint(args.model_name)), args.output_dir, 0)
    print(f"wrote drafter shard to {args.output_dir}")


if __name__ == "__main__":
    main()
