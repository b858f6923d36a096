"""A Llama-style decoder run through the tracing frontend: the layer, the embedding and the sampler are NumPy
kernel functions (`llama_kernels/`), compiled once with `DeviceKernel.compile_and_load` and called layer by layer
with device tensors -- the same way the reference drives its models
(examples/models/qwen3/qwen3.py:139-260 there).  Without a GPU the same functions run on NumPy arrays.

    python examples/models/llama/llama.py --layers 2 --batch 2 --prompt-len 16 -n 8
"""
from __future__ import annotations

import argparse
import os
import sys
import time
from typing import Dict, List, Optional

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(_HERE, "..", "..", ".."))
sys.path.insert(0, _HERE)

from llama_kernels import decode_layer, greedy_token, prefill_layer  # noqa: E402


def embed(ids, table):
    """Token embedding lookup: ids int32 [B, T] -> [B, T, H]."""
    return np.take(table, ids, axis=0)


def _np(t, dtype):
    """torch tensor (any float dtype) -> NumPy array of `dtype` (ml_dtypes bfloat16 included)."""
    import torch

    if isinstance(t, torch.Tensor):
        t = t.detach().to("cpu", torch.float32).numpy()
    return np.ascontiguousarray(t).astype(dtype)


class TracedLlama:
    """Weights and caches as device tensors, one compiled kernel per function and shape.

    backend "device": kernels are traced, compiled to a cubin and run by the C++ runtime;
    backend "numpy": the kernel functions are called directly on NumPy arrays (CPU direct mode)."""

    def __init__(self, cfg, weights: Dict, batch: int, prompt_len: int, max_seq_len: int, dtype=np.float32,
                 backend: Optional[str] = None, build_dir: Optional[str] = None):
        if cfg.is_moe or cfg.qk_norm:
            raise ValueError("this example covers dense Llama-style layers")
        self.cfg, self.batch, self.prompt_len, self.max_seq_len = cfg, batch, prompt_len, max_seq_len
        self.dtype = np.dtype(dtype)
        if backend is None:
            import torch

            backend = "device" if torch.cuda.is_available() else "numpy"
        self.backend = backend
        self.build_dir = build_dir
        self.scalars = dict(n_heads=cfg.num_heads, n_kv_heads=cfg.num_kv_heads, head_dim=cfg.head_dim,
                            rope_theta=float(cfg.rope_theta), norm_eps=float(cfg.rms_eps))
        d = self.dtype
        self.host = {"table": _np(weights["tok_embedding"], d), "final_norm": _np(weights["norm_weight"], d),
                     "lm_head": _np(weights["lm_head_weight"], d)}
        self.layers: List[Dict[str, np.ndarray]] = []
        for i in range(cfg.num_layers):
            p = f"layers.{i}."
            self.layers.append({
                "qkv_weight": _np(weights[p + "qkv_weight"], d), "o_weight": _np(weights[p + "o_weight"], d),
                "gate_up_weight": _np(weights[p + "gate_up_weight"], d), "down_weight": _np(weights[p + "down_weight"], d),
                "input_norm": _np(weights[p + "input_layernorm_weight"], d),
                "post_norm": _np(weights[p + "post_attention_layernorm_weight"], d),
                "cache_k": np.zeros((batch, max_seq_len, cfg.num_kv_heads, cfg.head_dim), d),
                "cache_v": np.zeros((batch, max_seq_len, cfg.num_kv_heads, cfg.head_dim), d)})
        self.kernels = {}
        if backend == "device":
            self._to_device()

    # ------------------------------------------------------------------ device backend
    def _to_device(self):
        from nkipy_b200.runtime import DeviceKernel, DeviceTensor

        cfg, B, T, H = self.cfg, self.batch, self.prompt_len, self.cfg.hidden_size
        d = self.dtype
        lw = self.layers[0]
        order = ["qkv_weight", "o_weight", "gate_up_weight", "down_weight", "input_norm", "post_norm", "cache_k",
                 "cache_v"]
        ex = [lw[k] for k in order]
        ids_p, ids_d = np.zeros((B, T), np.int32), np.zeros((B, 1), np.int32)
        x_p, x_d = np.zeros((B, T, H), d), np.zeros((B, 1, H), d)
        kw = dict(build_dir=self.build_dir) if self.build_dir else {}
        C = DeviceKernel.compile_and_load
        t0 = time.time()
        self.kernels = {
            "embed_prefill": C(embed, ids_p, self.host["table"], name="embed_prefill", **kw),
            "embed_decode": C(embed, ids_d, self.host["table"], name="embed_decode", **kw),
            "prefill": C(prefill_layer, x_p, *ex, name="prefill_layer", **self.scalars, **kw),
            "decode": C(decode_layer, x_d, np.zeros((1,), np.int32), *ex, name="decode_layer", **self.scalars, **kw),
            "sample_prefill": C(greedy_token, x_p, self.host["final_norm"], self.host["lm_head"],
                                name="sample_prefill", norm_eps=self.scalars["norm_eps"], **kw),
            "sample_decode": C(greedy_token, x_d, self.host["final_norm"], self.host["lm_head"],
                               name="sample_decode", norm_eps=self.scalars["norm_eps"], **kw),
        }
        self.compile_s = time.time() - t0
        self.dev = {k: DeviceTensor.from_numpy(v, k) for k, v in self.host.items()}
        self.dev_layers = [{k: DeviceTensor.from_numpy(v, f"l{i}.{k}") for k, v in lw.items()}
                           for i, lw in enumerate(self.layers)]
        self._DeviceTensor = DeviceTensor

    def _run_layers_device(self, which: str, x, start_pos=None):
        """x: DeviceTensor [B, T, H]; runs every layer in place of the residual stream, returns the last output."""
        kern = self.kernels[which]
        # an argument that the kernel writes through appears among the compiled inputs as
        # "<name>.must_alias_input" (the reference's naming): address every input by the name the kernel expects
        expected = {n.replace(".must_alias_input", ""): n for n in kern.input_info}
        for lw in self.dev_layers:
            by_arg = {"x": x, **{k: lw[k] for k in lw}}
            if start_pos is not None:
                by_arg["start_pos"] = start_pos
            inputs = {expected[k]: v for k, v in by_arg.items()}
            out = self._DeviceTensor.empty(x.shape, x.dtype, "output0")
            # the caches are written through: the same device tensors are passed as outputs
            kern(inputs=inputs, outputs={"output0": out, "cache_k": lw["cache_k"], "cache_v": lw["cache_v"]})
            x = out
        return x

    # ------------------------------------------------------------------ generation
    def generate(self, prompts, new_tokens: int) -> List[List[int]]:
        prompts = np.asarray(prompts, dtype=np.int32)
        B, T = prompts.shape
        if (B, T) != (self.batch, self.prompt_len):
            raise ValueError(f"compiled for prompts of shape {(self.batch, self.prompt_len)}, got {(B, T)}")
        if T + new_tokens > self.max_seq_len:
            raise ValueError("prompt + new tokens exceed the cache length")
        out = [[] for _ in range(B)]
        if self.backend == "numpy":
            x = embed(prompts, self.host["table"])
            for lw in self.layers:
                x = prefill_layer(x, *[lw[k] for k in lw], **self.scalars)
            tok = greedy_token(x, self.host["final_norm"], self.host["lm_head"], self.scalars["norm_eps"])
            for step in range(new_tokens):
                for b in range(B):
                    out[b].append(int(tok[b]))
                if step + 1 == new_tokens:
                    break
                x = embed(tok.reshape(B, 1).astype(np.int32), self.host["table"])
                pos = np.array([T + step], np.int32)
                for lw in self.layers:
                    x = decode_layer(x, pos, *[lw[k] for k in lw], **self.scalars)
                tok = greedy_token(x, self.host["final_norm"], self.host["lm_head"], self.scalars["norm_eps"])
            return out
        DT = self._DeviceTensor
        ids = DT.from_numpy(prompts, "ids")
        x = self.kernels["embed_prefill"](inputs={"ids": ids, "table": self.dev["table"]})["output0"]
        x = self._run_layers_device("prefill", x)
        head = {"final_norm": self.dev["final_norm"], "lm_head": self.dev["lm_head"]}
        tok = self.kernels["sample_prefill"](inputs={"x": x, **head})["output0"]
        pos = DT.from_numpy(np.array([T], np.int32), "start_pos")
        for step in range(new_tokens):
            host_tok = tok.numpy()
            for b in range(B):
                out[b].append(int(host_tok[b]))
            if step + 1 == new_tokens:
                break
            ids1 = DT.from_numpy(host_tok.reshape(B, 1).astype(np.int32), "ids")
            pos.write_from_numpy(np.array([T + step], np.int32))
            x = self.kernels["embed_decode"](inputs={"ids": ids1, "table": self.dev["table"]})["output0"]
            x = self._run_layers_device("decode", x, pos)
            tok = self.kernels["sample_decode"](inputs={"x": x, **head})["output0"]
        return out


def main(argv=None) -> int:
    import torch

    from nkipy_b200.models import config as C
    from nkipy_b200.models.weights import random_weights

    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--hidden", type=int, default=512)
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--prompt-len", type=int, default=16)
    ap.add_argument("-n", "--new-tokens", type=int, default=8)
    ap.add_argument("--backend", choices=["device", "numpy"], default=None)
    ap.add_argument("--dtype", choices=["float32", "bfloat16"], default="float32")
    args = ap.parse_args(argv)
    cfg = C.tiny(hidden_size=args.hidden, head_dim=64, num_heads=args.hidden // 64, num_kv_heads=max(1, args.hidden // 256),
                 intermediate_size=2 * args.hidden, vocab_size=2048, num_layers=args.layers)
    w = random_weights(cfg, seed=0, std=0.05)
    import ml_dtypes

    dtype = np.float32 if args.dtype == "float32" else ml_dtypes.bfloat16
    model = TracedLlama(cfg, w, args.batch, args.prompt_len, args.prompt_len + args.new_tokens, dtype=dtype,
                        backend=args.backend)
    g = torch.Generator().manual_seed(0)
    prompts = torch.randint(0, cfg.vocab_size, (args.batch, args.prompt_len), generator=g).numpy()
    t0 = time.time()
    toks = model.generate(prompts, args.new_tokens)
    dt = time.time() - t0
    print(f"backend {model.backend}: {args.batch * args.new_tokens} tokens in {dt:.2f} s")
    for b, t in enumerate(toks):
        print(b, t)
    return 0


if __name__ == "__main__":
    sys.exit(main())
