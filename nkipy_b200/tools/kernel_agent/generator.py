"""Kernel generation.  The reference asks an LLM (AWS Bedrock `converse` with a `submit_kernel` tool,
tools/kernel_agent/generator.py:20-163) for a NumPy kernel that uses a requested set of operations.
There is no network here, so generation is a pluggable client with a deterministic offline default:
`TemplateClient` composes a kernel from the operation catalogue.  A client only has to implement
`generate(ops, prompt) -> python source defining kernel(...) and make_inputs()`."""

from __future__ import annotations

import os
import random
from typing import List, Protocol

PROMPT_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "prompts")


class KernelClient(Protocol):
    def generate(self, ops: List[str], prompt: str) -> str: ...


def system_prompt() -> str:
    with open(os.path.join(PROMPT_DIR, "system.txt")) as f:
        return f.read()


_UNARY = {"exp": "np.exp({x} * 0.1)", "tanh": "np.tanh({x})", "abs": "np.abs({x})", "sqrt": "np.sqrt(np.abs({x}) + 1.0)",
          "square": "np.square({x})", "negative": "np.negative({x})", "sin": "np.sin({x})", "cos": "np.cos({x})",
          "log": "np.log(np.abs({x}) + 1.0)", "floor": "np.floor({x})", "ceil": "np.ceil({x})", "sign": "np.sign({x})"}
_BINARY = {"add": "({x} + {y})", "subtract": "({x} - {y})", "multiply": "({x} * {y})", "maximum": "np.maximum({x}, {y})",
           "minimum": "np.minimum({x}, {y})", "divide": "({x} / (np.abs({y}) + 1.0))"}
_REDUCE = {"sum": "np.sum({x}, axis=-1, keepdims=True)", "max": "np.max({x}, axis=-1, keepdims=True)",
           "mean": "np.mean({x}, axis=-1, keepdims=True)", "min": "np.min({x}, axis=-1, keepdims=True)"}


class TemplateClient:
    """Deterministic stand-in for the LLM: chains the requested operations into one kernel."""

    def __init__(self, seed: int = 0):
        self.rng = random.Random(seed)

    def generate(self, ops: List[str], prompt: str = "") -> str:
        body, cur = [], "a"
        for i, op in enumerate(ops):
            name = f"t{i}"
            if op in _UNARY:
                expr = _UNARY[op].format(x=cur)
            elif op in _BINARY:
                expr = _BINARY[op].format(x=cur, y="b")
            elif op in _REDUCE:
                expr = f"{cur} - {_REDUCE[op].format(x=cur)}"
            elif op == "matmul":
                expr = f"np.matmul({cur}, np.transpose({cur}, (1, 0))) @ b"
            elif op == "transpose":
                expr = f"np.transpose(np.transpose({cur}, (1, 0)), (1, 0))"
            elif op == "where":
                expr = f"np.where({cur} > 0, {cur}, 0.1 * {cur})"
            else:
                raise ValueError(f"the offline generator has no template for '{op}'")
            body.append(f"    {name} = {expr}")
            cur = name
        src = ["import numpy as np", "", "", "def kernel(a, b):", *body, f"    return {cur}", "", "",
               "def make_inputs(seed=0):", "    rng = np.random.default_rng(seed)",
               "    return [rng.standard_normal((16, 32)).astype(np.float32), "
               "rng.standard_normal((16, 32)).astype(np.float32)]", ""]
        return "\n".join(src)


class BedrockClient:
    """Placeholder for the reference's LLM backend: needs network access and AWS credentials."""

    def generate(self, ops: List[str], prompt: str = "") -> str:
        raise RuntimeError("LLM generation needs network access (AWS Bedrock); use --client template offline")


def load_kernel(source: str):
    ns: dict = {}
    exec(compile(source, "<generated-kernel>", "exec"), ns)
    return ns["kernel"], ns["make_inputs"]
