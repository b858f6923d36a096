"""Qwen3-30B-A3B-shaped generation: tensor-parallel attention, expert-parallel MoE, paged KV cache,
CUDA-graph decode (reference entry point: examples/models/qwen3/qwen3.py:450-541).

    python examples/models/qwen3/qwen3.py -n 64 --batch 8
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 examples/models/qwen3/qwen3.py \\
        --checkpoint ./tmp_qwen3 --model /path/to/Qwen3-30B-A3B "The capital of France is"
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", ".."))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from config import get_config  # noqa: E402

from nkipy_b200.models.runner import add_common_args, run_generation  # noqa: E402


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    add_common_args(ap)
    args = ap.parse_args()
    return run_generation(get_config(args.model), args)


if __name__ == "__main__":
    sys.exit(main())
