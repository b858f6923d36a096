"""gpt-oss-20b-shaped generation: attention sinks, sliding window on alternating layers, YaRN RoPE,
QKV / O / expert biases, clamped SwiGLU, top-k-then-softmax router
(reference entry point: examples/models/gpt_oss/gpt_oss.py:280-364).

    python examples/models/gpt_oss/gpt_oss.py -n 64 --batch 4
    python -m torch.distributed.run --nproc-per-node 4 --master-addr 127.0.0.1 examples/models/gpt_oss/gpt_oss.py \\
        --checkpoint ./tmp_gpt-oss-20b --model /path/to/gpt-oss-20b "Explain TCP slow start."
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
