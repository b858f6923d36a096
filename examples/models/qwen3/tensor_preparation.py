"""Shard a Hugging Face Qwen3-MoE checkpoint for `--world-size` ranks
(reference: examples/models/qwen3/tensor_preparation.py:126-324).

    python examples/models/qwen3/tensor_preparation.py --model-name /path/to/Qwen3-30B-A3B \\
        --world-size 8 --output-dir ./tmp_qwen3 [--moe-parallel ep|tp]
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", ".."))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from config import get_config  # noqa: E402

from nkipy_b200.models.checkpoint import prepare_checkpoint  # noqa: E402


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model-name", required=True, help="directory with config.json and *.safetensors")
    ap.add_argument("--world-size", type=int, default=1)
    ap.add_argument("--output-dir", required=True)
    ap.add_argument("--moe-parallel", choices=["ep", "tp"], default="ep")
    args = ap.parse_args()
    prepare_checkpoint(get_config(args.model_name), args.model_name, args.output_dir, args.world_size,
                       args.moe_parallel, family="qwen3_moe")
    print(f"wrote {args.world_size} shard(s) to {args.output_dir}")


if __name__ == "__main__":
    main()
