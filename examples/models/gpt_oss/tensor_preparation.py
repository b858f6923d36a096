"""Shard a Hugging Face gpt-oss checkpoint (bf16 or MXFP4 experts) for `--world-size` ranks
(reference: examples/models/gpt_oss/tensor_preparation.py:60-230).

    python examples/models/gpt_oss/tensor_preparation.py --model-name /path/to/gpt-oss-20b \\
        --world-size 4 --output-dir ./tmp_gpt-oss-20b
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
    ap.add_argument("--model-name", required=True)
    ap.add_argument("--world-size", type=int, default=1)
    ap.add_argument("--output-dir", required=True)
    ap.add_argument("--moe-parallel", choices=["ep", "tp"], default="ep")
    args = ap.parse_args()
    prepare_checkpoint(get_config(args.model_name), args.model_name, args.output_dir, args.world_size,
                       args.moe_parallel, family="gpt_oss")
    print(f"wrote {args.world_size} shard(s) to {args.output_dir}")


if __name__ == "__main__":
    main()
