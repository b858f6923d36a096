"""Convert a Hugging Face Qwen3-Embedding checkpoint to one shard
(reference: examples/models/qwen3_embedding/prepare_weights.py:37-148).

    python examples/models/qwen3_embedding/prepare_weights.py --model-name /path/to/Qwen3-Embedding-0.6B --output-dir ./tmp_emb
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", ".."))

from nkipy_b200.models.checkpoint import prepare_checkpoint  # noqa: E402
from nkipy_b200.models.config import qwen3_embedding  # noqa: E402


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model-name", required=True)
    ap.add_argument("--size", choices=["0.6b", "8b"], default="0.6b")
    ap.add_argument("--output-dir", required=True)
    args = ap.parse_args()
    prepare_checkpoint(qwen3_embedding(args.size), args.model_name, args.output_dir, 1, family="dense")
    print(f"wrote shard to {args.output_dir}")


if __name__ == "__main__":
    main()
