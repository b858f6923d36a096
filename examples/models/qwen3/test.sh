#!/bin/bash
# Smoke run of the Qwen3 example on N GPUs (default 1) with random-init weights.
set -e
N=${1:-1}
cd "$(dirname "$0")/../../.."
if [ "$N" = "1" ]; then
  python examples/models/qwen3/qwen3.py --layers 4 --batch 8 --prompt-len 128 -n 32
else
  python -m torch.distributed.run --nnodes=1 --nproc-per-node "$N" --master-addr 127.0.0.1 --master-port 29700 \
    examples/models/qwen3/qwen3.py --layers 4 --batch 8 --prompt-len 128 -n 32
fi
