#!/bin/bash
set -e
cd "$(dirname "$0")/../../.."
python examples/models/qwen3_embedding/example_retrieval.py --layers 4
