#!/usr/bin/env bash
# Throughput of one fine-tuning configuration: takes an example config, swaps the model and the recipe, trains 20 steps on
# synthetic tokens and shows the run's throughput lines.  Counterpart of the reference's benchmarks/benchmark_sft.sh.
#   benchmarks/benchmark_sft.sh <model dir or hub id> [recipe: bf16|fp8-hybrid|nvfp4] [gpus] [example yaml]
set -euo pipefail
MODEL=${1:?model directory or hub id}
RECIPE=${2:-bf16}
GPUS=${3:-1}
HERE=$(cd "$(dirname "$0")/.." && pwd)
EXAMPLE=${4:-$HERE/examples/sft/qwen3-lora-bf16.yaml}
WORK=$(mktemp -d)
cp "$EXAMPLE" "$WORK/config.yaml"
cd "$HERE"
python -m surogate_b200.cli.main sft "$WORK/config.yaml" --model "$MODEL" --recipe "$RECIPE" --gpus "$GPUS" --max-steps 20 --synthetic-data \
    --output-dir "$WORK/out" 2>&1 | tee "$WORK/log.txt"
grep -E "tps" "$WORK/log.txt" | tail -5 || true
echo "run directory: $WORK"
