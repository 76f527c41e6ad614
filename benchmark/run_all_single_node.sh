#!/usr/bin/env bash
# Everything the single-node figures need, in one go: the environment report, the sweep over the
# models / GPU counts of a configuration file, the headline benchmark with both arms at 1, 2, 4
# and 8 GPUs, and the figures.
#
#   benchmark/run_all_single_node.sh [benchmark/configs/single_node_b200.cfg] [out_dir]
#
# Parity: benchmark/run_all_single_node.sh of the reference.
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
ROOT="$(dirname "$HERE")"
CFG="${1:-$HERE/configs/single_node_b200.cfg}"
OUT="${2:-$ROOT/results-$(date +%Y-%m-%d-%H%M%S)}"
mkdir -p "$OUT"
cd "$ROOT"
export MASTER_ADDR=127.0.0.1

python benchmark/bench_single_node.py env --append-to "$OUT/env.txt"
python benchmark/bench_single_node.py sweep --config "$CFG" --out "$OUT/sweep.tsv"

GPUS=$(python -c "import torch; print(torch.cuda.device_count())")
: > "$OUT/headline.jsonl"
for n in 1 2 4 8; do
  [ "$n" -le "$GPUS" ] || continue
  for impl in native reference; do
    if [ "$n" -eq 1 ]; then
      python bench.py --impl "$impl" --gpus 1 --steps 10 --warmup 3 | tail -1 >> "$OUT/headline.jsonl"
    else
      python -m torch.distributed.run --nnodes=1 --nproc-per-node "$n" --master-addr 127.0.0.1 \
        --master-port $((29600 + n)) bench.py --impl "$impl" --gpus "$n" --steps 10 --warmup 3 \
        | tail -1 >> "$OUT/headline.jsonl"
    fi
  done
done

python benchmark/plot/single_device.py "$OUT/headline.jsonl" "$OUT/single_device.svg"
python benchmark/plot/single_node.py "$OUT/headline.jsonl" "$OUT/single_node_headline.svg"
python benchmark/plot/single_node.py "$OUT/sweep.tsv" "$OUT/single_node_models.svg"
echo "results in $OUT"
