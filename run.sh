#!/bin/bash
# Launch train.py on every GPU of this node with the compressed collectives on: the counterpart of
# the reference's launch line (reference: run.sh:1 -- GPT-2-XL, batch 2 per GPU, seq 1024,
# `-q --zip-ccl --profiler`, error file and per-rank logs from torchelastic).
#   ./run.sh                      synthetic tokens, GPT-2-XL shape (no network needed)
#   ./run.sh hf                   the reference's data path: tatsu-lab/alpaca + gpt2-xl from the HF hub
#   MODEL_SHAPE=llama3-8b SEQ=4096 BATCH=1 ./run.sh       another shape
set -euo pipefail
cd "$(dirname "$0")"
NGPU=${NGPU:-$(nvidia-smi -L | wc -l)}
BATCH=${BATCH:-2}
SEQ=${SEQ:-1024}
export TORCHELASTIC_ERROR_FILE=${TORCHELASTIC_ERROR_FILE:-./error.json}
if [ "${1:-synthetic}" = "hf" ]; then
  DATA=(-d tatsu-lab/alpaca -m openai-community/gpt2-xl)   # the hub id of the reference's launch line
else
  DATA=(--synthetic --model-shape "${MODEL_SHAPE:-gpt2-xl}")
fi
exec python -m torch.distributed.run --standalone --local-addr 127.0.0.1 --nproc-per-node "$NGPU" \
  --redirects 3 --log-dir ./logs \
  train.py -e "${EXPERIMENT:-zipccl-b200}" "${DATA[@]}" -b "$BATCH" -s "$SEQ" \
  -q --zip-ccl --compress-rs ${PROFILE:+--profiler} "${@:2}"
