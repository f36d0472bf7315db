#!/bin/bash
# Sweep over models x top_k x methods (the grid of the reference's run_all.sh:4-23), one 8-GPU box.
# Each model entry is name:tp:layers.  NPROC defaults to the GPUs visible on this box.  The grid and the run length
# can be cut down from the environment for a short pass:
#   NPROC=2 STEPS=30 TIME_FROM=15 TIME_TO=30 METHODS="3 0" TOPKS="1" ./run_all.sh
NPROC=${NPROC:-$(python -c "import torch; print(max(1, torch.cuda.device_count()))")}
STEPS=${STEPS:-100}
TIME_FROM=${TIME_FROM:-80}
TIME_TO=${TIME_TO:-95}
OUT=${OUT:-results}
read -r -a models <<< "${MODELS:-google/gemma-2-2b:1:28 meta-llama/Llama-3.2-3B:1:28 facebook/opt-2.7b:1:12}"
read -r -a methods <<< "${METHODS:-3 2 0}"
read -r -a top_k_values <<< "${TOPKS:-10 5 1}"
mkdir -p "$OUT"
for model_config in "${models[@]}"; do
  IFS=':' read -r model_name tp layers <<< "$model_config"
  for top_k in "${top_k_values[@]}"; do
    for method in "${methods[@]}"; do
      echo "Running: $model_name top_k=$top_k method=$method tp=$tp on $NPROC GPUs"
      python -m torch.distributed.run --nnodes=1 --nproc-per-node "$NPROC" --master-addr 127.0.0.1 --master-port 29533 \
        train.py --model_name "$model_name" --grad_checkpoint --tp "$tp" --method "$method" \
        --num_hidden_layers "$layers" --bucket_cap 128 --top_k "$top_k" -s "$STEPS" --time_from "$TIME_FROM" --time_to "$TIME_TO" \
        --time_file "$OUT/time.txt" --log_dir "$OUT" --metrics_out "$OUT/sweep.jsonl"
    done
  done
done
