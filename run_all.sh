#!/bin/bash
# Sweep over models x top_k x methods (the grid of the reference's run_all.sh:4-23), one 8-GPU box.
# Each entry is name:tp:layers.  NPROC defaults to the GPUs visible on this box.
NPROC=${NPROC:-$(python -c "import torch; print(max(1, torch.cuda.device_count()))")}
STEPS=${STEPS:-100}
models=("google/gemma-2-2b:1:28" "meta-llama/Llama-3.2-3B:1:28" "facebook/opt-2.7b:1:12")
methods=(3 2 0)
top_k_values=(10 5 1)
for model_config in "${models[@]}"; do
  IFS=':' read -r model_name tp layers <<< "$model_config"
  for top_k in "${top_k_values[@]}"; do
    for method in "${methods[@]}"; do
      echo "Running: $model_name top_k=$top_k method=$method tp=$tp on $NPROC GPUs"
      python -m torch.distributed.run --nnodes=1 --nproc-per-node "$NPROC" --master-addr 127.0.0.1 --master-port 29533 \
        train.py --model_name "$model_name" --grad_checkpoint --tp "$tp" --method "$method" \
        --num_hidden_layers "$layers" --bucket_cap 128 --top_k "$top_k" -s "$STEPS" --metrics_out results/sweep.jsonl
    done
  done
done
