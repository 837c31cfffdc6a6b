#!/bin/bash
# One process per GPU on one node (the reference launches the same script through `accelerate launch`,
# workspace/lerobot_example/run.sh:1-23).
set -e
export CUDA_VISIBLE_DEVICES=${CUDA_VISIBLE_DEVICES:-0,1,2,3,4,5,6,7}
NUM_GPUS=$(echo "$CUDA_VISIBLE_DEVICES" | tr ',' '\n' | wc -l)
echo "[current time: $(date +'%Y-%m-%d %H:%M:%S')]"

code_dir="$(cd "$(dirname "$0")/../.." && pwd)"
config_path="${CONFIG:-$code_dir/workspace/lerobot_example/finetune_flow.yml}"
PORT=${PORT:-$((21000 + RANDOM % 30000))}
SEED=${SEED:-10239}

LAUNCHER="python -m torch.distributed.run --nnodes=1 --nproc-per-node $NUM_GPUS --master-addr 127.0.0.1 --master-port $PORT"
echo "Running: $LAUNCHER $code_dir/train_qact.py --config $config_path --seed $SEED"
$LAUNCHER "$code_dir/train_qact.py" --config "$config_path" --seed "$SEED"
