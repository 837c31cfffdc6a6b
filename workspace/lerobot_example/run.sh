#!/usr/bin/env bash
# Fine-tune on every visible GPU of this node: one process per GPU through torch.distributed.run.
#   CONFIG=/path/to.yml SEED=42 GPUS=0,1,2,3 bash workspace/lerobot_example/run.sh
set -euo pipefail

here="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
repo="$(cd "$here/../.." && pwd)"
config="${CONFIG:-$here/finetune_flow.yml}"
seed="${SEED:-42}"

if [[ -n "${GPUS:-}" ]]; then
  export CUDA_VISIBLE_DEVICES="$GPUS"
fi
if [[ -n "${CUDA_VISIBLE_DEVICES:-}" ]]; then
  IFS=',' read -r -a devs <<< "$CUDA_VISIBLE_DEVICES"
  nproc="${#devs[@]}"
else
  nproc="$(python -c 'import torch; print(max(torch.cuda.device_count(), 1))')"
fi
port="${PORT:-$((20000 + RANDOM % 20000))}"

echo "$(date '+%F %T') launching $nproc process(es), config $config, seed $seed, rendezvous 127.0.0.1:$port"
if [[ "$nproc" -eq 1 ]]; then
  exec python "$repo/train_qact.py" --config "$config" --seed "$seed"
fi
exec python -m torch.distributed.run --nnodes=1 --nproc-per-node "$nproc" \
  --master-addr 127.0.0.1 --master-port "$port" \
  "$repo/train_qact.py" --config "$config" --seed "$seed"
