#!/bin/bash
# Launch N DiLoCo workers on one machine, each a separate torchrun over its own slice of the GPUs
# (reference: scripts/simulate_multi_node_diloco.sh).
#
#   ./simulate_multi_worker.sh <N workers> <GPUs per worker> -m prime_b200.train @configs/debug/diloco.toml [overrides]
#
# Worker i uses devices [i*G, (i+1)*G) (selected with PRIME_DEVICE_OFFSET so that all GPUs stay
# visible to every process and NVLink peer access between workers keeps working), reads data shard
# i of N, and logs to logs/log<i>.log. Ctrl-C stops every worker.
set -e
if [ "$#" -lt 3 ]; then
    echo "Usage: $0 <N> <gpus per worker> <python args ...>"
    exit 1
fi
N=$1; shift
G=$1; shift
export GLOBAL_ADDR=${GLOBAL_ADDR:-127.0.0.1}
export GLOBAL_PORT=${GLOBAL_PORT:-5565}
export GLOBAL_WORLD_SIZE=$N
BASE_PORT=${BASE_PORT:-10001}
mkdir -p logs
pids=()
cleanup() {
    echo "Stopping workers"
    for pid in "${pids[@]}"; do kill "$pid" 2>/dev/null || true; done
    wait
    exit 1
}
trap cleanup SIGINT SIGTERM
for i in $(seq 0 $((N - 1))); do
    GLOBAL_UNIQUE_ID=$i GLOBAL_RANK=$i PRIME_DEVICE_OFFSET=$((i * G)) WANDB_MODE=${WANDB_MODE:-disabled} \
    python -m torch.distributed.run --nproc-per-node="$G" --nnodes=1 --master-addr 127.0.0.1 --master-port $((BASE_PORT + i)) \
        "$@" --data.data_rank "$i" --data.data_world_size "$N" > "logs/log$i.log" 2>&1 &
    pids+=($!)
done
tail -f logs/log0.log &
tailpid=$!
for pid in "${pids[@]}"; do wait "$pid"; done
kill $tailpid 2>/dev/null || true
