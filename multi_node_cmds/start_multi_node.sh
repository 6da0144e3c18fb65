#!/bin/bash
# Start one torchrun agent on every node listed in HOSTS (ssh fan-out); counterpart of the reference's
# multi_node_cmds/startup.sh + start_multi_node.sh. Usage:
#   HOSTS="node0 node1" MASTER_ADDR=node0 ./start_multi_node.sh -s <scene> -m <model> --bvh_depth 4 \
#       --MAX_BATCH_SIZE 4 --MAX_LOAD 8 --iterations 60000
set -euo pipefail
HOSTS=(${HOSTS:?space separated host list})
MASTER_ADDR=${MASTER_ADDR:-${HOSTS[0]}}
MASTER_PORT=${MASTER_PORT:-29500}
GPUS_PER_NODE=${GPUS_PER_NODE:-8}
REPO=${REPO:-$(cd "$(dirname "$0")/.." && pwd)}
NNODES=${#HOSTS[@]}
for i in "${!HOSTS[@]}"; do
  ssh "${HOSTS[$i]}" "cd $REPO && NCCL_SOCKET_TIMEOUT=60000 nohup setsid python -m torch.distributed.run --nnodes=$NNODES \
    --node_rank=$i --nproc_per_node=$GPUS_PER_NODE --master_addr=$MASTER_ADDR --master_port=$MASTER_PORT main.py $* \
    > train_node$i.log 2>&1 & echo \$! > torchrun_$i.pid" &
done
wait
echo "started $NNODES nodes x $GPUS_PER_NODE GPUs; logs: train_node<i>.log on each host"
