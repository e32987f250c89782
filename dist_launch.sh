#!/bin/bash
# Distributed launcher: same environment interface as the reference's dist_mpi.sh
#   dnn=resnet20 nworkers=4 threshold=0 lr=0.1 batch_size=32 max_epochs=1 ./dist_launch.sh
# One process per GPU is started with torchrun instead of mpirun + hostfile.  For several nodes set
# nnodes / node_rank / master_addr on every node (nwpernode GPUs each).
set -e
cd "$(dirname "$0")"
dnn="${dnn:-resnet20}"
source exp_configs/$dnn.conf
nworkers="${nworkers:-4}"
threshold="${threshold:-0}"
nnodes="${nnodes:-1}"
node_rank="${node_rank:-0}"
master_addr="${master_addr:-127.0.0.1}"
master_port="${master_port:-29511}"
nwpernode="${nwpernode:-$(( nworkers / nnodes ))}"
nstepsupdate="${nstepsupdate:-1}"
PY="${PY:-python}"
GRADSPATH=./logs
export NCCL_DEBUG="${NCCL_DEBUG:-WARN}"

exec $PY -m torch.distributed.run --nnodes=$nnodes --node-rank=$node_rank --nproc-per-node=$nwpernode \
    --master-addr $master_addr --master-port $master_port \
    dist_trainer.py --dnn $dnn --dataset $dataset --max-epochs $max_epochs --batch-size $batch_size \
    --nworkers $nworkers --data-dir $data_dir --lr $lr --nsteps-update $nstepsupdate --nwpernode $nwpernode \
    --threshold $threshold --saved-dir $GRADSPATH ${max_iters:+--max-iters $max_iters}
