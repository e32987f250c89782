#!/bin/bash
# Single-GPU run:  dnn=resnet50 data_dir=synthetic ./single.sh
set -e
cd "$(dirname "$0")"
dnn="${dnn:-resnet50}"
source exp_configs/$dnn.conf
nstepsupdate="${nstepsupdate:-1}"
PY="${PY:-python}"
exec $PY dl_trainer.py --dnn $dnn --dataset $dataset --max-epochs $max_epochs --batch-size $batch_size \
    --data-dir $data_dir --lr $lr --nsteps-update $nstepsupdate ${max_iters:+--max-iters $max_iters}
