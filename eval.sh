#!/bin/bash
# Example: evaluate the checkpoints of a finished run.
python evaluate.py --model-path "${model_path:-weights/allreduce/resnet20-n4-bs32-lr0.1000}" --dnn "${dnn:-resnet20}" \
    --dataset "${dataset:-cifar10}" --nepochs "${nepochs:-140}" --data-dir "${data_dir:-./data}"
