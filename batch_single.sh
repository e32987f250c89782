#!/bin/bash
# Single-GPU sweep over the models of the reference's batch_single.sh (one epoch each).
# Usage: [data_dir=/path] [models="resnet50 googlenet"] ./batch_single.sh
here="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
models="${models:-resnet50 googlenet resnet152 inceptionv4 densenet161 densenet201}"
export data_dir="${data_dir:-synthetic}" max_epochs="${max_epochs:-1}"
status=0
for model in $models; do
  echo "== $model"
  dnn="$model" "$here/single.sh" || { echo "$model failed" >&2; status=1; }
done
exit $status
