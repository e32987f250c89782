#!/bin/bash
# Sweep: models x merge policy (single buffer / per-tensor WFBP / MG-WFBP) x worker counts, one epoch each.
# MG-WFBP is the default policy of dist_trainer.py; a fixed threshold needs MGWFBP_ADAPTIVE_MERGE=0.
dnns=( "resnet50" "googlenet" "resnet152" "inceptionv4" "densenet161" "densenet201" )
policies=( "mgwfbp" "524288000" "0" )
ns=( "8" "4" "2" )
for dnn in "${dnns[@]}"; do
  for policy in "${policies[@]}"; do
    for nworkers in "${ns[@]}"; do
      if [ "$policy" == "mgwfbp" ]; then
        MGWFBP_ADAPTIVE_MERGE=1 max_epochs=1 dnn=$dnn nworkers=$nworkers data_dir="${data_dir:-synthetic}" ./dist_launch.sh
      else
        MGWFBP_ADAPTIVE_MERGE=0 max_epochs=1 dnn=$dnn threshold=$policy nworkers=$nworkers data_dir="${data_dir:-synthetic}" ./dist_launch.sh
      fi
    done
  done
done
