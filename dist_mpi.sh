#!/bin/bash
# The reference launcher's name (it wrapped mpirun + a hostfile); here it is the torchrun launcher.
exec "$(dirname "$0")/dist_launch.sh" "$@"
