# -*- coding: utf-8 -*-
"""Drop-in module for scripts that do ``import distributed_optimizer as hvd``."""
from mgwfbp_b200.parallel.runtime import (init, shutdown, size, local_size, rank, local_rank,  # noqa: F401
                                          broadcast, broadcast_object)
from mgwfbp_b200.parallel.optimizer import DistributedOptimizer, HookOrderError  # noqa: F401
from mgwfbp_b200.parallel.broadcast import broadcast_parameters, broadcast_optimizer_state  # noqa: F401
