# -*- coding: utf-8 -*-
"""MG-WFBP data-parallel training for NVIDIA B200 / NVSwitch boxes.

``import mgwfbp_b200 as hvd`` gives the module-level surface the reference exposes through
``import distributed_optimizer as hvd`` (``dist_trainer.py:15``): ``init, rank, size, local_rank,
local_size, broadcast, DistributedOptimizer, broadcast_parameters, broadcast_optimizer_state``.
"""
from . import settings  # noqa: F401
from .parallel.runtime import (init, shutdown, rank, size, local_rank, local_size, broadcast,  # noqa: F401
                               broadcast_object, barrier, is_initialized)
from .parallel.optimizer import DistributedOptimizer, HookOrderError  # noqa: F401
from .parallel.broadcast import broadcast_parameters, broadcast_optimizer_state  # noqa: F401
from .parallel.scheduler import groups_by_threshold, groups_mgwfbp, MergeSchedule  # noqa: F401
from .parallel.costmodel import AlphaBeta, PiecewiseAlphaBeta, fit_alpha_beta  # noqa: F401

__version__ = '0.1.0'
