# -*- coding: utf-8 -*-
"""Helpers shared by the trainer, the optimizer and the CLIs."""
from .misc import (check_unique, create_path, force_insert_item, gen_random_id,  # noqa: F401
                   gen_threshold_from_normal_distribution, predict_allreduce_time_with_size,
                   topk, topk_perf_model, allgather_perf_model, get_approximate_sigma_scale,
                   predict_density_with_size_and_computation,
                   GbE_multi_p_ab_small, GbE_multi_p_ab_large, tenGbE_multi_p_ab)
