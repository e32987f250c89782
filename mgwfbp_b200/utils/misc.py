# -*- coding: utf-8 -*-
"""Small utilities with the names the reference's ``utils.py`` exports.

The communication-cost tables (``utils.py:62-88``) are measurement data from the reference
authors' 1 GbE / 10 GbE clusters and are reproduced as constants so that code written against
``utils.tenGbE_multi_p_ab`` and friends keeps working; nothing in this package's scheduler uses
them (it fits its own constants, see ``mgwfbp_b200.parallel.costmodel``).
"""
from __future__ import annotations

import hashlib
import math
import os
import time
from typing import Dict, List, Sequence, Tuple

import numpy as np

from ..parallel.costmodel import predict_allreduce_time_with_size  # noqa: F401  (re-export)
from ..parallel.scheduler import check_unique as _check_unique

# top-k selection cost constant (seconds per element*log2(element)); reference utils.py:62
s = 2.18896957e-10

# all-gather (a seconds, b seconds/byte) on 1 GbE, messages < 1 MB; reference utils.py:66-73
GbE_multi_p_ab_small: Dict[int, Tuple[float, float]] = {2: (1.6e-3, 1.0e-8), 4: (2.7e-3, 1.3e-8),
                                                        8: (4.0e-3, 1.5e-8), 16: (1.7e-3, 1.7e-8)}
# messages >= 1 MB; reference utils.py:76-81
GbE_multi_p_ab_large: Dict[int, Tuple[float, float]] = {2: (4.4e-3, 5.8e-9), 4: (5.6e-3, 7.4e-9),
                                                        8: (7.68e-3, 8.2e-9), 16: (2.1e-3, 1.7e-8)}
# all-reduce on 10 GbE; reference utils.py:83-88
tenGbE_multi_p_ab: Dict[int, Tuple[float, float]] = {2: (1.5e-5, 5.7e-11), 4: (3.6e-5, 1.1e-10),
                                                     8: (8.5e-5, 1.4e-10), 16: (1.4e-4, 2.0e-10)}


def gen_random_id() -> str:
    return hashlib.sha256(repr(time.time()).encode()).hexdigest()


def create_path(relative_path: str, base: str = None) -> str:
    """``mkdir -p`` relative to ``base`` (default: current directory); returns the path."""
    path = relative_path if os.path.isabs(relative_path) else os.path.join(base or os.getcwd(), relative_path)
    os.makedirs(path, exist_ok=True)
    return path


def force_insert_item(d: dict, key, val) -> None:
    d.setdefault(key, []).append(val)


def check_unique(names: Sequence) -> bool:
    return _check_unique(list(names))


def topk(tensor: np.ndarray, k: int):
    idx = np.abs(tensor).argsort()[-k:]
    return idx, tensor[idx]


def get_approximate_sigma_scale(density: float) -> float:
    if density > 0.7:
        return 0.5
    if density > 0.05:
        return 1.5
    if density > 0.01:
        return 2.0
    return 3.0


def topk_perf_model(x: float, s: float = s) -> float:
    """Cost of selecting the top-k of ``x`` elements: ``s * x * log2(x)``."""
    return 0.0 if x == 0 else s * x * math.log2(x)


def allgather_perf_model(x: float, P: int, density: float = 0.001, eth: str = 'GbE') -> float:
    """Sparse all-gather time for ``x`` parameters at ``density`` over ``P`` workers (values+indices)."""
    if x == 0:
        return 0.0
    size = x * P * 4 * density
    table = GbE_multi_p_ab_large if size >= 1024 * 1024 else GbE_multi_p_ab_small
    a, b = table[P]
    return (a + b * size) * 2


def predict_density_with_size_and_computation(m: float, comp_time: float, P: int) -> float:
    """The reference's sparsification planner is stubbed to a constant (``utils.py:127``)."""
    return 0.001


def gen_threshold_from_normal_distribution(p_value: float, mu: float, sigma: float):
    from scipy import stats
    z = stats.norm.ppf((1 - p_value) / 2)
    return mu + z * sigma, mu - z * sigma
