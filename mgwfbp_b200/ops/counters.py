# -*- coding: utf-8 -*-
"""Counts launches of this package's own CUDA kernels (per kernel family), for benchmark reports.

Python wrappers call :func:`bump` right after a successful native launch.  A replay of a captured
CUDA graph launches everything that was counted during its capture again; ``TrainStep`` adds that
amount per replay through :func:`bump_many`.
"""
from collections import Counter
from typing import Dict

_counts: Counter = Counter()


def bump(name: str, n: int = 1) -> None:
    _counts[name] += n


def bump_many(delta: Dict[str, int], times: int = 1) -> None:
    for k, v in delta.items():
        _counts[k] += v * times


def snapshot() -> Dict[str, int]:
    return dict(_counts)


def diff(before: Dict[str, int]) -> Dict[str, int]:
    return {k: v - before.get(k, 0) for k, v in _counts.items() if v - before.get(k, 0)}


def total() -> int:
    """Kernel launches counted so far.  Names that start with ``note:`` mark WHICH path a call took (for tests and the
    smoke run) on top of its launch count and are left out."""
    return int(sum(v for k, v in _counts.items() if not k.startswith('note:')))


def reset() -> None:
    _counts.clear()
