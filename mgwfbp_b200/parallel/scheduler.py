# -*- coding: utf-8 -*-
"""Gradient-merge schedules: which consecutive tensors share one all-reduce.

Pure functions (no torch, no communication) so they can be tested against the reference's
``_generate_groups_with_threshold`` / ``_generate_groups_mgwfbp``
(``distributed_optimizer.py:140-162`` and ``:164-261``).

Conventions shared by both policies
-----------------------------------
* Inputs are in **forward order** (index 0 = first layer), like ``model.named_parameters()``.
* Groups are emitted in **backward order**: ``groups[0]`` holds the tensors whose gradients
  are produced first (the last layers) and, inside a group, names are ordered as they become
  ready.  The offset of a tensor inside its merged buffer follows that order.
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

from .costmodel import AlphaBeta


@dataclass
class MergeSchedule:
    groups: List[List[str]]
    key_groupidx: Dict[str, int]
    offsets: List[List[int]]            # element offset of each tensor inside its group buffer
    group_sizes: List[int]              # elements per group
    predicted: Dict[str, float] = field(default_factory=dict)

    @property
    def keys(self) -> List[str]:
        """Buffer key of every group: member names joined by ':' (reference :285)."""
        return [':'.join(g) for g in self.groups]

    def digest(self) -> str:
        """Stable hash of the schedule; ranks compare it before training starts."""
        h = hashlib.sha256()
        for g, offs in zip(self.groups, self.offsets):
            h.update(('|'.join(g) + '#' + ','.join(map(str, offs)) + ';').encode())
        return h.hexdigest()


def _finish(groups: List[List[str]], key_groupidx: Dict[str, int], size_of: Dict[str, int],
            predicted: Optional[Dict[str, float]] = None) -> MergeSchedule:
    offsets, totals = [], []
    for g in groups:
        run, offs = 0, []
        for name in g:
            offs.append(run)
            run += size_of[name]
        offsets.append(offs)
        totals.append(run)
    return MergeSchedule(groups, key_groupidx, offsets, totals, predicted or {})


def check_unique(names: Sequence[str]) -> bool:
    """True when no layer name repeats (reference ``utils.py:160-167``)."""
    return len(set(names)) == len(names)


def groups_by_threshold(names: Sequence[str], sizes: Sequence[int], threshold: int) -> MergeSchedule:
    """Fixed-size bucketing over tensors visited last-to-first.

    A bucket is closed as soon as its accumulated **element count** reaches ``threshold``
    (so ``threshold=0`` gives one tensor per bucket -- plain WFBP -- and a huge threshold gives
    a single bucket).  Semantics of reference ``distributed_optimizer.py:140-162``.
    """
    size_of = dict(zip(names, sizes))
    groups: List[List[str]] = []
    key_groupidx: Dict[str, int] = {}
    current: List[str] = []
    filled = 0
    for name in reversed(list(names)):
        key_groupidx[name] = len(groups)
        current.append(name)
        filled += size_of[name]
        if filled >= threshold:
            groups.append(current)
            current, filled = [], 0
    if current:
        groups.append(current)
    return _finish(groups, key_groupidx, size_of)


def _comm_starts(tc: List[float], tb: Sequence[float], taob: List[float]) -> List[float]:
    """Earliest start of each layer's all-reduce: after its own backward finished and after
    the previous (deeper) layer's all-reduce completed."""
    L = len(tc)
    taoc = [0.0] * L
    taoc[L - 1] = taob[L - 1] + tb[L - 1]
    for l in range(L - 2, -1, -1):
        taoc[l] = max(taoc[l + 1] + tc[l + 1], taob[l] + tb[l])
    return taoc


def groups_mgwfbp(names: Sequence[str], sizes: Sequence[int], tb: Sequence[float],
                  cost: Callable[[float], float], bytes_per_elem: int = 4,
                  startup: Optional[Callable[[float], float]] = None) -> MergeSchedule:
    """MG-WFBP: merge layer ``l`` into ``l-1`` when sending it alone cannot be hidden.

    ``tb[l]`` is the measured backward time of layer ``l`` and ``cost(nbytes)`` the all-reduce
    model.  Walking from the last layer to the first, layer ``l``'s message is merged with its
    predecessor's when the predecessor's gradient becomes ready before ``l``'s all-reduce would
    finish and either (a) that all-reduce could not even have started yet, or (b) the wait
    until the predecessor is ready is shorter than one start-up latency.  Recurrences and the
    tie-breaking order follow reference ``distributed_optimizer.py:187-254`` exactly; the cost
    model is a callable so a per-algorithm piecewise model can be used.
    """
    names = list(names)
    if not check_unique(names):
        raise ValueError('layer names must be unique')
    L = len(names)
    if not (len(sizes) == L and len(tb) == L):
        raise ValueError('names, sizes and tb must have equal length')
    if startup is None:
        startup = getattr(cost, 'startup', None)
    if startup is None:
        a0 = cost(1) - (cost(2) - cost(1))
        startup = lambda nbytes, _a=a0: _a  # noqa: E731
    size_of = dict(zip(names, sizes))
    if L == 0:
        return _finish([], {}, size_of)
    p = list(sizes)
    tb = [float(t) for t in tb]
    tc = [cost(s * bytes_per_elem) for s in sizes]
    tc_unmerged_sum = float(sum(tc))
    taob = [0.0] * L
    for l in range(L - 2, -1, -1):
        taob[l] = taob[l + 1] + tb[l + 1]
    taoc = _comm_starts(tc, tb, taob)

    groups: List[List[str]] = []
    key_groupidx: Dict[str, int] = {names[L - 1]: 0}
    current: List[str] = []
    for l in range(L - 1, 0, -1):
        current.append(names[l])
        key_groupidx[names[l]] = len(groups)
        ready_prev = taob[l - 1] + tb[l - 1]
        merge = False
        if ready_prev < taoc[l] + tc[l]:
            if taoc[l] > ready_prev:
                merge = True
            elif ready_prev - taoc[l] < startup(p[l] * bytes_per_elem):
                merge = True
        if merge:
            tc[l] = 0.0
            p[l - 1] += p[l]
            p[l] = 0
            tc[l - 1] = cost(p[l - 1] * bytes_per_elem)
            taoc = _comm_starts(tc, tb, taob)
        else:
            groups.append(current)
            current = []
    key_groupidx[names[0]] = len(groups)
    current.append(names[0])
    groups.append(current)

    predicted = {
        'tc_sum': tc_unmerged_sum,
        'merged_tc_sum': float(sum(tc)),
        'non_overlapped': taoc[0] + tc[0] - (taob[0] + tb[0]),
        'tb_plus_tc': taoc[0] + tc[0],
        'tb_sum': float(sum(tb)),
    }
    return _finish(groups, key_groupidx, size_of, predicted)


def simulate_schedule(schedule: MergeSchedule, names: Sequence[str], sizes: Sequence[int],
                      tb: Sequence[float], cost: Callable[[float], float],
                      bytes_per_elem: int = 4) -> Dict[str, float]:
    """Predicted iteration timeline of an arbitrary schedule under the same model.

    Returns the backward time, the finish time of the last all-reduce and the part of
    communication that is not hidden under backward.  Used to compare WFBP / single-buffer /
    MG-WFBP predictions with measured iteration times.
    """
    names = list(names)
    L = len(names)
    idx = {n: i for i, n in enumerate(names)}
    taob = [0.0] * L
    for l in range(L - 2, -1, -1):
        taob[l] = taob[l + 1] + tb[l + 1]
    ready = [taob[l] + tb[l] for l in range(L)]
    t_comm_free = 0.0
    total_tc = 0.0
    for g, n_el in zip(schedule.groups, schedule.group_sizes):
        t_ready = max(ready[idx[n]] for n in g)
        start = max(t_ready, t_comm_free)
        c = cost(n_el * bytes_per_elem)
        total_tc += c
        t_comm_free = start + c
    tb_total = ready[0] if L else 0.0
    return {'tb_sum': tb_total, 'finish': t_comm_free, 'non_overlapped': max(t_comm_free - tb_total, 0.0),
            'merged_tc_sum': total_tc}
