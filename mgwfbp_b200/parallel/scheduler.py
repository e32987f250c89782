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


# ---------------------------------------------------------------------------------------------------------------
# Interference-aware selection
#
# The MG-WFBP recurrences treat communication that overlaps backward as free.  That holds when the wire is the
# bottleneck (the reference's Ethernet / InfiniBand clusters: a message costs hundreds of microseconds of NIC
# time and no GPU time).  With peer-memory kernels over NVLink the message itself takes tens of microseconds, but
# the kernel that moves it occupies SMs and memory bandwidth that the backward kernels running beside it want
# too, so every second of overlapped communication delays backward by a fraction `interference` of a second.
# Under that model many small hidden messages can cost more than a few large exposed ones, and the best
# schedule lies somewhere between the MG-WFBP one and a single buffer.  The selection below keeps the MG-WFBP
# machinery and searches that range: candidates are MG-WFBP schedules computed with the start-up term
# inflated by 1x, 1.5x, 2x, ... (each step merges more), fixed-size buckets, and one single group; every candidate is played
# through the interference-aware timeline with the TRUE cost model, and the earliest finish wins.

def simulate_contended(schedule: MergeSchedule, names: Sequence[str], sizes: Sequence[int], tb: Sequence[float],
                       cost: Callable[[float], float], interference: float, bytes_per_elem: int = 4,
                       cost_last: Optional[Callable[[float], float]] = None) -> Dict[str, float]:
    """Timeline of ``schedule`` when backward runs at rate ``1 - interference`` while a message is in flight.

    Messages are sent in group order, one at a time, each as soon as its last gradient exists and the
    previous message is done.  Returns the finish time of the iteration's backward + communication
    (``finish``), when backward itself ended (``backward_end``), the summed message time and the number of groups.
    ``cost_last`` (optional) prices the schedule's last message, which is launched when backward is over and may
    therefore use the whole GPU instead of the few CTAs an overlapped message gets.
    """
    rho = min(max(float(interference), 0.0), 1.0)
    names = list(names)
    idx = {n: i for i, n in enumerate(names)}
    L = len(names)
    # backward work done when layer l's gradient exists (backward runs from layer L-1 down to 0)
    done_at = [0.0] * L
    run = 0.0
    for l in range(L - 1, -1, -1):
        run += float(tb[l])
        done_at[l] = run
    total_work = run
    need = [max(done_at[idx[n]] for n in g) for g in schedule.groups]
    tcs = [float(cost(n_el * bytes_per_elem)) for n_el in schedule.group_sizes]
    if cost_last is not None and tcs:
        tcs[-1] = float(cost_last(schedule.group_sizes[-1] * bytes_per_elem))
    t = w = 0.0
    qi, G = 0, len(need)
    backward_end = 0.0 if total_work <= 0.0 else None
    eps = 1e-15
    rate = 1.0 - rho
    while True:
        if qi < G and w >= need[qi] - eps:
            # the link is idle and the next group is complete: its message runs to the end, backward crawls beside it
            gain = tcs[qi] * rate
            if backward_end is None and w + gain >= total_work - eps:
                backward_end = t + ((total_work - w) / rate if rate > 0.0 else 0.0)
            w = min(w + gain, total_work)
            t += tcs[qi]
            qi += 1
            continue
        if qi >= G and w >= total_work - eps:
            break
        target = need[qi] if qi < G else total_work           # nothing to send yet: backward runs alone
        t += max(target - w, 0.0)
        w = target
        if backward_end is None and w >= total_work - eps:
            backward_end = t
    return {'finish': t, 'backward_end': backward_end if backward_end is not None else t, 'tb_sum': total_work,
            'merged_tc_sum': float(sum(tcs)), 'groups': float(G)}


def groups_mgwfbp_contended(names: Sequence[str], sizes: Sequence[int], tb: Sequence[float],
                            cost: Callable[[float], float], interference: float, bytes_per_elem: int = 4,
                            startup: Optional[Callable[[float], float]] = None,
                            inflations: Sequence[float] = (1, 1.5, 2, 2.5, 3, 3.5, 4, 6, 8, 16, 32, 64, 256, 1024),
                            buckets: Sequence[int] = (1 << 18, 1 << 19, 1 << 20, 1 << 21, 1 << 22, 1 << 23, 1 << 24, 1 << 25),
                            cost_last: Optional[Callable[[float], float]] = None) -> MergeSchedule:
    """The MG-WFBP schedule that finishes first when overlapped communication slows backward down.

    ``interference`` = 0 returns exactly :func:`groups_mgwfbp`.  Otherwise the candidates described above are
    compared under :func:`simulate_contended`; ties go to the schedule with fewer groups.  The winner's
    ``predicted`` dict carries the comparison (``candidates``: inflation factor or minus the bucket size in elements,
    number of groups, predicted finish).
    """
    base = groups_mgwfbp(names, sizes, tb, cost, bytes_per_elem, startup)
    if interference <= 0.0 or len(names) <= 1:
        return base
    if startup is None:
        startup = getattr(cost, 'startup', None)
    if startup is None:
        a0 = cost(1) - (cost(2) - cost(1))
        startup = lambda nbytes, _a=a0: _a  # noqa: E731
    seen: Dict[str, MergeSchedule] = {}
    table = []
    best = None
    for k in inflations:
        if k == 1:
            cand = base
        else:
            cand = groups_mgwfbp(names, sizes, tb, (lambda nb, _k=k: cost(nb) + (_k - 1.0) * startup(nb)), bytes_per_elem,
                                 (lambda nb, _k=k: _k * startup(nb)))
        sig = cand.digest()
        if sig in seen:
            continue
        seen[sig] = cand
        sim = simulate_contended(cand, names, sizes, tb, cost, interference, bytes_per_elem, cost_last)
        table.append((float(k), len(cand.groups), sim['finish']))
        key = (sim['finish'], len(cand.groups))
        if best is None or key < best[0]:
            best = (key, cand, sim)
    # fixed-size buckets (in elements) fill the range between the inflated schedules and one single message
    for thr in list(buckets) + [1 << 62]:
        cand = groups_by_threshold(names, sizes, thr)
        sig = cand.digest()
        if sig in seen:
            continue
        seen[sig] = cand
        sim = simulate_contended(cand, names, sizes, tb, cost, interference, bytes_per_elem, cost_last)
        table.append((-float(thr), len(cand.groups), sim['finish']))
        key = (sim['finish'], len(cand.groups))
        if key < best[0]:
            best = (key, cand, sim)
    _, chosen, sim = best
    predicted = dict(chosen.predicted)
    predicted.update({'interference': float(interference), 'contended_finish': sim['finish'],
                      'contended_backward_end': sim['backward_end'], 'merged_tc_sum': sim['merged_tc_sum'],
                      'tb_sum': sim['tb_sum'], 'non_overlapped': sim['finish'] - sim['tb_sum'],
                      'tb_plus_tc': sim['finish'], 'tc_sum': base.predicted.get('tc_sum', 0.0), 'candidates': table})
    return MergeSchedule(chosen.groups, chosen.key_groupidx, chosen.offsets, chosen.group_sizes, predicted)


def groups_time_sliced(names: Sequence[str], sizes: Sequence[int], tb: Sequence[float], n_slices: int,
                       tail_elems: int = 256 * 1024) -> MergeSchedule:
    """Groups cut at equal intervals of BACKWARD TIME, plus a small last group.

    The MG-WFBP recurrences decide merges from the cost model alone; when overlapped messages are cheap but not free and
    the link is far faster than backward (NVLink), many schedules tie under that model and the recurrences tend to one
    large late message.  This policy spends the slack the other way round: the tensors whose gradients appear first are
    sent first, in ``n_slices`` messages that become ready at roughly equal distances in time, so each message has the
    rest of backward to hide under; the last message (the first layers, up to ``tail_elems`` elements) is kept small
    because nothing can hide it.  Used as extra candidates of the schedule trial (``engine.tune_schedule``)."""
    names = list(names)
    L = len(names)
    if not (len(sizes) == L and len(tb) == L):
        raise ValueError('names, sizes and tb must have equal length')
    size_of = dict(zip(names, sizes))
    if L == 0:
        return _finish([], {}, size_of)
    order = list(range(L - 1, -1, -1))                       # backward order
    # the tail: trailing tensors of the backward pass (layer 0 last) up to tail_elems elements, at least one tensor
    tail, acc = [order[-1]], sizes[order[-1]]
    for l in reversed(order[:-1]):
        if acc + sizes[l] > tail_elems:
            break
        tail.insert(0, l)
        acc += sizes[l]
    head = order[:L - len(tail)]
    groups: List[List[str]] = []
    if head:
        total = float(sum(tb[l] for l in head)) or 1.0
        n = max(1, min(int(n_slices), len(head)))
        cur: List[str] = []
        run, k = 0.0, 1
        for l in head:
            cur.append(names[l])
            run += float(tb[l])
            if run >= total * k / n - 1e-15 and k < n:
                groups.append(cur)
                cur = []
                k += 1
        if cur:
            groups.append(cur)
    groups.append([names[l] for l in tail])
    key_groupidx = {name: gi for gi, g in enumerate(groups) for name in g}
    return _finish(groups, key_groupidx, size_of, {'policy': float(n_slices)})
