# -*- coding: utf-8 -*-
"""One-time state broadcasts from a root rank.

``broadcast_parameters`` and ``broadcast_optimizer_state`` keep the call shapes of reference
``distributed_optimizer.py:474-503`` and ``:506-622``.  The reference issues one Horovod
broadcast per ``state_dict`` entry (320 messages for ResNet-50, 1207 for DenseNet-201); here
entries are grouped by (device, dtype), flattened into one buffer per group, broadcast once and
scattered back, so start-up cost does not grow with the number of tensors.
"""
from __future__ import annotations

import collections
from typing import Dict, Iterable, List, Tuple, Union

import torch
import torch.distributed as dist

from . import runtime


def _named_tensors(params) -> List[Tuple[str, torch.Tensor]]:
    if isinstance(params, dict):
        items = sorted(params.items())
    elif isinstance(params, (list, tuple)):
        items = [p if isinstance(p, tuple) else (None, p) for p in params]
    else:
        raise ValueError('invalid params of type: %s' % type(params))
    return [(k, v) for k, v in items if torch.is_tensor(v)]


def _flat_broadcast(tensors: List[torch.Tensor], root_rank: int) -> None:
    buckets: Dict[Tuple[torch.device, torch.dtype], List[torch.Tensor]] = collections.OrderedDict()
    for t in tensors:
        buckets.setdefault((t.device, t.dtype), []).append(t)
    for (device, dtype), members in buckets.items():
        group = runtime.control_group() if device.type == 'cpu' else runtime.data_group()
        flat = torch.cat([m.detach().reshape(-1) for m in members]) if len(members) > 1 else members[0].detach().reshape(-1).clone()
        dist.broadcast(flat, src=root_rank, group=group)
        off = 0
        with torch.no_grad():
            for m in members:
                n = m.numel()
                if m.is_contiguous():
                    m.view(-1).copy_(flat[off:off + n])
                else:
                    m.copy_(flat[off:off + n].view(m.shape))
                off += n


def broadcast_parameters(params: Union[dict, Iterable], root_rank: int = 0) -> None:
    """Overwrite every tensor in ``params`` (a ``state_dict()`` or a list of tensors /
    ``(name, tensor)`` pairs) with rank ``root_rank``'s value.  Buffers such as BatchNorm running
    statistics and ``num_batches_tracked`` are included when a ``state_dict`` is passed."""
    named = _named_tensors(params)
    if runtime.size() == 1 or not named:
        return
    _flat_broadcast([t for _, t in named], root_rank)


def broadcast_optimizer_state(optimizer: torch.optim.Optimizer, root_rank: int = 0) -> None:
    """Make every rank's optimizer state and hyper-parameters equal to the root's.

    Tensor state (momentum buffers, Adam moments) is broadcast flat; scalar state and the
    ``param_groups`` options travel as one pickled object.  State that does not exist yet is
    materialised with a zero-gradient ``step()`` first, as Horovod does
    (reference ``:519-533``)."""
    if isinstance(optimizer, torch.optim.LBFGS):
        raise ValueError('cannot broadcast torch.optim.LBFGS state')
    if runtime.size() == 1:
        return
    state_dict = optimizer.state_dict()
    if len(state_dict['state']) == 0:
        saved = []
        for group in optimizer.param_groups:
            for p in group['params']:
                saved.append((p, p.grad))
                if p.requires_grad:
                    p.grad = torch.zeros_like(p)
        params_before = [p.detach().clone() for p, _ in saved]
        base = getattr(optimizer, '_base_cls', None)
        (base.step(optimizer) if base is not None else optimizer.step())
        with torch.no_grad():
            for (p, g), before in zip(saved, params_before):
                p.copy_(before)
                p.grad = g
        state_dict = optimizer.state_dict()

    # options and scalar state from the root
    def scalars(sd):
        groups = [{k: v for k, v in g.items() if k != 'params'} for g in sd['param_groups']]
        st = {pid: {k: v for k, v in s.items() if not torch.is_tensor(v)} for pid, s in sd['state'].items()}
        return groups, st
    groups, st = runtime.broadcast_object(scalars(state_dict), root_rank)
    for g_live, g_root in zip(optimizer.param_groups, groups):
        g_live.update(g_root)
    tensors = []
    for group in optimizer.param_groups:
        for p in group['params']:
            s = optimizer.state.get(p, {})
            for k in sorted(s):
                if torch.is_tensor(s[k]):
                    tensors.append(s[k])
    pid = 0
    for group in optimizer.param_groups:
        for p in group['params']:
            if pid in st and p in optimizer.state:
                optimizer.state[p].update(st[pid])
            pid += 1
    if tensors:
        _flat_broadcast(tensors, root_rank)
