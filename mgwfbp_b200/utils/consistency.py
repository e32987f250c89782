# -*- coding: utf-8 -*-
"""Replica-consistency checks (the race detector of a data-parallel job).

Synchronous data parallelism keeps every replica bit-identical: all ranks apply the same arithmetic
to the same averaged gradients.  A data race in a communication kernel, a missed stream dependency
or a rank that silently skipped a message shows up as replicas that differ.  ``replica_fingerprint``
folds the raw bit patterns of a set of tensors into one 64-bit value on the device (one reduction
per tensor, one host read in total); ``check_replicas`` compares the values of all ranks over the
control plane and raises :class:`ReplicaDivergenceError` naming the first differing tensor.
The reference has no such check (Horovod is trusted); here it is cheap enough to run every few
hundred iterations (``ReplicaGuard``) and in the multi-GPU tests.
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import torch

from ..parallel import runtime


class ReplicaDivergenceError(RuntimeError):
    pass


def _bits_sum(t: torch.Tensor) -> torch.Tensor:
    """Order-independent 64-bit fold of a tensor's bit pattern (wrap-around integer sum)."""
    flat = t.detach().reshape(-1)
    if not flat.is_contiguous():
        flat = flat.contiguous()
    if flat.element_size() == 4:
        ints = flat.view(torch.int32)
    elif flat.element_size() == 2:
        ints = flat.view(torch.int16)
    elif flat.element_size() == 8:
        ints = flat.view(torch.int64)
    else:
        ints = flat.view(torch.uint8)
    return ints.to(torch.int64).sum()


def replica_fingerprint(named_tensors: Iterable[Tuple[str, torch.Tensor]]) -> Tuple[List[str], torch.Tensor]:
    names, sums = [], []
    for name, t in named_tensors:
        names.append(name)
        sums.append(_bits_sum(t))
    if not sums:
        return names, torch.zeros(0, dtype=torch.int64)
    return names, torch.stack(sums).cpu()          # one device->host transfer


def check_replicas(named_tensors: Iterable[Tuple[str, torch.Tensor]], what: str = 'parameters') -> None:
    """Raise if any rank's tensors differ bitwise from rank 0's (collective over the control plane)."""
    names, mine = replica_fingerprint(named_tensors)
    if runtime.size() == 1:
        return
    everyone = runtime.allgather_object(mine.tolist())
    ref = everyone[0]
    for r, other in enumerate(everyone[1:], start=1):
        if other != ref:
            bad = next((names[i] for i, (a, b) in enumerate(zip(ref, other)) if a != b), '<length mismatch>')
            raise ReplicaDivergenceError('%s of rank %d differ from rank 0, first at %s' % (what, r, bad))


class ReplicaGuard:
    """``guard.step()`` after every ``optimizer.step()``; every ``every`` calls the model's trainable
    parameters are compared across ranks."""

    def __init__(self, model: torch.nn.Module, every: int = 500, include_buffers: bool = False):
        self.model, self.every, self.include_buffers = model, max(int(every), 1), include_buffers
        self.calls = 0

    def step(self) -> bool:
        self.calls += 1
        if self.calls % self.every:
            return False
        items = [(n, p) for n, p in self.model.named_parameters() if p.requires_grad]
        if self.include_buffers:
            items += [(n, b) for n, b in self.model.named_buffers()]
        check_replicas(items)
        return True
