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

``ShadowChecker`` is the second, slower check: it re-computes one whole iteration of the fused data
plane (pack, sum over ranks, 1/N, clip, weight decay, momentum, update) through an independent
path -- gradients gathered over the CPU control plane, summed in rank order, the update written
out in plain PyTorch -- and compares the parameters the fused kernels produced against it.
Replica agreement cannot see an error that every rank makes alike (a wrong scale, a dropped
tensor, a stale momentum); the shadow can.
"""
from __future__ import annotations

import math
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


class ShadowMismatchError(ReplicaDivergenceError):
    pass


def reference_sgd_update(w: torch.Tensor, g: torch.Tensor, buf: Optional[torch.Tensor], lr: float, weight_decay: float = 0.0,
                         momentum: float = 0.0, dampening: float = 0.0, nesterov: bool = False, first_step: bool = False
                         ) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """One momentum-SGD update written out tensor-wise (the arithmetic of ``torch.optim.SGD``, which the
    fused kernels reproduce); returns the new weight and the new momentum buffer without touching the inputs."""
    g = g.clone()
    if weight_decay != 0.0:
        g = g + weight_decay * w
    new_buf = buf
    if momentum != 0.0:
        if first_step or buf is None:
            new_buf = g.clone()
        else:
            new_buf = momentum * buf + (1.0 - dampening) * g
        g = g + momentum * new_buf if nesterov else new_buf
    return w - lr * g, new_buf


class ShadowChecker:
    """Lock-step shadow of the fused all-reduce + update path, run every ``every`` iterations.

    ``snapshot(opt, names, first_step)`` is called by the distributed optimizer right before a merged group is
    handed to the fused kernel (stream order puts the copies ahead of the kernel); ``verify(opt)`` after
    ``step()``.  The snapshots are moved to the host, all-gathered over the control plane (gloo) and summed in
    rank order, so the only code the two paths share is the hyper-parameter table of the optimizer.
    Layers updated from gathered activations (``GatheredWgradLinear``) are outside the merged groups and are
    not covered.
    """

    def __init__(self, every: int, rtol: float = 2e-5, atol: float = 1e-7):
        self.every = max(int(every), 1)
        self.rtol, self.atol = rtol, atol
        self.checked = 0
        self._snap: List[Tuple[str, torch.Tensor, torch.Tensor, Optional[torch.Tensor], bool]] = []

    def active(self, iteration: int) -> bool:
        return iteration % self.every == 0

    def snapshot(self, opt, names: Sequence[str], first_step: bool) -> None:
        with torch.no_grad():
            for name in names:
                p = opt._named_parameters[name]
                buf = opt.state.get(p, {}).get('momentum_buffer')
                self._snap.append((name, p.grad.detach().clone(), p.detach().clone(),
                                   None if buf is None else buf.detach().clone(), bool(first_step)))

    def verify(self, opt) -> int:
        """Compare the parameters now in place with the shadow's; returns the number of tensors checked."""
        if not self._snap:
            return 0
        snap, self._snap = self._snap, []
        world = runtime.size()
        flat = torch.cat([g.reshape(-1).float().cpu() for _, g, _, _, _ in snap])
        if world > 1:
            parts = runtime.allgather_tensor(flat)
            total = parts[0].clone()
            for other in parts[1:]:
                total += other                                  # rank order, as the kernels sum
            flat = total / float(world)
        coef = 1.0
        if getattr(opt, '_norm_clip', None) is not None:
            norm = math.sqrt(float((flat.double() ** 2).sum()))
            coef = min(1.0, float(opt._norm_clip) / (norm + 1e-6))
        hyper = {}
        for group in opt.param_groups:
            for p in group['params']:
                hyper[id(p)] = group
        off = 0
        for name, g, w, buf, first in snap:
            n = g.numel()
            avg = (flat[off:off + n] * coef).view(g.shape)
            off += n
            p = opt._named_parameters[name]
            h = hyper[id(p)]
            want, _ = reference_sgd_update(w.float().cpu(), avg, None if buf is None else buf.float().cpu(), float(h['lr']),
                                           float(h.get('weight_decay', 0.0)), float(h.get('momentum', 0.0)),
                                           float(h.get('dampening', 0.0)), bool(h.get('nesterov', False)), first)
            got = p.detach().float().cpu()
            if not torch.allclose(got, want, rtol=self.rtol, atol=self.atol):
                err = float((got - want).abs().max())
                raise ShadowMismatchError('parameter %s after the fused step differs from the shadow path: max |diff| = %.3e '
                                          '(iteration %d, rank %d)' % (name, err, getattr(opt, 'train_iter', -1), runtime.rank()))
        self.checked += len(snap)
        return len(snap)
