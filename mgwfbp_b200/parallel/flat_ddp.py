# -*- coding: utf-8 -*-
"""Whole-model gradient averaging after backward: the simplest data-parallel wrapper.

The reference ships one beside its speech data tools (``audio_data/distributed.py:17-65``: broadcast the
state at construction, then after every backward pass flatten all gradients of one tensor type,
all-reduce, divide, copy back) together with ``reduce_tensor`` (``audio_data/utils.py:39-43``) for
averaging metrics.  It is the no-overlap baseline that WFBP and MG-WFBP improve on, and handy for
models whose optimizer is not wrapped.

Here the state goes out as one flat message per dtype (``broadcast_parameters``), and the gradients
are averaged in ONE flat buffer per dtype that is allocated once and reused; the callback is queued on
the autograd engine by the first gradient hook of a backward pass, so it runs exactly once when that
pass has finished.  Collectives run on the process group of :mod:`mgwfbp_b200.parallel.runtime`.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.distributed as dist
from torch.autograd import Variable

from . import runtime
from .broadcast import broadcast_parameters


def reduce_tensor(tensor: torch.Tensor, world_size: Optional[int] = None) -> torch.Tensor:
    """Average of ``tensor`` over all ranks as a new tensor (the input is left untouched)."""
    out = tensor.detach().clone()
    n = runtime.size() if world_size is None else int(world_size)
    if runtime.size() > 1:
        dist.all_reduce(out, op=dist.ReduceOp.SUM, group=runtime.data_group())
    out /= n
    return out


class FlatAllreduceDataParallel(torch.nn.Module):
    """``module`` with its state broadcast from rank 0 and its gradients averaged after each backward pass."""

    def __init__(self, module: torch.nn.Module):
        super().__init__()
        self.module = module
        self._flat: Dict[torch.dtype, torch.Tensor] = {}
        self._pending = False
        self.reductions = 0
        if runtime.size() > 1:
            broadcast_parameters(self.module.state_dict(), root_rank=0)
        for p in self.module.parameters():
            if p.requires_grad:
                p.register_hook(self._on_first_gradient)

    def _on_first_gradient(self, grad):
        if self._pending:
            self._pending = False
            Variable._execution_engine.queue_callback(self._average_gradients)
        return grad

    def _average_gradients(self) -> None:
        world = runtime.size()
        by_dtype: Dict[torch.dtype, List[torch.Tensor]] = {}
        for p in self.module.parameters():
            if p.requires_grad and p.grad is not None:
                by_dtype.setdefault(p.grad.dtype, []).append(p.grad)
        for dtype, grads in by_dtype.items():
            total = sum(g.numel() for g in grads)
            flat = self._flat.get(dtype)
            if flat is None or flat.numel() != total or flat.device != grads[0].device:
                flat = torch.empty(total, dtype=dtype, device=grads[0].device)
                self._flat[dtype] = flat
            views = flat.split([g.numel() for g in grads])
            torch._foreach_copy_(list(views), [g.reshape(-1) for g in grads])
            if world > 1:
                dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=runtime.data_group())
                flat /= world
            torch._foreach_copy_([g.view(-1) if g.is_contiguous() else g for g in grads],
                                 [v if g.is_contiguous() else v.view_as(g) for v, g in zip(views, grads)])
        self.reductions += 1

    def forward(self, *inputs, **kwargs):
        self._pending = True
        return self.module(*inputs, **kwargs)


# the reference's name for it
DistributedDataParallel = FlatAllreduceDataParallel
