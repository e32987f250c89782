# -*- coding: utf-8 -*-
"""Single-launch momentum SGD over all parameters of a model (``csrc/multi_tensor_sgd.cu``).

Used by ``DistributedOptimizer`` on one GPU (where the reference just calls
``torch.optim.SGD.step``, ``distributed_optimizer.py:428-431``), after local gradient accumulation,
and for the clipped LSTM update: the global L2 norm, the clip coefficient and the update are three
launches with no host synchronisation in between.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional

import torch

from . import _lib, counters
from .tables import GroupTable, HyperTable, ensure_momentum_buffers, param_group_index


def _stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


class FastSGD:
    MAX_CTAS = 296           # 148 SMs x 2 resident 512-thread CTAs

    def __init__(self, optimizer, params: List[torch.Tensor], norm_clip: Optional[float] = None):
        self.lib = _lib.load()
        self.params = params
        self.device = params[0].device
        self.norm_clip = norm_clip
        momenta, created = ensure_momentum_buffers(optimizer, params)
        self.first_step = created
        self.fallback_steps = 0          # steps that went through torch.optim.SGD.step instead of the kernel
        self.table = GroupTable(params, param_group_index(optimizer, params), momenta, self.device)
        self.hyper = HyperTable(self.device)
        self.n_ctas = max(1, min(self.MAX_CTAS, (self.table.n_vec + 2047) // 2048))
        self.partials = torch.zeros(self.n_ctas, dtype=torch.float32, device=self.device)
        self.clip_out = torch.ones(2, dtype=torch.float32, device=self.device)

    @classmethod
    def try_create(cls, optimizer, norm_clip: Optional[float] = None) -> Optional['FastSGD']:
        params = [p for g in optimizer.param_groups for p in g['params'] if p.requires_grad]
        if not params or any((not p.is_cuda) or p.dtype != torch.float32 for p in params):
            return None
        if len(optimizer.param_groups) > _lib.MAX_PARAM_GROUPS:
            return None
        return cls(optimizer, params, norm_clip)

    def grad_norm(self) -> torch.Tensor:
        """Global L2 norm of the current gradients as a device scalar (after :meth:`step` with a clip)."""
        return self.clip_out[0]

    def step(self, optimizer, grad_scale: float = 1.0):
        grads = [p.grad for p in self.params]
        if any(g is None for g in grads) or any(g.stride() != p.stride() for g, p in zip(grads, self.params)):
            # a parameter without gradient, or an unusual gradient layout: use the stock update (which also creates
            # and fills the momentum buffers, so the next fast step must not treat them as fresh)
            self.first_step = False
            self.fallback_steps += 1
            return optimizer._base_cls.step(optimizer)
        self.table.refresh_grads(grads)
        if not torch.cuda.is_current_stream_capturing():
            self.hyper.sync(optimizer.param_groups)
        s = _stream_ptr()
        clip_ptr = None
        if self.norm_clip is not None:
            _lib.check(self.lib.mgw_group_sumsq(C.byref(self.table.struct), self.partials.data_ptr(), self.n_ctas, s), 'group_sumsq')
            _lib.check(self.lib.mgw_clip_coef(self.partials.data_ptr(), self.n_ctas, float(self.norm_clip),
                                              self.clip_out.data_ptr(), s), 'clip_coef')
            clip_ptr = self.clip_out.data_ptr() + 4
            counters.bump('group_sumsq')
            counters.bump('clip_coef')
        _lib.check(self.lib.mgw_multi_tensor_sgd(C.byref(self.table.struct), self.hyper.data_ptr(), clip_ptr,
                                                 float(grad_scale), int(self.first_step), _lib.MODE_UPDATE, None,
                                                 self.n_ctas, s), 'multi_tensor_sgd')
        counters.bump('multi_tensor_sgd')
        self.first_step = False
        return None

    def sync_hyper(self, optimizer) -> None:
        self.hyper.sync(optimizer.param_groups)
