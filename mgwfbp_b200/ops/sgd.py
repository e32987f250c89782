# -*- coding: utf-8 -*-
"""Single-launch momentum SGD over all parameters of a model (``csrc/multi_tensor_sgd.cu``).

Used by ``DistributedOptimizer`` on one GPU (where the reference just calls
``torch.optim.SGD.step``, ``distributed_optimizer.py:428-431``), after local gradient accumulation,
and for the clipped LSTM update: the global L2 norm, the clip coefficient and the update are three
launches with no host synchronisation in between.
"""
from __future__ import annotations

import ctypes as C
import weakref
from typing import List, Optional

import torch

from .. import settings
from . import _lib, counters
from .tables import GroupTable, HyperTable, ensure_momentum_buffers, param_group_index


def _stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


class FastSGD:
    MAX_CTAS = 296           # 148 SMs x 2 resident 512-thread CTAs

    def __init__(self, optimizer, params: List[torch.Tensor], norm_clip: Optional[float] = None, external=()):
        self.lib = _lib.load()
        self.device = params[0].device
        self.norm_clip = norm_clip
        self.hyper = HyperTable(self.device)
        # Large linear layers fed by few rows (ops.wgrad.GatheredWgradLinear): their backward runs the tensor-core
        # weight-gradient GEMM whose epilogue IS the update, so dW is never written and these weights take no part in
        # the multi-tensor launch below.
        self._optimizer = weakref.ref(optimizer)
        self._ext = {}
        taken = set()
        for p, module in external:
            mom, created = ensure_momentum_buffers(optimizer, [p])
            self._ext[id(module)] = dict(param=p, module=module, mom=mom[0], pg=param_group_index(optimizer, [p])[0], first=created)
            module._exchange = self._fused_wgrad
            taken.add(id(p))
        params = [p for p in params if id(p) not in taken]
        self.params = params
        momenta, created = ensure_momentum_buffers(optimizer, params)
        self.first_step = created
        self.fallback_steps = 0          # steps that went through torch.optim.SGD.step instead of the kernel
        self.table = GroupTable(params, param_group_index(optimizer, params), momenta, self.device)
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
        external = []
        if norm_clip is None and settings.GATHERED_WGRAD and settings.FUSED_WGRAD_1GPU:
            for p in params:
                module = getattr(p, '_mgw_gathered', None)
                if (module is not None and module.gathered_is_profitable(1) and p.is_contiguous() and p.dim() == 2
                        and sum(1 for q in params if q is p) == 1):
                    external.append((p, module))
            if len(external) == len(params):
                external = external[:-1]         # the multi-tensor launch keeps at least one tensor
        return cls(optimizer, params, norm_clip, external)

    @property
    def external_layers(self) -> int:
        """How many layers are updated by the epilogue of their weight-gradient GEMM."""
        return len(self._ext)

    def _fused_wgrad(self, module, dy: torch.Tensor, x: torch.Tensor) -> None:
        """Backward of a large linear layer on one GPU: ``W -= lr * (...)`` straight from ``dy^T x`` (current stream)."""
        from . import wgrad
        st = self._ext[id(module)]
        opt = self._optimizer()
        if not torch.cuda.is_current_stream_capturing():
            self.hyper.sync(opt.param_groups)
        if dy.data_ptr() % 16:
            dy = dy.clone()                  # a view at an odd offset: the bulk-tensor loads need 16-byte aligned bases
        if x.data_ptr() % 16:
            x = x.clone()
        wgrad.wgrad_sgd_(dy, x, st['param'].data, st['mom'], self.hyper.data_ptr(), st['pg'],
                         scale=float(getattr(opt, '_grad_scale', 1.0)), first_step=bool(st['first']))
        st['first'] = False

    def release_external(self, optimizer) -> None:
        """Give the externally updated layers back to autograd and the multi-tensor launch (needed before gradients
        are accumulated over several backward passes)."""
        if not self._ext:
            return
        back = [st['param'] for st in self._ext.values()]
        for st in self._ext.values():
            st['module']._exchange = None
        first = self.first_step
        self.__init__(optimizer, self.params + back, self.norm_clip)
        self.first_step = first

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
