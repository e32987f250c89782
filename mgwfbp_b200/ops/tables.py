# -*- coding: utf-8 -*-
"""Device-side descriptor tables consumed by the fused kernels.

``GroupTable`` describes a set of tensors as one flat, float4-padded index space (the layout
``MgwGroup`` in ``csrc/common.cuh``): static per-tensor entries (parameter pointer, momentum
pointer, element count, parameter-group index), the float4 offset of every tensor, and a small
array of *current gradient pointers* that is refreshed only when autograd handed out a gradient
tensor at a new address.  ``HyperTable`` mirrors the optimizer's per-group hyper-parameters in
device memory so that a learning-rate change never alters kernel arguments.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch

from . import _lib

_TENSOR_DT = np.dtype([('param', '<u8'), ('mom', '<u8'), ('numel', '<i4'), ('pg', '<i4')])
_HYPER_DT = np.dtype([('lr', '<f4'), ('wd', '<f4'), ('momentum', '<f4'), ('dampening', '<f4'),
                      ('nesterov', '<i4'), ('pad', '<i4', (3,))])
assert _TENSOR_DT.itemsize == 24 and _HYPER_DT.itemsize == 32


def is_dense(p: torch.Tensor) -> bool:
    return p.is_contiguous() or p.is_contiguous(memory_format=torch.channels_last) or \
        (p.dim() == 5 and p.is_contiguous(memory_format=torch.channels_last_3d)) or \
        p.numel() == p.untyped_storage().nbytes() // p.element_size()


class _nullcontext:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


def _pinned_empty(n: int, dtype) -> torch.Tensor:
    t = torch.zeros(n, dtype=dtype)
    return t.pin_memory() if torch.cuda.is_available() else t


def _to_device_bytes(arr: np.ndarray, device: torch.device) -> torch.Tensor:
    host = torch.from_numpy(arr.view(np.uint8).reshape(-1).copy())
    return host.to(device)


class GroupTable:
    def __init__(self, params: Sequence[torch.Tensor], pg_index: Sequence[int],
                 momenta: Sequence[Optional[torch.Tensor]], device: torch.device):
        self.params = list(params)
        self.device = device
        n = len(self.params)
        numels = [p.numel() for p in self.params]
        nvecs = [(k + 3) // 4 for k in numels]
        voff = np.zeros(n + 1, dtype=np.int64)
        voff[1:] = np.cumsum(nvecs)
        if voff[-1] >= 2 ** 31:
            raise ValueError('group too large for 32-bit slot indices')
        self.n_tensors, self.n_vec = n, int(voff[-1])
        self.voff_host = voff.astype(np.int32)
        self.voff = torch.from_numpy(self.voff_host.copy()).to(device)
        table = np.zeros(n, dtype=_TENSOR_DT)
        for i, (p, pg, m) in enumerate(zip(self.params, pg_index, momenta)):
            if p.dtype != torch.float32 or not is_dense(p):
                raise ValueError('fused kernels need dense float32 parameters')
            if m is not None and m.stride() != p.stride():
                raise ValueError('momentum buffer layout differs from its parameter')
            table[i] = (p.data_ptr(), m.data_ptr() if m is not None else 0, numels[i], pg)
        self._momenta = list(momenta)          # keep the buffers alive
        self.tensors = _to_device_bytes(table, device)
        self.grad_ptrs = torch.zeros(max(n, 1), dtype=torch.int64, device=device)
        self._grad_ptr_cache: Optional[List[int]] = None
        # pinned staging slots, allocated once (no host allocation on the hot path): eager refreshes alternate
        # between slots 0 and 1; slot 2 belongs to CUDA graph capture -- a captured upload re-reads its slot on every
        # replay, so eager steps that run between replays must never write there
        self._pinned = [_pinned_empty(max(n, 1), torch.int64) for _ in range(3)]
        self._pinned_events: List[Optional[torch.cuda.Event]] = [None, None, None]
        self._slot = 0
        self._struct = _lib.MgwGroup(self.tensors.data_ptr(), self.grad_ptrs.data_ptr(), self.voff.data_ptr(), n, self.n_vec)

    @property
    def struct(self) -> _lib.MgwGroup:
        return self._struct

    def refresh_grads(self, grads: Sequence[torch.Tensor], stream: Optional[torch.cuda.Stream] = None) -> bool:
        """Point the table at this iteration's gradient tensors.  Returns True when a copy was issued."""
        return self.refresh_grad_ptrs([g.data_ptr() for g in grads], stream)

    def refresh_grad_ptrs(self, ptrs: Sequence[int], stream: Optional[torch.cuda.Stream] = None) -> bool:
        """As :meth:`refresh_grads` with raw device addresses (a gradient may live somewhere else than in ``p.grad``,
        e.g. already averaged in a communication staging area)."""
        ptrs = [int(p) for p in ptrs]
        if ptrs == self._grad_ptr_cache:
            return False
        capturing = torch.cuda.is_current_stream_capturing()
        if capturing:
            slot = 2
        else:
            self._slot ^= 1
            slot = self._slot
            ev = self._pinned_events[slot]
            if ev is not None:
                ev.synchronize()                   # the previous copy out of this slot has finished
        host = self._pinned[slot]
        host[:len(ptrs)] = torch.tensor(ptrs, dtype=torch.int64)
        with torch.cuda.stream(stream) if stream is not None else _nullcontext():
            self.grad_ptrs[:len(ptrs)].copy_(host[:len(ptrs)], non_blocking=True)
            ev = None
            if not capturing:
                ev = torch.cuda.Event()
                ev.record()
        self._pinned_events[slot] = ev
        self._grad_ptr_cache = ptrs
        return True

    def invalidate(self) -> None:
        self._grad_ptr_cache = None


class HyperTable:
    """``MgwHyper[MAX_PARAM_GROUPS]`` in device memory, re-uploaded only when a value changed."""

    def __init__(self, device: torch.device):
        self.device = device
        self._host = np.zeros(_lib.MAX_PARAM_GROUPS, dtype=_HYPER_DT)
        self.dev = torch.zeros(_lib.MAX_PARAM_GROUPS * _HYPER_DT.itemsize, dtype=torch.uint8, device=device)
        self._pinned = [_pinned_empty(self.dev.numel(), torch.uint8) for _ in range(2)]
        self._pinned_events: List[Optional[torch.cuda.Event]] = [None, None]
        self._slot = 0
        self._last = None

    def sync(self, param_groups, stream: Optional[torch.cuda.Stream] = None, lr_scale: float = 1.0) -> bool:
        if len(param_groups) > _lib.MAX_PARAM_GROUPS:
            raise ValueError('at most %d parameter groups are supported by the fused kernels' % _lib.MAX_PARAM_GROUPS)
        key = tuple((g['lr'] * lr_scale, g.get('weight_decay', 0.0), g.get('momentum', 0.0), g.get('dampening', 0.0),
                     bool(g.get('nesterov', False))) for g in param_groups)
        if key == self._last:
            return False
        for i, (lr, wd, mom, damp, nest) in enumerate(key):
            self._host[i] = (lr, wd, mom, damp, int(nest), (0, 0, 0))
        if torch.cuda.is_current_stream_capturing():
            # a copy captured into a graph would re-upload today's values on every replay;
            # callers refresh the table outside the graph before each replay instead
            raise RuntimeError('hyper-parameters changed during CUDA graph capture')
        self._slot ^= 1
        ev = self._pinned_events[self._slot]
        if ev is not None:
            ev.synchronize()
        host = self._pinned[self._slot]
        host.copy_(torch.from_numpy(self._host.view(np.uint8).reshape(-1).copy()))
        with torch.cuda.stream(stream) if stream is not None else _nullcontext():
            self.dev.copy_(host, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
        self._pinned_events[self._slot] = ev
        self._last = key
        return True

    def data_ptr(self) -> int:
        return self.dev.data_ptr()


def ensure_momentum_buffers(optimizer, params: Sequence[torch.Tensor]) -> (List[Optional[torch.Tensor]], bool):
    """Momentum buffers of ``params`` inside ``optimizer.state`` (created as zeros when absent).

    Returns the buffers (``None`` where the group has no momentum) and whether any had to be
    created, i.e. whether the next update is the very first one."""
    pg_of = {}
    for gi, g in enumerate(optimizer.param_groups):
        for p in g['params']:
            pg_of[p] = (gi, g)
    bufs, created = [], False
    for p in params:
        gi, g = pg_of[p]
        if g.get('momentum', 0.0) == 0.0:
            bufs.append(None)
            continue
        st = optimizer.state[p]
        buf = st.get('momentum_buffer')
        if buf is None or buf.stride() != p.stride():
            new = torch.zeros_like(p, memory_format=torch.preserve_format)
            if buf is not None:
                new.copy_(buf)
            else:
                created = True
            st['momentum_buffer'] = buf = new
        bufs.append(buf)
    return bufs, created


def param_group_index(optimizer, params: Sequence[torch.Tensor]) -> List[int]:
    pg_of = {p: gi for gi, g in enumerate(optimizer.param_groups) for p in g['params']}
    return [pg_of[p] for p in params]
