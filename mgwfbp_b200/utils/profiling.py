# -*- coding: utf-8 -*-
"""Layer-wise backward profiler and communication profiler.

API of the reference's ``profiling.py``: ``benchmark(trainer)`` returns
``(seq_layernames, layerwise_times, layerwise_sizes)`` in forward order (``profiling.py:95-147``),
``Profiling(model)`` collects per-parameter gradient-ready timestamps (``:13-92``) and
``CommunicationProfiler(comm_op, sync_op, sizes).benchmark(num_iters)`` sweeps all-reduce sizes
(``:150-183``).

Differences in mechanism: on CUDA each hook records an event on the compute stream instead of
calling ``torch.cuda.synchronize()`` and reading the wall clock, so the measured per-layer time
is device time and the backward pass is not serialised layer by layer; hooks are removed when
profiling stops; the communication sweep is timed with CUDA events as well.
"""
from __future__ import annotations

import time
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.nn as nn


class Profiling(object):
    def __init__(self, model: nn.Module):
        if not isinstance(model, nn.Module):
            raise ValueError("Not a valid model, please provide a 'nn.Module' instance.")
        self.model = model
        self._named = [(k, p) for k, p in model.named_parameters() if p.requires_grad]
        self._seq_keys = [k for k, _ in self._named]
        self._numel = {k: p.numel() for k, p in self._named}
        self._backward_seq_keys: List[str] = []
        self._backward_key_sizes: List[int] = []
        self._is_profiling = False
        self._use_events = any(p.is_cuda for _, p in self._named)
        self._trials: List[List[Tuple[str, object]]] = []   # per trial: [(name, event|time)]
        self._starts: List[object] = []
        self._handles = []
        self._register_hooks()

    # hooks ---------------------------------------------------------------
    def _register_hooks(self) -> None:
        for name, p in self._named:
            self._handles.append(p.register_hook(self._make_hook(name)))

    def remove_hooks(self) -> None:
        for h in self._handles:
            h.remove()
        self._handles = []

    def _stamp(self):
        if self._use_events:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            return ev
        return time.perf_counter()

    def _make_hook(self, name: str) -> Callable:
        def hook(grad):
            if not self._is_profiling:
                return None
            if len(self._backward_seq_keys) != len(self._seq_keys) and name not in self._first_pass_seen:
                self._first_pass_seen.add(name)
                self._backward_seq_keys.append(name)
                self._backward_key_sizes.append(self._numel[name])
            self._trials[-1].append((name, self._stamp()))
            return None
        return hook

    # control -------------------------------------------------------------
    def start(self) -> None:
        """Begin one timed backward pass; call right before ``loss.backward()``."""
        if not hasattr(self, '_first_pass_seen'):
            self._first_pass_seen = set()
        self._is_profiling = True
        self._trials.append([])
        self._starts.append(self._stamp())

    def stop(self) -> None:
        self._is_profiling = False
        self.remove_hooks()

    def reset(self) -> None:
        self._trials, self._starts = [], []

    def get_backward_seq_keys(self) -> List[str]:
        return self._backward_seq_keys

    def get_backward_key_sizes(self) -> List[int]:
        return self._backward_key_sizes

    def get_layerwise_times(self) -> Tuple[np.ndarray, float]:
        """Mean seconds between consecutive gradient-ready points, in backward order."""
        if self._use_events:
            torch.cuda.synchronize()
        order = self._backward_seq_keys
        rows = []
        for start, trial in zip(self._starts, self._trials):
            last_stamp: Dict[str, object] = {}
            for name, stamp in trial:          # a shared parameter fires several times: keep the last
                last_stamp[name] = stamp
            if len(last_stamp) != len(order):
                continue
            prev, row = start, []
            for name in order:
                cur = last_stamp[name]
                if self._use_events:
                    dt = prev.elapsed_time(cur) * 1e-3
                else:
                    dt = cur - prev
                row.append(max(dt, 0.0))
                prev = cur
            rows.append(row)
        if not rows:
            raise RuntimeError('no complete backward pass was profiled')
        arr = np.asarray(rows, dtype=np.float64)
        return arr.mean(axis=0), float(arr.sum(axis=1).mean())


def _forward_loss(trainer, data):
    """One forward pass + loss on the trainer's model, for every model family."""
    return trainer.forward_loss(data, hidden='fresh')[0]


def benchmark(trainer, warmup: int = 5, iteration: int = 50):
    """Measure per-layer backward time on ``trainer.net`` (5 warm-up + 50 timed passes, as the
    reference).  Returns names, seconds and element counts in **forward** order."""
    p = Profiling(trainer.net)
    try:
        for i in range(iteration + warmup):
            data = trainer.data_iter()
            trainer.net.zero_grad(set_to_none=True)
            loss = _forward_loss(trainer, data)
            if trainer.is_cuda:
                torch.cuda.synchronize()
            if i >= warmup:
                p.start()
            loss.backward()
            if trainer.is_cuda:
                torch.cuda.synchronize()
            p._is_profiling = False
        layerwise_times, _total = p.get_layerwise_times()
        seq_keys = p.get_backward_seq_keys()
        sizes = p.get_backward_key_sizes()
    finally:
        p.stop()
        trainer.net.zero_grad(set_to_none=True)
    return seq_keys[::-1], list(layerwise_times[::-1]), sizes[::-1]


class CommunicationProfiler(object):
    """Time ``comm_op(tensor, average=True, name=...)`` + ``sync_op(handle)`` over message sizes.

    Default sweep: ``8192*i`` floats for ``i`` in 1..63 (32 KB .. 2 MB, reference
    ``profiling.py:158``) extended by powers of two up to 128 Mi floats so that the bandwidth
    term is resolved on NVLink.  Returns ``(sizes_in_elements, mean_seconds)``.
    """

    def __init__(self, comm_op, sync_op, sizes: Optional[Sequence[int]] = None, device=None):
        self.comm_op = comm_op
        self.sync_op = sync_op
        self.sizes = list(sizes) if sizes is not None else None
        self.device = torch.device(device) if device is not None else torch.device(
            'cuda' if torch.cuda.is_available() else 'cpu')

    def default_sizes(self) -> List[int]:
        small = [8 * 1024 * i for i in range(1, 64)]
        large = [1 << k for k in range(20, 28)] if self.device.type == 'cuda' else []
        return small + large

    def _time_block(self, fn, iters: int) -> float:
        if self.device.type == 'cuda':
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(iters):
                fn(i)
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) * 1e-3 / iters
        t0 = time.perf_counter()
        for i in range(iters):
            fn(i)
        return (time.perf_counter() - t0) / iters

    def benchmark(self, num_iters: int = 100):
        sizes = self.sizes if self.sizes is not None else self.default_sizes()
        warm = torch.rand(1024, device=self.device)
        for i in range(5):
            self.sync_op(self.comm_op(warm, average=True, name='warmup-%d' % i))
        elapsed = []
        for s in sizes:
            tensor = torch.rand(int(s), device=self.device)

            def once(i, _t=tensor, _s=s):
                self.sync_op(self.comm_op(_t, average=True, name='run-size%d-%d' % (_s, i)))
            once(-1)
            elapsed.append(self._time_block(once, num_iters))
        return list(sizes), elapsed
