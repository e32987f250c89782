# -*- coding: utf-8 -*-
"""Training-step driver: one call = inputs to the device, forward, backward (with the merged-gradient
communication launched from hooks), update, loss back to the host.

``TrainStep(trainer).run(host_batch)`` does what the reference's hot loop does per iteration
(``dist_trainer.py:77-95``: ``zero_grad`` / ``trainer.train(1)`` / ``trainer.update_model()``) with two
B200-oriented differences:

* the whole device side of the step (forward, backward, side-stream all-reduce + update kernels,
  optimizer) can be captured once into a **CUDA graph** and replayed, which removes the per-kernel
  launch cost that dominates small-batch steps on a GPU this fast.  Communication kernels keep
  their launch counters in device memory, and learning rates live in a device table refreshed
  before each replay, so replays stay correct while the schedule moves;
* the loss is copied to pinned host memory asynchronously and read one step later, so the host
  never stalls the device between steps (``drain()`` waits for what is outstanding).
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from .ops import counters
from .parallel.costmodel import PiecewiseAlphaBeta, fit_piecewise
from .parallel import runtime
from . import settings
from .settings import logger


class TrainStep:
    WARMUP_EAGER_STEPS = 3

    def __init__(self, trainer, use_graph: bool = True, loss_ring: int = 4):
        self.trainer = trainer
        self.optimizer = trainer.optimizer
        self.cuda = trainer.is_cuda
        self.want_graph = bool(use_graph and self.cuda and trainer.dnn != 'lstman4' and settings.SHADOW_EVERY <= 0)
        self._static_hidden = None
        self.graphed = False
        self._graph: Optional[torch.cuda.CUDAGraph] = None
        self._static_batch: Optional[Tuple[torch.Tensor, ...]] = None
        self._static_loss: Optional[torch.Tensor] = None
        self._eager_steps = 0
        self._launches_per_replay = {}
        self._hidden = None
        self._ring = loss_ring
        self._pending: List[Tuple[object, torch.Tensor]] = []
        self._pinned_losses = [torch.zeros(1).pin_memory() if self.cuda else torch.zeros(1) for _ in range(loss_ring)]
        self._slot = 0
        self.losses: List[float] = []
        # input prefetch: a copy stream moves the next host batch while the current step computes
        self._copy_stream = torch.cuda.Stream() if self.cuda else None
        self._prefetched = None          # (host_batch, device_batch, ready_event)
        self._staging_free: List[object] = []

    # ------------------------------------------------------------------ pieces
    def _host_bookkeeping(self):
        t = self.trainer
        t.adjust_learning_rate(t.train_epoch, t.optimizer)
        if t.train_iter % t.num_batches_per_epoch == 0 and t.train_iter > 0:
            t._on_epoch_boundary()
        t.train_iter += 1

    def _eager(self, batch) -> torch.Tensor:
        t = self.trainer
        t.optimizer.zero_grad()
        loss, outputs, labels, hidden = t.forward_loss(batch, self._hidden, on_device=True)
        if t.dnn == 'lstm':
            # keep only the values: a live reference into this step's autograd graph would keep its
            # gradient-accumulator nodes (and their stream) alive into the next step / a later capture
            from .models.lstm import repackage_hidden
            self._hidden = repackage_hidden(hidden)
        t.backward(loss)
        t.optimizer.step()
        return loss.detach()

    def _capture(self, batch) -> None:
        t = self.trainer
        self._static_batch = tuple(b.clone() if torch.is_tensor(b) else b for b in batch)
        t.optimizer.zero_grad(set_to_none=True)
        before = counters.snapshot()
        g = torch.cuda.CUDAGraph()
        torch.cuda.synchronize()
        if t.dnn == 'lstm':
            # the recurrent state lives in static buffers that the captured step reads and then overwrites
            start = self._hidden if self._hidden is not None else t.net.init_hidden()
            self._static_hidden = tuple(h.detach().clone() for h in start)
            self._hidden = None
        with torch.cuda.graph(g):
            loss, _o, _l, hid = t.forward_loss(self._static_batch, self._static_hidden, on_device=True)
            t.backward(loss)
            t.optimizer.step()
            self._static_loss = loss.detach()
            if self._static_hidden is not None:
                for dst, src in zip(self._static_hidden, hid):
                    dst.copy_(src.detach())
        self._launches_per_replay = counters.diff(before)
        self._graph = g
        self.graphed = True
        logger.info('training step captured in a CUDA graph (%d own kernel launches per replay)',
                    sum(self._launches_per_replay.values()))

    def _device_step(self, batch) -> torch.Tensor:
        if self.want_graph and not self.graphed and self._eager_steps >= self.WARMUP_EAGER_STEPS:
            try:
                self._capture(batch)
            except Exception as e:      # capture is an optimisation; fall back to eager execution
                logger.warning('CUDA graph capture failed (%s: %s); running eagerly', type(e).__name__, e)
                self.want_graph = False
                torch.cuda.synchronize()
                self.trainer.optimizer.zero_grad(set_to_none=True)
                for tbl in _tables_of(self.trainer.optimizer):
                    tbl.invalidate()
        if self.graphed:
            if batch is not self._static_batch:
                for dst, src in zip(self._static_batch, batch):
                    if torch.is_tensor(dst):
                        dst.copy_(src, non_blocking=True)
            sync = getattr(self.trainer.optimizer, 'sync_hyper', None)
            if sync is not None:
                sync()
            self._graph.replay()
            counters.bump_many(self._launches_per_replay)
            return self._static_loss
        self._eager_steps += 1
        return self._eager(batch)

    # ------------------------------------------------------------------ public
    def run_on_device(self, device_batch) -> torch.Tensor:
        """One training step on a batch that already lives on the device.  Returns the loss tensor."""
        self._host_bookkeeping()
        if self.graphed and self._static_batch is not None and device_batch is not self._static_batch:
            pass
        return self._device_step(device_batch)

    def prefetch(self, host_batch) -> None:
        """Start copying ``host_batch`` (pinned memory) to the device on the copy stream.  The next
        ``run(host_batch)`` with the same object uses the copy instead of issuing its own."""
        if not self.cuda or host_batch is None:
            return
        with torch.cuda.stream(self._copy_stream):
            dev = self.trainer.to_device(host_batch)
            ev = torch.cuda.Event()
            ev.record()
        self._prefetched = (host_batch, dev, ev)

    def _take_inputs(self, host_batch):
        pre = self._prefetched
        if pre is not None and pre[0] is host_batch:
            self._prefetched = None
            torch.cuda.current_stream().wait_event(pre[2])
            for t in pre[1]:
                if torch.is_tensor(t) and t.is_cuda:
                    t.record_stream(torch.cuda.current_stream())     # allocated on the copy stream, consumed here
            return pre[1]
        return self.trainer.to_device(host_batch)

    def run(self, host_batch, next_host_batch=None) -> Optional[float]:
        """One end-to-end step from a host batch.  Returns the most recent loss value that has
        arrived on the host (the loss of an earlier step), or ``None`` before the first arrives.
        ``next_host_batch`` (optional) is copied to the device on a second stream while this step
        computes, so that its host-to-device transfer is off the critical path of the next call."""
        self._host_bookkeeping()
        batch = self._take_inputs(host_batch)
        loss = self._device_step(batch)
        if next_host_batch is not None:
            self.prefetch(next_host_batch)
        if self.cuda:
            if len(self._pending) >= self._ring:
                self._collect(1)
            slot = self._pinned_losses[self._slot % self._ring]
            self._slot += 1
            slot.copy_(loss.reshape(1), non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
            self._pending.append((ev, slot))
            self._collect(0)
        else:
            self.losses.append(float(loss))
        return self.losses[-1] if self.losses else None

    def _collect(self, force: int) -> None:
        while self._pending:
            ev, slot = self._pending[0]
            if force > 0:
                ev.synchronize()
                force -= 1
            elif not ev.query():
                break
            self.losses.append(float(slot[0]))
            self._pending.pop(0)

    def reset_state(self) -> None:
        """Forget the recurrent state carried between steps (the reference starts every epoch of the PTB model from
        ``init_hidden()``, ``dist_trainer.py:74-76``).  No effect for feed-forward models."""
        self._hidden = None
        if self._static_hidden is not None:
            for h in self._static_hidden:
                h.zero_()

    def drain(self) -> None:
        """Wait for every outstanding loss read."""
        self._collect(len(self._pending))

    def last_loss(self) -> Optional[float]:
        self.drain()
        return self.losses[-1] if self.losses else None


def _tables_of(optimizer):
    out = []
    fast = getattr(optimizer, '_fast_sgd', None)
    if fast is not None:
        out.append(fast.table)
    comm = getattr(optimizer, '_comm', None)
    plans = getattr(comm, '_plans', {}).get(id(optimizer), []) if comm is not None else []
    out += [p.table for p in plans]
    if getattr(optimizer, '_nvl_all', None) is not None:
        out.append(optimizer._nvl_all)
    return out


def fit_comm_model(comm=None, iters: int = 20) -> PiecewiseAlphaBeta:
    """Measure the fused all-reduce kernels of this box and fit one alpha-beta line per algorithm.

    The sweep covers the reference's 32 KB - 2 MB grid (``profiling.py:158``) in coarser steps
    and extends it to 64 MB so that the bandwidth term is resolved.  Rank 0's fit is broadcast;
    the returned piecewise model feeds ``DistributedOptimizer(cost_model=...)``."""
    from .parallel.comm.nvl import NvlComm
    from .utils.profiling import CommunicationProfiler
    comm = comm or NvlComm.shared()
    one_max = comm.oneshot_max_bytes // 4
    plans = {
        'oneshot': [n for n in (1024, 4096, 16384, 65536, 131072) if n <= one_max],
        'nvls' if comm.nvls_available else 'twoshot': [1 << k for k in range(15, 25)],
    }
    samples, ranges = {}, {}
    for algo, sizes in plans.items():
        op = (lambda t, average=True, name=None, _a=algo: comm.allreduce_async_(t, average, name, algo=_a))
        prof = CommunicationProfiler(op, comm.synchronize, sizes, device=comm.device)
        samples[algo] = prof.benchmark(num_iters=iters)
        ranges[algo] = (0.0, float(comm.oneshot_max_bytes) + 1) if algo == 'oneshot' else (0.0, float('inf'))
    samples = runtime.broadcast_object(samples, 0)
    model = fit_piecewise(samples, ranges)
    for lo, hi, ab in model.pieces:
        logger.info('comm model %-8s alpha = %.2f us, beta = %.3e s/B (%.0f GB/s algorithm bandwidth)',
                    ab.name, ab.alpha * 1e6, ab.beta, 1e-9 / ab.beta if ab.beta > 0 else float('inf'))
    return model
