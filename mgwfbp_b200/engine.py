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

import time
from typing import List, Optional, Sequence, Tuple

import torch

from .ops import counters
from .parallel.costmodel import PiecewiseAlphaBeta, fit_piecewise
from .parallel import runtime
from . import settings
from .settings import logger


class TrainStep:
    WARMUP_EAGER_STEPS = 3

    def __init__(self, trainer, use_graph: bool = True, loss_ring: int = 4, track_accuracy: bool = False):
        self.trainer = trainer
        self.track_accuracy = bool(track_accuracy)
        self.eager_after_capture = 0     # steps that ran eagerly after the capture because their batch had another shape
        self.replays, self.replay_host_s = 0, 0.0       # graph replays and the host time their launch calls took
        self._replayed_last = False
        self.optimizer = trainer.optimizer
        self.cuda = trainer.is_cuda
        comm = getattr(self.optimizer, '_comm', None)
        library_comm = comm is not None and comm.size() > 1 and not getattr(comm, 'fused', False)
        # not captured: CTC models (host-side label handling), the shadow checker (host round trips) and the stock arm
        # (torch.distributed work handles)
        self.want_graph = bool(use_graph and self.cuda and trainer.dnn != 'lstman4' and settings.SHADOW_EVERY <= 0
                               and not library_comm)
        self._static_hidden = None
        self.graphed = False
        self._graph: Optional[torch.cuda.CUDAGraph] = None
        self._static_batch: Optional[Tuple[torch.Tensor, ...]] = None
        self._static_loss: Optional[torch.Tensor] = None
        self._static_outputs = None
        self._static_labels = None
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

    def _track(self, loss: torch.Tensor, outputs, labels) -> None:
        """Epoch statistics on the device (no host read): the summed loss and, when asked for, the summed top-1
        accuracy, which ``DLTrainer._on_epoch_boundary`` averages and logs (reference ``dl_trainer.py:752-771``)."""
        t = self.trainer
        ld = loss.detach()
        if t._epoch_loss_t is None:
            t._epoch_loss_t = ld.clone()
        else:
            t._epoch_loss_t.add_(ld)
        if self.track_accuracy and outputs is not None and t.dnn not in ('lstm', 'lstman4'):
            with torch.no_grad():
                acc = (outputs.detach().argmax(1) == labels).float().mean().mul_(100.0)
            if t._acc_sum_t is None:
                t._acc_sum_t, t._acc_steps = acc.clone(), 1
            else:
                t._acc_sum_t.add_(acc)
                t._acc_steps += 1

    def _eager(self, batch) -> torch.Tensor:
        t = self.trainer
        t.optimizer.zero_grad()
        hidden_in = self._hidden
        if t.dnn == 'lstm' and self._static_hidden is not None:
            # after the capture the recurrent state lives in the static buffers; an eager step reads and refreshes them
            hidden_in = tuple(h.clone() for h in self._static_hidden) if self._shapes_match_hidden(batch) else None
        loss, outputs, labels, hidden = t.forward_loss(batch, hidden_in, on_device=True)
        if t.dnn == 'lstm':
            # keep only the values: a live reference into this step's autograd graph would keep its
            # gradient-accumulator nodes (and their stream) alive into the next step / a later capture
            from .models.lstm import repackage_hidden
            self._hidden = repackage_hidden(hidden)
            if self._static_hidden is not None and self._shapes_match_hidden(batch):
                for dst, src in zip(self._static_hidden, self._hidden):
                    dst.copy_(src)
        t.backward(loss)
        t.optimizer.step()
        self._track(loss, outputs, labels)
        return loss.detach()

    def _shapes_match_hidden(self, batch) -> bool:
        sb = self._static_batch
        return sb is not None and torch.is_tensor(batch[0]) and batch[0].shape == sb[0].shape

    def _same_shapes(self, batch) -> bool:
        sb = self._static_batch
        if sb is None or len(batch) != len(sb):
            return False
        for a, b in zip(sb, batch):
            if torch.is_tensor(a) != torch.is_tensor(b):
                return False
            if torch.is_tensor(a) and (a.shape != b.shape or a.dtype != b.dtype):
                return False
        return True

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
            loss, out, lab, hid = t.forward_loss(self._static_batch, self._static_hidden, on_device=True)
            t.backward(loss)
            t.optimizer.step()
            self._static_loss = loss.detach()
            self._static_outputs = out.detach() if (self.track_accuracy and torch.is_tensor(out)) else None
            self._static_labels = lab if torch.is_tensor(lab) else None
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
        if self.graphed and (batch is self._static_batch or self._same_shapes(batch)):
            if batch is not self._static_batch:
                for dst, src in zip(self._static_batch, batch):
                    if torch.is_tensor(dst):
                        dst.copy_(src, non_blocking=True)
            sync = getattr(self.trainer.optimizer, 'sync_hyper', None)
            if sync is not None:
                sync()                         # on the replaying stream: ordered after the previous replay, before this one
            t_host = time.perf_counter()
            self._graph.replay()
            self.replay_host_s += time.perf_counter() - t_host          # what the host spends handing one step to the driver
            self.replays += 1
            self._replayed_last = True
            counters.bump_many(self._launches_per_replay)
            self._track(self._static_loss, self._static_outputs, self._static_labels)
            return self._static_loss
        if self.graphed:
            # A batch of another shape (the short last batch of an epoch): this one step runs eagerly.  The graph
            # re-uploads its own gradient-pointer slots on every replay, so the tables only have to forget what
            # they believe the device holds.
            self.eager_after_capture += 1
        if self._replayed_last:
            for tbl in _tables_of(self.trainer.optimizer):
                tbl.invalidate()
            self._replayed_last = False
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

    def check_status(self) -> None:
        """Raise :class:`CommTimeoutError` when a communication kernel of an earlier step gave up waiting for a peer
        (the kernels record that in host-mapped memory; reading it costs no synchronisation, so this runs every step,
        graph replay included), or when the weight-gradient GEMM reported a failed wait."""
        comm = getattr(self.optimizer, '_comm', None)
        check = getattr(comm, 'check_status', None)
        if check is not None:
            check()
        from .ops import wgrad
        wgrad.check_status_nosync()

    def _collect(self, force: int) -> None:
        if self.cuda:
            self.check_status()
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
        """Wait for every outstanding loss read (and look at the kernels' status words once more afterwards)."""
        self._collect(len(self._pending))
        if self.cuda:
            self.check_status()

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


def fit_comm_model(comm=None, iters: int = 20, n_ctas: Optional[int] = None) -> PiecewiseAlphaBeta:
    """Measure the fused all-reduce kernels of this box and fit one alpha-beta line per algorithm.

    The sweep covers the reference's 32 KB - 2 MB grid (``profiling.py:158``) in coarser steps
    and extends it to 64 MB so that the bandwidth term is resolved.  ``n_ctas`` caps the CTA count of
    the large-message algorithm (pass ``comm.overlap_ctas`` for the model of a message that runs beside
    backward; ``None`` for one that has the GPU to itself).  Rank 0's fit is broadcast;
    the returned piecewise model feeds ``DistributedOptimizer(cost_model=...)``."""
    from .parallel.comm.nvl import NvlComm
    from .ops import _lib
    from .utils.profiling import CommunicationProfiler
    comm = comm or NvlComm.shared()
    one_max = comm.oneshot_max_bytes // 4
    big = {v: k for k, v in _lib.ALGO_NAMES.items()}[comm.big_algo()]
    plans = {
        'oneshot': [n for n in (1024, 4096, 16384, 65536, 131072) if n <= one_max],
        big: [1 << k for k in range(15, 25)],
    }
    samples, ranges = {}, {}
    for algo, sizes in plans.items():
        cap = n_ctas if algo != 'oneshot' else None

        def op(t, average=True, name=None, _a=algo, _c=cap):
            want = None if _c is None else min(_c, comm.choose((t.numel() + 3) // 4)[1])
            return comm.allreduce_async_(t, average, name, algo=_a, n_ctas=want)
        prof = CommunicationProfiler(op, comm.synchronize, sizes, device=comm.device)
        samples[algo] = prof.benchmark(num_iters=iters)
        ranges[algo] = (0.0, float(comm.oneshot_max_bytes) + 1) if algo == 'oneshot' else (0.0, float('inf'))
    samples = runtime.broadcast_object(samples, 0)
    model = fit_piecewise(samples, ranges)
    for lo, hi, ab in model.pieces:
        logger.info('comm model %-8s%s alpha = %.2f us, beta = %.3e s/B (%.0f GB/s algorithm bandwidth)',
                    ab.name, '' if n_ctas is None else ' (<= %d CTAs)' % n_ctas, ab.alpha * 1e6, ab.beta,
                    1e-9 / ab.beta if ab.beta > 0 else float('inf'))
    return model


def fit_interference(trainer, comm=None, n_ctas: Optional[int] = None, message_bytes: int = 8 << 20,
                     reps: int = 4, cost_model=None) -> dict:
    """How much does a communication kernel that runs beside backward slow backward down?

    The MG-WFBP recurrences (reference ``distributed_optimizer.py:164-261``) assume the answer is "not at all".
    On an NVSwitch box the kernel that moves a message shares SMs and memory bandwidth with the backward kernels, so
    this measures it on the running box: forward + backward of ``trainer``'s model is timed alone and then beside a
    side stream that runs all-reduce kernels of ``message_bytes`` with ``n_ctas`` CTAs back to back (the planned
    algorithm and CTA count of overlapped groups).  With ``t0`` / ``t1`` the two times and ``c`` the time the side
    stream was busy, ``rho = (t1 - t0) / min(c, t1)``: seconds of backward lost per second of overlapped
    communication.  Rank 0's value (from max-over-ranks times) is broadcast.  Collective; takes a few hundred ms.
    Returns ``{'rho', 't_alone_ms', 't_beside_ms', 'comm_busy_ms', 'n_ctas', 'messages'}``."""
    from .ops import _lib
    from .parallel.comm.nvl import NvlComm
    comm = comm or NvlComm.shared()
    if n_ctas is None:
        n_ctas = comm.overlap_ctas
    batch = trainer.to_device(trainer.data_iter())
    net = trainer.net

    def fwd_bwd():
        for p in net.parameters():
            p.grad = None
        loss, _o, _l, _h = trainer.forward_loss(batch, None, on_device=True)
        trainer.backward(loss)

    def timed(fn) -> float:
        torch.cuda.synchronize()
        runtime.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return runtime.max_over_ranks(e0.elapsed_time(e1) / reps)

    opt = trainer.optimizer
    was_local = getattr(opt, 'local', None)
    if was_local is not None:
        opt.local = True                       # hooks of an already wrapped optimizer stay quiet
    try:
        for _ in range(2):
            fwd_bwd()
        run = fwd_bwd
        graph = None
        if trainer.dnn != 'lstman4':
            try:                               # replay removes the launch gaps that would soak up the slow-down
                for p in net.parameters():
                    p.grad = None
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    loss, _o, _l, _h = trainer.forward_loss(batch, None, on_device=True)
                    trainer.backward(loss)
                run = graph.replay
            except Exception as e:
                logger.warning('interference fit: graph capture failed (%s); timing eager passes', e)
                torch.cuda.synchronize()
                graph, run = None, fwd_bwd
        run()
        t0 = timed(run)
        buf = torch.zeros(message_bytes // 4, device=comm.device)
        algo = {v: k for k, v in _lib.ALGO_NAMES.items()}[comm.big_algo()]
        want = min(n_ctas, comm.choose(buf.numel() // 4)[1])
        comm.synchronize(comm.allreduce_async_(buf, True, None, algo=algo, n_ctas=want))       # scratch + geometry settle here
        per_msg = float(cost_model(message_bytes)) * 1e3 if cost_model is not None else 0.1
        messages = int(runtime.broadcast_object(max(4, min(4000, int(1.5 * reps * t0 / max(per_msg, 1e-3)))), 0))
        torch.cuda.synchronize()
        runtime.barrier()
        side = comm.stream
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record(side)
        for _ in range(messages):
            comm.allreduce_async_(buf, True, None, algo=algo, n_ctas=want)
        s1.record(side)
        e0.record()
        for _ in range(reps):
            run()
        e1.record()
        torch.cuda.synchronize()
        comm.check_status()
        t1 = runtime.max_over_ranks(e0.elapsed_time(e1) / reps)
        busy = runtime.max_over_ranks(s0.elapsed_time(s1) / reps)
        del graph
    finally:
        if was_local is not None:
            opt.local = was_local
        for p in net.parameters():
            p.grad = None
    overlap = max(min(busy, t1), 1e-6)
    rho = min(max((t1 - t0) / overlap, 0.0), 1.0)
    rho = float(runtime.broadcast_object(rho, 0))
    out = {'rho': rho, 't_alone_ms': t0, 't_beside_ms': t1, 'comm_busy_ms': busy, 'n_ctas': int(want), 'messages': messages,
           'message_bytes': int(message_bytes)}
    logger.info('interference of a %d-CTA %s all-reduce beside forward+backward: rho = %.3f (%.3f ms alone, %.3f ms beside, '
                'side stream busy %.3f ms per pass)', want, algo, rho, t0, t1, busy)
    return out


def tune_schedule(trainer, build_optimizer, candidates: Sequence[dict], steps: int = 20, use_graph: bool = True):
    """Pick the merge schedule (and where the update runs) by running the candidates.

    ``build_optimizer(**candidate)`` must return a ``DistributedOptimizer`` around the SAME base optimizer; a candidate is
    a dict such as ``{'rho': 0.17, 'update': 'deferred'}`` (interference for the scheduler: 0 reproduces the reference's
    MG-WFBP schedule, 1 collapses to one message; update mode: see ``settings.UPDATE_MODE``).  Every distinct
    (schedule, update mode) that results is trained for a few steps through :class:`TrainStep` (eager warm-up, graph
    capture, ``steps`` timed replays on one device-resident batch; device time, max over ranks), and the fastest is
    rebuilt and installed with ``trainer.update_optimizer``.  Collective.  Returns ``(optimizer, report)`` where
    ``report`` lists the candidates with ``groups`` and ``ms_per_step``.  These are real training steps on real data."""
    batch = trainer.to_device(trainer.data_iter()) if trainer.is_cuda else trainer.data_iter()
    seen, report = {}, []
    for cand in candidates:
        opt = build_optimizer(**cand)
        key = (opt.merge_schedule.digest(), getattr(opt, '_update_mode', ''), tuple(sorted(getattr(opt, '_late_groups', ()))))
        row = dict(cand, groups=len(opt.merge_schedule.groups), update=getattr(opt, '_update_mode', None),
                   late_groups=sorted(getattr(opt, '_late_groups', ())),
                   group_mb=[round(4e-6 * n, 2) for n in opt.merge_schedule.group_sizes])
        if key in seen:
            opt.close()
            report.append(dict(row, ms_per_step=seen[key], same_as_earlier=True))
            continue
        trainer.update_optimizer(opt)
        step = TrainStep(trainer, use_graph=use_graph)
        for _ in range(TrainStep.WARMUP_EAGER_STEPS + 2):
            step.run_on_device(batch)
        ms = _time_replays(step, batch, steps)
        seen[key] = ms
        report.append(dict(row, ms_per_step=ms))
        step.drain()
        del step
        opt.close()
    fresh = [r for r in report if not r.get('same_as_earlier')]
    best = min(range(len(fresh)), key=lambda i: (fresh[i]['ms_per_step'], fresh[i]['groups']))
    best = int(runtime.broadcast_object(best, 0))
    chosen = {k: fresh[best][k] for k in candidates[0].keys()}
    opt = build_optimizer(**chosen)
    trainer.update_optimizer(opt)
    if runtime.rank() == 0:
        logger.info('schedule trial: %s -> %s (%d groups)',
                    [(r.get('rho'), r.get('update'), r['groups'], round(r['ms_per_step'], 3)) for r in report], chosen,
                    len(opt.merge_schedule.groups))
    return opt, report


def _time_replays(step: 'TrainStep', batch, steps: int) -> float:
    if not step.cuda:
        import time
        t0 = time.perf_counter()
        for _ in range(steps):
            step.run_on_device(batch)
        return runtime.max_over_ranks((time.perf_counter() - t0) * 1e3 / steps)
    torch.cuda.synchronize()
    runtime.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step.run_on_device(batch)
    e1.record()
    torch.cuda.synchronize()
    return runtime.max_over_ranks(e0.elapsed_time(e1) / steps)


def build_distributed_optimizer(trainer, seq_layernames=None, layerwise_times=None, threshold: int = 0, norm_clip=None,
                                compression=None, writer=None, gradient_path=None, tune: bool = True,
                                fit_comm: bool = True, trial_steps: int = 20, use_graph: bool = True):
    """What the entry points do between profiling backward and the first training step (reference
    ``dist_trainer.py:55-66``: build the wrapped optimizer, broadcast the parameters), plus the measurements the merge
    scheduler needs on an NVSwitch box.

    With the fused NVLink data plane and the adaptive policy this (1) fits the all-reduce cost model of this box for a
    message that has the GPU to itself and for one that runs beside backward with ``comm.overlap_ctas`` CTAs
    (:func:`fit_comm_model`), (2) measures how much such a message slows backward down (:func:`fit_interference`),
    (3) builds the interference-aware MG-WFBP schedule for that value and a few neighbours and keeps the one that
    trains fastest (:func:`tune_schedule`).  In every other configuration it just wraps the optimizer.  Parameters are
    broadcast from rank 0 before the first step either way.  Returns ``(optimizer, info)``; ``info`` holds what was
    measured (``None`` entries where nothing was)."""
    from .parallel.broadcast import broadcast_parameters
    from .parallel.optimizer import DistributedOptimizer
    from .parallel.scheduler import groups_time_sliced
    base = trainer.optimizer
    named = list(trainer.net.named_parameters())
    info = {'interference': None, 'trial': None, 'cost_model': None, 'cost_model_overlapped': None}

    def build(rho=None, cost=None, cost_last=None, update=None, slices=None, late=False):
        schedule = None
        if slices:
            schedule = lambda n, s, t, _k=int(slices): groups_time_sliced(n, s, t, _k)      # noqa: E731
        return DistributedOptimizer(base, named_parameters=named, compression=compression, seq_layernames=seq_layernames,
                                    layerwise_times=layerwise_times, norm_clip=norm_clip, threshold=threshold, writer=writer,
                                    gradient_path=gradient_path, cost_model=cost, cost_model_last=cost_last, interference=rho,
                                    fused_update=update, schedule=schedule, late_full=bool(late))

    adaptive_fused = (runtime.size() > 1 and trainer.is_cuda and not settings.ORIGINAL_HOROVOD and settings.ADAPTIVE_MERGE
                      and layerwise_times is not None)
    if not adaptive_fused:
        opt = build()
        broadcast_parameters(trainer.net.state_dict(), root_rank=0)
        trainer.update_optimizer(opt)
        return opt, info
    from .parallel.comm.nvl import NvlComm
    comm = NvlComm.shared()
    cost_full = cost_ovl = None
    if fit_comm:
        cost_full = fit_comm_model(comm)
        cost_ovl = fit_comm_model(comm, n_ctas=comm.overlap_ctas)
        info['cost_model'] = [(ab.name, ab.alpha, ab.beta) for _lo, _hi, ab in cost_full.pieces]
        info['cost_model_overlapped'] = [(ab.name, ab.alpha, ab.beta) for _lo, _hi, ab in cost_ovl.pieces]
    broadcast_parameters(trainer.net.state_dict(), root_rank=0)
    if settings.INTERFERENCE_PINNED:
        rhos = [settings.INTERFERENCE]
    else:
        info['interference'] = fit_interference(trainer, comm, cost_model=cost_ovl)
        rho = info['interference']['rho']
        rhos = []
        for r in (rho, min(1.0, 2.0 * rho), 1.0):
            r = round(max(r, 1e-3), 4)
            if r not in rhos:
                rhos.append(r)
    mk = lambda rho, update, slices, late=False: build(rho, cost_ovl, cost_full, update, slices, late)      # noqa: E731
    # plain SGD without clipping may run its update inside the group kernels or once after backward: try both
    modes = ['fused', 'deferred'] if (norm_clip is None and settings.UPDATE_MODE == 'fused' and
                                      isinstance(base, torch.optim.SGD)) else [None]
    # schedules from the interference-aware MG-WFBP search, and time-sliced ones (messages ready at equal distances in
    # backward time + a small last message) that the cost model cannot tell apart from them
    candidates = [{'rho': r, 'update': m, 'slices': None, 'late': False} for m in modes for r in rhos]
    if not settings.INTERFERENCE_PINNED:
        candidates += [{'rho': None, 'update': m, 'slices': k, 'late': False} for m in modes for k in (3, 6)]
    if settings.TRY_LATE_GROUPS:
        # the same schedules with their late groups (ready within settings.LATE_GROUP_MS of the end of backward) given the
        # whole GPU; a candidate without such a group is recognised as a repetition and not run again
        candidates += [dict(c, late=True) for c in candidates]
    if tune and len(candidates) > 1:
        opt, info['trial'] = tune_schedule(trainer, mk, candidates, steps=trial_steps, use_graph=use_graph)
    else:
        opt = mk(**candidates[0])
        trainer.update_optimizer(opt)
    return opt, info
