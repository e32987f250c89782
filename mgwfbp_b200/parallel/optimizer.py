# -*- coding: utf-8 -*-
"""``DistributedOptimizer``: merged-gradient, wait-free-backpropagation data parallelism.

Public contract of the reference's ``_DistributedOptimizer`` / ``DistributedOptimizer``
(``distributed_optimizer.py:41-471``): the returned object is an instance of a dynamic subclass
of the wrapped optimizer's class built on its ``param_groups``; gradients are all-reduced
(averaged) group by group from hooks that fire as soon as each parameter's gradient has been
accumulated during ``backward()``; ``step()`` waits for the communication and applies the
update; ``local=True`` suppresses communication for gradient-accumulation micro-steps;
``synchronize()`` exposes the averaged gradients before ``step()``.

Two data planes sit behind the same object:

* **unfused** (CPU/gloo, or any communicator with ``fused == False``): gradients are packed
  into one flat buffer per group, all-reduced asynchronously, and ``p.grad`` is re-pointed at
  its slice of the buffer afterwards, exactly like reference ``:300-340,369-404``;
* **fused** (``NvlComm`` on a B200 NVSwitch box): one kernel launch per group on a side stream
  packs from a pointer table, reduces across GPUs through peer memory, applies 1/N and -- for
  plain SGD -- the weight-decay / momentum / learning-rate update in the same pass.  ``step()``
  then only makes the compute stream wait for the side stream.
"""
from __future__ import annotations

import math
import time
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import settings
from ..settings import logger
from . import runtime
from .comm import Communicator, LocalComm, make_communicator
from .costmodel import AlphaBeta, fit_alpha_beta, table_lookup
from .scheduler import MergeSchedule, groups_by_threshold, groups_mgwfbp, groups_mgwfbp_contended


class HookOrderError(RuntimeError):
    """Gradients became ready in an order different from the profiled layer sequence."""


def _is_plain_sgd(opt: torch.optim.Optimizer) -> bool:
    if not isinstance(opt, torch.optim.SGD):
        return False
    for g in opt.param_groups:
        if g.get('maximize', False):
            return False
    return True


class _DistributedMixin:
    """Behaviour mixed into a dynamic subclass of the user's optimizer class."""

    # ------------------------------------------------------------------ construction
    def _dist_init(self, base_optimizer, named_parameters, compression, seq_layernames, layerwise_times,
                   norm_clip, threshold, writer, gradient_path, comm, cost_model, fused_update, interference=None,
                   cost_model_last=None, schedule=None, late_full=False):
        self._wrapped = base_optimizer
        self._given_schedule = schedule
        self._late_full = bool(late_full)
        self._late_groups = frozenset()
        self._interference = interference
        self._cost_model_last = cost_model_last
        self._compression = compression
        self._density = 1
        self._profiling = False
        self._seq_layernames = list(seq_layernames) if seq_layernames is not None else None
        self._layerwise_times = list(layerwise_times) if layerwise_times is not None else None
        self._norm_clip = norm_clip
        self._threshold = threshold
        self._writer = writer
        self._gradient_path = gradient_path
        self.alpha = None
        self.beta = None
        self._cost_model = cost_model
        self.train_epoch = 0
        self.train_iter = 0
        self._local = False
        self._allreduce_timers: Dict[str, List[float]] = {}
        self._update_times: Dict[str, List[float]] = {}
        self._compression_timers: Dict[str, List[float]] = {}

        named_parameters = list(named_parameters) if named_parameters is not None else []
        if any(not isinstance(item, tuple) for item in named_parameters):
            raise ValueError('named_parameters should be a sequence of tuples (name, parameter), '
                             'usually produced by model.named_parameters().')
        if named_parameters:
            self._named_parameters = {k: v for k, v in named_parameters}
        else:
            self._named_parameters = {}
            for gi, group in enumerate(self.param_groups):
                for i, p in enumerate(group['params']):
                    # the reference reuses the per-group index, which collides across groups;
                    # qualify it so every tensor keeps a distinct name
                    key = 'allreduce.noname.%s' % i if gi == 0 else 'allreduce.noname.%d.%s' % (gi, i)
                    self._named_parameters[key] = p
        # Only tensors that receive gradients take part in communication.
        self._named_parameters = {k: v for k, v in self._named_parameters.items() if v.requires_grad}
        self._parameter_names = {v: k for k, v in self._named_parameters.items()}
        if self._seq_layernames is not None:
            missing = [k for k in self._seq_layernames if k not in self._named_parameters]
            if missing:
                raise ValueError('seq_layernames contains unknown parameters: %s' % missing[:3])
            self._sequential_keys = list(self._seq_layernames)
        else:
            self._sequential_keys = list(self._named_parameters.keys())
        self._seq_index = {k: i for i, k in enumerate(self._sequential_keys)}

        self._comm: Communicator = comm if comm is not None else self._default_comm()
        self._world = self._comm.size()
        self._base_is_sgd = _is_plain_sgd(base_optimizer)
        # fused_update: None (settings.UPDATE_MODE), True / 'fused', 'deferred', False / 'separate'
        want = settings.UPDATE_MODE if fused_update is None else fused_update
        want = {True: 'fused', False: 'separate'}.get(want, want)
        if want not in ('fused', 'deferred', 'separate'):
            raise ValueError("fused_update must be True, False, 'fused', 'deferred' or 'separate'")
        self._fused_comm = bool(getattr(self._comm, 'fused', False))
        in_plane = bool(self._fused_comm and self._base_is_sgd and norm_clip is None)
        self._fused_update = in_plane and want == 'fused'
        self._deferred_update = in_plane and want == 'deferred'
        self._update_mode = 'fused' if self._fused_update else ('deferred' if self._deferred_update else 'separate')
        self._grad_scale = 1.0           # see set_grad_scale
        self._shadow = None
        if settings.SHADOW_EVERY > 0 and self._fused_comm and self._base_is_sgd:
            from ..utils.consistency import ShadowChecker
            self._shadow = ShadowChecker(settings.SHADOW_EVERY)

        # Large linear layers fed by small batches exchange activations instead of weight gradients
        # (mgwfbp_b200.ops.wgrad.GatheredWgradLinear); their weights leave the merge schedule.
        self._external = []
        if (self._fused_update or self._deferred_update) and self._world > 1 and settings.GATHERED_WGRAD:
            for name, p in list(self._named_parameters.items()):
                module = getattr(p, '_mgw_gathered', None)
                if module is not None and module.gathered_is_profitable(self._world):
                    self._external.append((name, p, module))
        # Large 2-D weights for which gathering does not pay but whose gradient is a single GEMM: the GEMM's epilogue
        # scatters its tiles to their owner ranks and the owners broadcast the sums (csrc/wgrad_gemm_sm100.cu,
        # WG_MODE_SCATTER); these weights leave the merge schedule as well.  Works with every update mode and with clipping:
        # the result is an ordinary averaged gradient in p.grad.
        self._scatter = []
        if self._fused_comm and self._world > 1 and settings.SCATTER_WGRAD and not settings.FP16:
            taken = {id(p) for _n, p, _m in self._external}
            for name, p in list(self._named_parameters.items()):
                cand = getattr(p, '_mgw_scatter_candidate', False) or getattr(p, '_mgw_gathered', None) is not None
                if (cand and id(p) not in taken and p.is_cuda and p.dim() == 2 and p.dtype == torch.float32 and p.is_contiguous()
                        and p.shape[0] % 4 == 0 and p.shape[1] % 4 == 0 and p.numel() >= 4 * 1024 * 1024):
                    self._scatter.append((name, p))
        if self._external or self._scatter:
            gone = {name for name, _, _ in self._external} | {name for name, _ in self._scatter}
            if gone:
                self._named_parameters = {k: v for k, v in self._named_parameters.items() if k not in gone}
                self._parameter_names = {v: k for k, v in self._named_parameters.items()}
                keep = [i for i, k in enumerate(self._sequential_keys) if k not in gone]
                if self._layerwise_times is not None:
                    # the removed layer's backward time still elapses before the next gradient is ready
                    tb = list(self._layerwise_times)
                    for i, k in enumerate(self._sequential_keys):
                        if k in gone:
                            j = next((q for q in range(i - 1, -1, -1) if self._sequential_keys[q] not in gone),
                                     next((q for q in range(i + 1, len(tb)) if self._sequential_keys[q] not in gone), None))
                            if j is not None:
                                tb[j] += tb[i]
                    self._layerwise_times = [tb[i] for i in keep]
                self._sequential_keys = [self._sequential_keys[i] for i in keep]
                if self._seq_layernames is not None:
                    self._seq_layernames = list(self._sequential_keys)
                self._seq_index = {k: i for i, k in enumerate(self._sequential_keys)}
                logger.info('weights outside the merge schedule: %s updated through gathered activations, %s reduced by the '
                            'scatter epilogue of their gradient GEMM', sorted(n for n, _, _ in self._external),
                            sorted(n for n, _ in self._scatter))

        self._generate_merged_parameters()

        self._handles: Dict[int, tuple] = {}
        self._hook_handles = []
        self._requires_update = set()
        self._hook_checked_idx = 0
        self._groups_pending: List[int] = []
        self._synchronized = True
        # An explicitly supplied fused communicator is also used on a single GPU (the update then
        # overlaps with backward); otherwise one worker behaves like the plain optimizer.
        self._active = self._world > 1 or (self._fused_comm and comm is not None)
        if self._active:
            self._verify_schedule_agreement()
            self._register_hooks()
            if self._fused_comm:
                self._comm.attach(self)

    def _default_comm(self) -> Communicator:
        if runtime.size() == 1:
            return LocalComm()
        first = next(iter(self._named_parameters.values()), None)
        device = first.device if first is not None else torch.device('cpu')
        return make_communicator(device)

    # ------------------------------------------------------------------ schedule
    def _resolve_cost_model(self):
        if self._cost_model is not None:
            return self._cost_model
        if self.alpha is not None:
            return AlphaBeta(float(self.alpha), float(self.beta), 'measured')
        return table_lookup(settings.CONNECTION, self._world)

    def _generate_merged_parameters(self) -> None:
        names = self._sequential_keys
        sizes = [self._named_parameters[k].numel() for k in names]
        self._sizes = sizes
        if self._given_schedule is not None:
            # an explicit schedule (e.g. a candidate of the schedule trial); it must cover exactly the scheduled tensors
            sched = self._given_schedule
            if callable(sched):               # (names, sizes, layer-wise backward times) -> MergeSchedule
                sched = sched(names, sizes, self._layerwise_times)
            if sorted(n for g in sched.groups for n in g) != sorted(names):
                raise ValueError('the given merge schedule does not cover the optimizer\'s tensors')
        elif settings.ORIGINAL_HOROVOD and not self._fused_comm:
            # the stock arm: Horovod's tensor fusion is a fixed-size bucket, no profile involved
            sched = groups_by_threshold(names, sizes, settings.HOROVOD_FUSION_ELEMENTS)
        elif settings.ADAPTIVE_MERGE and self._layerwise_times is not None:
            if len(self._layerwise_times) != len(names):
                raise ValueError('layerwise_times and seq_layernames differ in length')
            nbytes = 2 if settings.FP16 else 4
            cost = self._resolve_cost_model()
            # kernels of the fused data plane compete with backward for SMs and bandwidth; other backends
            # (NCCL / gloo behind torch.distributed) are scheduled by the reference's recurrences unchanged
            rho = 0.0
            if self._fused_comm:
                rho = settings.INTERFERENCE if self._interference is None else float(self._interference)
            if rho > 0.0:
                sched = groups_mgwfbp_contended(names, sizes, self._layerwise_times, cost, rho, nbytes,
                                                cost_last=self._cost_model_last)
            else:
                sched = groups_mgwfbp(names, sizes, self._layerwise_times, cost, nbytes)
            if runtime.rank() == 0:
                pr = sched.predicted
                logger.info('tc sum: %f', pr['tc_sum'])
                logger.info('Predicted non-overlapped time: %f', pr['non_overlapped'])
                logger.info('Predicted tb+tc= %f', pr['tb_plus_tc'])
                logger.info('Merged tc sum: %f', pr['merged_tc_sum'])
        else:
            sched = groups_by_threshold(names, sizes, self._threshold)
        self._schedule: MergeSchedule = sched
        if self._late_full and self._layerwise_times is not None and len(self._layerwise_times) == len(names):
            # groups (other than the last) that become ready when less than LATE_GROUP_MS of profiled backward time is left:
            # a group is ready with its earliest layer, and what is left of backward then is the time of the layers before it
            pos = {n: i for i, n in enumerate(names)}
            before = np.concatenate(([0.0], np.cumsum(np.asarray(self._layerwise_times, dtype=np.float64))))
            self._late_groups = frozenset(gi for gi, g in enumerate(sched.groups[:-1])
                                          if before[min(pos[n] for n in g)] < 1e-3 * settings.LATE_GROUP_MS)
        logger.info('# of parameters: %d', int(np.sum(sizes)) if sizes else 0)
        logger.info('Total number of tensors: %s', len(sizes))
        logger.info('Merged Number of groups: %s', len(sched.groups))
        self._groups = sched.groups
        self._key_groupidx_maps = sched.key_groupidx
        self._merged_parameter_offsets = dict(zip(sched.keys, sched.offsets))
        self._group_keys = sched.keys
        # position of each tensor inside its group (O(1) replacement for list.index per hook)
        self._pos_in_group = {name: (gi, li) for gi, g in enumerate(sched.groups) for li, name in enumerate(g)}
        self._group_missing = [len(g) for g in sched.groups]
        self._merged_parameters: Dict[str, torch.Tensor] = {}
        self._merged_parameter_names: Dict[int, str] = {}
        self._one_tensor_per_group = len(sched.groups) == len(names)
        if not self._fused_comm and not self._one_tensor_per_group:
            for key, g, n_el in zip(sched.keys, sched.groups, sched.group_sizes):
                first = self._named_parameters[g[0]]
                buf = torch.zeros(n_el, device=first.device, dtype=first.dtype, requires_grad=False)
                self._merged_parameters[key] = buf
                self._merged_parameter_names[id(buf)] = key

    def _verify_schedule_agreement(self) -> None:
        """Every rank must hold the same schedule: the kernels rely on identical launch order
        instead of Horovod's per-tensor name negotiation."""
        # (the late groups change how many CTAs a group's kernel has, and CTAs of different ranks wait for one another)
        digests = runtime.allgather_object(self._schedule.digest() + '/' + ','.join(map(str, sorted(self._late_groups))))
        if len(set(digests)) != 1:
            raise RuntimeError('ranks disagree on the merge schedule: %s' % digests)

    def benchmark_communication(self, num_iters: int = 10, sizes: Optional[Sequence[int]] = None,
                                rebuild: bool = True) -> Tuple[float, float]:
        """Measure ``alpha, beta`` of the active data plane and optionally rebuild the schedule.

        Counterpart of the reference's never-called ``_benchmark_communication``
        (``distributed_optimizer.py:105-127``); rank 0's fit is broadcast so all ranks agree.
        """
        from ..utils.profiling import CommunicationProfiler
        first = next(iter(self._named_parameters.values()))
        prof = CommunicationProfiler(self._comm.allreduce_async_, self._comm.synchronize, sizes, device=first.device)
        sz, times = prof.benchmark(num_iters=num_iters)
        ab = fit_alpha_beta(sz, times, 4)
        alpha, beta = runtime.broadcast_object((ab.alpha, ab.beta), 0)
        self.alpha, self.beta = float(alpha), float(beta)
        logger.info('[rank:%d] Communication performance fitted with f(p)=a+b*p, where a=%s and b=%s',
                    runtime.rank(), self.alpha, self.beta)
        if rebuild and self._world > 1 and not self._fused_comm:
            self._generate_merged_parameters()
        return self.alpha, self.beta

    # ------------------------------------------------------------------ hooks
    def _register_hooks(self) -> None:
        for group in self.param_groups:
            for p in group['params']:
                if not p.requires_grad:
                    continue
                if p not in self._parameter_names:
                    continue
                self._requires_update.add(p)
                if not self._fused_comm and p.grad is None:
                    p.grad = torch.zeros_like(p, memory_format=torch.contiguous_format)
                self._hook_handles.append(p.register_post_accumulate_grad_hook(self._make_hook(p)))

    def remove_hooks(self) -> None:
        for h in self._hook_handles:
            h.remove()
        self._hook_handles = []

    def close(self) -> None:
        """Retire this wrapper (collective when a fused communicator is attached): hooks are removed, staging memory
        goes back to the communicator, and the optimizer state (momentum buffers created meanwhile) is handed to the
        optimizer it was built from, so that a new wrapper around that optimizer continues where this one stopped."""
        self.remove_hooks()
        if self._active and self._fused_comm and hasattr(self._comm, 'detach'):
            self._comm.detach(self)
        wrapped = getattr(self, '_wrapped', None)
        if wrapped is not None:
            wrapped.state.update(self.state)
        self._active = False

    def check_hooked_tensor_sequence(self, name: str) -> None:
        """With a profiled layer sequence, gradients must arrive last layer first
        (reference ``distributed_optimizer.py:342-354``)."""
        if self._seq_layernames is None:
            return
        n = len(self._seq_layernames)
        idx = self._seq_index[name]
        if idx == n - self._hook_checked_idx - 1:
            self._hook_checked_idx += 1
            if idx == 0:
                self._hook_checked_idx = 0
        else:
            expected = n - self._hook_checked_idx - 1
            self._hook_checked_idx = 0
            raise HookOrderError('gradient of %s (layer %d) arrived where layer %d was expected; '
                                 're-run the layer-wise profiler for this model' % (name, idx, expected))

    def _make_hook(self, p: torch.Tensor) -> Callable:
        name = self._parameter_names[p]
        gi, li = self._pos_in_group[name]

        def hook(param):
            if self.local:
                return
            self.check_hooked_tensor_sequence(name)
            self._synchronized = False
            if self._fused_comm:
                self._group_missing[gi] -= 1
                if self._group_missing[gi] == 0:
                    self._group_missing[gi] = len(self._groups[gi])
                    if self._shadow is not None and self._shadow.active(self.train_iter):
                        self._shadow.snapshot(self, self._groups[gi], getattr(self, '_nvl_first_step', False))
                    self._comm.launch_group(self, gi)
                    self._groups_pending.append(gi)
                return
            tensor = self._push_to_buffer(name, gi, li, param.grad)
            if tensor is not None:
                key = name if self._one_tensor_per_group else self._group_keys[gi]
                assert gi not in self._handles, 'group %d was already sent this iteration' % gi
                self._handles[gi] = (self._allreduce_grad_async(tensor, key), tensor)
        return hook

    def _push_to_buffer(self, name: str, gi: int, li: int, grad: torch.Tensor) -> Optional[torch.Tensor]:
        with torch.no_grad():
            if self._one_tensor_per_group:
                if not grad.is_contiguous():
                    # e.g. channels-last convolution weights: give the parameter a dense
                    # row-major gradient once; later passes accumulate into it in place
                    p = self._named_parameters[name]
                    p.grad = grad.contiguous()
                    grad = p.grad
                return grad.view(-1)
            key = self._group_keys[gi]
            buf = self._merged_parameters[key]
            off = self._merged_parameter_offsets[key][li]
            n = grad.numel()
            slot = buf[off:off + n]
            if grad.data_ptr() != slot.data_ptr():     # after the first iteration p.grad *is* the slot
                slot.copy_(grad.reshape(n))
            self._group_missing[gi] -= 1
            if self._group_missing[gi] > 0:
                return None
            self._group_missing[gi] = len(self._groups[gi])
            return buf

    def _allreduce_grad_async(self, tensor: torch.Tensor, name: str):
        if len(name) > 100:
            name = name[0:50] + '...' + name[50:100]
        return self._comm.allreduce_async_(tensor.view(-1), average=True, name=name)

    # ------------------------------------------------------------------ synchronize / step
    def synchronize(self) -> None:
        """Wait until every group launched during this backward pass has been reduced.

        Afterwards ``p.grad`` holds the averaged gradient of every parameter (when the fused
        data plane is used with ``settings.WRITE_BACK_GRADS`` off and the update fused, the
        gradients have already been consumed and ``p.grad`` keeps the local values).
        """
        if not self._active or self._synchronized:
            return
        if self._fused_comm:
            self._comm.wait_groups(self, self._groups_pending)
            self._groups_pending = []
        else:
            for gi, (handle, tensor) in self._handles.items():
                t0 = time.time()
                out = self._comm.synchronize(handle)
                if self._profiling:
                    self._allreduce_timers.setdefault(self._group_keys[gi], []).append(time.time() - t0)
                if not self._one_tensor_per_group:
                    key = self._group_keys[gi]
                    for name, off in zip(self._groups[gi], self._merged_parameter_offsets[key]):
                        p = self._named_parameters[name]
                        view = tensor[off:off + p.numel()].view(p.shape)
                        if p.grad is None or p.grad.data_ptr() != view.data_ptr():
                            p.grad = view
            self._handles.clear()
            self._print_profiling()
        self._synchronized = True
        self.train_iter += 1

    def step(self, closure=None):
        if self._active and not self.local:
            self.synchronize()
            if self._fused_comm:
                loss = self._comm.finish_step(self, closure)
                if self._shadow is not None:
                    self._shadow.verify(self)
                return loss
        if self._norm_clip is not None and not self.local and getattr(self, '_fast_sgd', None) is None:
            # global L2-norm clip of the averaged gradient (the reference's loop calls
            # clip_grad_norm_ between synchronize() and step(), dist_trainer.py:89-94)
            self._unscale_grads_()
            scale, self._grad_scale = self._grad_scale, 1.0          # already divided out
            try:
                params = [p for g in self.param_groups for p in g['params'] if p.grad is not None]
                torch.nn.utils.clip_grad_norm_(params, self._norm_clip)
                return self._local_step(closure)
            finally:
                self._grad_scale = scale
        return self._local_step(closure)

    def _print_profiling(self) -> None:
        """Log mean wait / update times per merged group once 40 samples exist (enable with
        ``optimizer._profiling = True``; unfused data plane only).  Reference ``:407-425``."""
        ars = self._allreduce_timers
        if not (self._profiling and runtime.rank() == 0 and ars and len(next(iter(ars.values()))) >= 40):
            return
        tar = sum(float(np.mean(v)) for v in ars.values())
        tup = sum(float(np.mean(v)) for v in self._update_times.values()) if self._update_times else 0.0
        logger.info('[%d]: Total compress: %f, allreduce: %f, update: %f, total: %f', runtime.rank(), 0.0, tar, tup, tar + tup)
        self._compression_timers.clear()
        ars.clear()
        self._update_times.clear()

    def sync_hyper(self) -> None:
        """Push the current ``param_groups`` hyper-parameters to the device tables of the fused
        kernels.  Needed only by callers that replay a captured CUDA graph of the training step."""
        if self._active and self._fused_comm:
            self._comm.sync_hyper(self)
        elif getattr(self, '_fast_sgd', None) is not None:
            self._fast_sgd.sync_hyper(self)

    @property
    def local(self) -> bool:
        return self._local

    @local.setter
    def local(self, value: bool) -> None:
        if value and (getattr(self, '_external', None) or getattr(self, '_scatter', None)):
            raise RuntimeError('gradient accumulation (optimizer.local = True) cannot be combined with gathered '
                               'weight-gradient layers; construct the model with MGWFBP_GATHERED_WGRAD=0')
        if value:
            self.release_external_layers()
        self._local = bool(value)

    def release_external_layers(self) -> None:
        """One GPU: layers whose weight-gradient GEMM applies the update in its epilogue go back to ordinary gradients
        plus the multi-tensor update (call before accumulating gradients over several backward passes)."""
        fast = getattr(self, '_fast_sgd', None)
        if fast is not None:
            fast.release_external(self)

    def set_grad_scale(self, scale: float) -> None:
        """Gradients arrive multiplied by ``1 / scale`` (a static loss scale): every update path divides it out --
        inside the fused all-reduce kernel and the multi-tensor SGD kernel, by one ``_foreach_mul_`` elsewhere."""
        if not scale > 0.0:
            raise ValueError('gradient scale must be positive')
        self._grad_scale = float(scale)

    def _unscale_grads_(self) -> None:
        grads = [p.grad for g in self.param_groups for p in g['params'] if p.grad is not None]
        if grads and self._grad_scale != 1.0:
            torch._foreach_mul_(grads, self._grad_scale)

    def _local_step(self, closure=None):
        fast = getattr(self, '_fast_sgd', None)
        if fast is not None and closure is None:
            if self._norm_clip is not None and self._grad_scale != 1.0:
                self._unscale_grads_()           # the clip needs the norm of the true gradient
                return fast.step(self)
            return fast.step(self, grad_scale=self._grad_scale)
        self._unscale_grads_()
        return self._base_cls.step(self, closure)

    def zero_grad(self, set_to_none: Optional[bool] = None):
        """Clear gradients.

        With the unfused data plane ``p.grad`` aliases the merged buffers after the first
        iteration, so gradients are zeroed in place (one fill per buffer).  With the fused data
        plane gradients are dropped (autograd hands over fresh tensors, whose addresses the
        kernels pick up from a pointer table).
        """
        if self._active and not self._fused_comm and not set_to_none:
            if self._merged_parameters:
                for buf in self._merged_parameters.values():
                    buf.zero_()
                for p in self._requires_update:
                    if p.grad is not None and not self._aliases_buffer(p):
                        p.grad.zero_()
            else:
                for p in self._requires_update:
                    if p.grad is not None:
                        p.grad.zero_()
            return
        if set_to_none is None:
            set_to_none = True
        return self._base_cls.zero_grad(self, set_to_none=set_to_none)

    def _aliases_buffer(self, p: torch.Tensor) -> bool:
        name = self._parameter_names.get(p)
        if name is None:
            return False
        gi, li = self._pos_in_group[name]
        key = self._group_keys[gi]
        buf = self._merged_parameters.get(key)
        if buf is None:
            return False
        off = self._merged_parameter_offsets[key][li]
        return p.grad.data_ptr() == buf.data_ptr() + off * buf.element_size()

    # ------------------------------------------------------------------ introspection
    @property
    def merge_schedule(self) -> MergeSchedule:
        return self._schedule

    @property
    def communicator(self) -> Communicator:
        return self._comm


def DistributedOptimizer(optimizer, named_parameters=None, compression=None, density=0.001, seq_layernames=None,
                         layerwise_times=None, norm_clip=None, threshold=0, writer=None, gradient_path=None,
                         comm: Optional[Communicator] = None, cost_model=None, fused_update: Optional[bool] = None,
                         interference: Optional[float] = None, cost_model_last=None, schedule: Optional[MergeSchedule] = None,
                         late_full: bool = False):
    """Wrap ``optimizer`` so that gradients are averaged across workers before each update.

    Signature and merge policies follow reference ``distributed_optimizer.py:435-471``:

    * ``threshold`` -- element-count bucketing (0: one message per tensor; huge: one message);
    * ``seq_layernames`` + ``layerwise_times`` (with ``settings.ADAPTIVE_MERGE``) -- MG-WFBP;
    * ``norm_clip`` -- honoured here (the reference accepts and then drops it, ``:471``): the
      global L2 norm of the averaged gradient is clipped before the update;
    * ``compression`` / ``density`` -- accepted for call compatibility; only the identity
      compressor exists, as in the reference (``compression.py:5-19``).

    Extra keyword arguments select the data plane (``comm``), the all-reduce cost model
    (``cost_model``; default: measured alpha/beta if available, else the table for
    ``settings.CONNECTION``), whether the update is fused into the all-reduce kernels, and -- for the
    fused NVLink data plane -- how much a second of communication kernel running beside backward slows
    backward down (``interference``, see ``engine.fit_interference``; default ``settings.INTERFERENCE``)
    and the cost model of the schedule's last message, which runs with the whole GPU (``cost_model_last``).
    ``schedule`` installs a given :class:`MergeSchedule` (or the result of calling it with the scheduled names, sizes and
    layer-wise backward times) instead of deriving one.  ``late_full`` gives groups that become ready within
    ``settings.LATE_GROUP_MS`` of the end of backward the CTA count of a message that has the GPU to itself.

    Example of gradient clipping::

        loss.backward()
        optimizer.synchronize()
        torch.nn.utils.clip_grad_norm_(model.parameters(), clip)
        optimizer.step()
    """
    base_cls = optimizer.__class__
    cls = type(base_cls.__name__, (_DistributedMixin, base_cls), {'_base_cls': base_cls})
    obj = cls.__new__(cls)
    # Re-run the wrapped class's constructor on the existing param_groups: every group already
    # carries its full hyper-parameter set, so the positional defaults are irrelevant.
    base_cls.__init__(obj, optimizer.param_groups)
    obj.defaults = dict(optimizer.defaults)
    obj.state.update(optimizer.state)
    obj._dist_init(optimizer, named_parameters, compression, seq_layernames, layerwise_times, norm_clip,
                   threshold, writer, gradient_path, comm, cost_model, fused_update, interference, cost_model_last, schedule,
                   late_full)
    if not obj._active and obj._base_is_sgd:
        first = next(iter(obj._named_parameters.values()), None)
        if first is not None and first.is_cuda:
            from ..ops.sgd import FastSGD
            obj._fast_sgd = FastSGD.try_create(obj, norm_clip=norm_clip)
    return obj
