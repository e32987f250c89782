# -*- coding: utf-8 -*-
"""``NvlComm``: the NVLink / NVSwitch data plane with the fused all-reduce + SGD kernels.

Replaces what Horovod's C++ core does for the reference (coordinator thread, name negotiation,
tensor queue, NCCL launch; see ``distributed_optimizer.py:21-26,339,375``) with:

* a **symmetric arena** (``heap.py``, ``csrc/symm_heap.cu``): ``cuMemCreate`` memory per rank, mapped into
  every peer and -- behind an NVSwitch -- bound to a multicast object; file descriptors are exchanged
  once over Unix sockets, everything else over the gloo control plane.  Flag rows, staging areas,
  gathered activation rows and scratch space are blocks of that one arena;
* **flag rows** for CTA-to-CTA barriers between ranks (bounded waits);
* one **kernel launch per merged group** on a high-priority side stream
  (``csrc/allreduce_fused.cu``): pack through a pointer table, reduce over peer memory (one-shot,
  two-shot, or NVLS ``multimem.ld_reduce`` / ``multimem.st`` through the switch), average, and -- for
  plain SGD -- update the weights in the same pass.  Groups whose kernel runs beside backward get a
  small number of CTAs (``MGWFBP_OVERLAP_CTAS``); only the schedule's last group, which nothing can
  hide, uses the whole GPU;
* no negotiation: every rank launches groups in the order their gradients complete, which is the
  same on every rank because the schedule digest was compared at construction.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ... import settings
from ...ops import _lib, counters
from ...ops.tables import GroupTable, HyperTable, ensure_momentum_buffers, param_group_index
from ...settings import logger
from .. import runtime
from .base import CommTimeoutError, Communicator
from .heap import Block, SymmArena

_ALIGN = 256


def _env_int(name: str, default: int) -> int:
    try:
        return int(os.environ.get(name, default))
    except ValueError:
        return default


def _wrap_device_memory(ptr: int, n_floats: int, device: torch.device) -> torch.Tensor:
    """A float32 tensor view of raw device memory that this module owns (symmetric heap)."""
    class _Mem:
        pass
    holder = _Mem()
    holder.__cuda_array_interface__ = {'shape': (int(n_floats),), 'typestr': '<f4', 'data': (int(ptr), False), 'version': 2}
    return torch.as_tensor(holder, device=device)


class _GroupPlan:
    __slots__ = ('table', 'params', 'algo', 'n_ctas', 'stage_off', 'args', 'partials_off', 'block', 'overlapped', 'mode',
                 'copy_pack', 'stage_views')



class NvlComm(Communicator):
    fused = True
    _shared: Optional['NvlComm'] = None

    # ------------------------------------------------------------------ construction
    def __init__(self):
        if not torch.cuda.is_available():
            raise RuntimeError('NvlComm needs a CUDA device')
        self.lib = _lib.load(allow_build=False)
        self._rank, self._world = runtime.rank(), runtime.size()
        self.device = torch.device('cuda', torch.cuda.current_device())
        self._side_stream = torch.cuda.Stream(device=self.device, priority=-1)
        self._on_main = os.environ.get('MGWFBP_COMM_STREAM', 'side').strip().lower() == 'main'
        self.timeout_ns = int(float(os.environ.get('MGWFBP_COMM_TIMEOUT_S', '10')) * 1e9)
        self.oneshot_max_bytes = _env_int('MGWFBP_ONESHOT_MAX_BYTES', 512 * 1024)
        self.max_ctas_oneshot = min(_env_int('MGWFBP_ONESHOT_CTAS', 8), _lib.MAX_CTAS)
        self.max_ctas_twoshot = min(_env_int('MGWFBP_TWOSHOT_CTAS', 128), _lib.MAX_CTAS)
        # groups whose kernel runs beside backward get few CTAs: what such a kernel costs is the SM time it holds
        # (including the time its CTAs spin while a peer is late), not its latency
        self.overlap_ctas = max(1, min(_env_int('MGWFBP_OVERLAP_CTAS', 16), _lib.MAX_CTAS))
        # the switch-side reduction pays from this many ranks on (with two ranks a pull is as cheap as a multimem load)
        self.nvls_min_world = _env_int('MGWFBP_NVLS_MIN_WORLD', 4)
        # How the gradients of a group that overlaps backward reach its staging area: 'kernel' = the kernel's own pack
        # loop (default), 'copy' = one device-to-device copy per tensor queued in front of the kernel.  Measured on B200
        # the copies lose: the driver serves the many small ones with copy kernels of 1.5-2 us each, one after the other,
        # which pushes the group's kernel to the end of backward.  The schedule's last group always packs in the kernel.
        self.pack_mode = os.environ.get('MGWFBP_PACK', 'kernel').strip().lower()
        self.n_threads = _env_int('MGWFBP_COMM_THREADS', 512)
        # two-shot / NVLS kernels work through a CTA's chunk in pieces (pack, reduce and update of successive pieces
        # of different CTAs overlap); large messages use narrower CTAs, two of which fit on an SM
        self.max_pieces = max(1, _env_int('MGWFBP_PIECES', 1))
        self.piece_slots = max(1, _env_int('MGWFBP_PIECE_SLOTS', 4096))
        self.big_threads = _env_int('MGWFBP_BIG_THREADS', 512)
        self.big_bytes = _env_int('MGWFBP_BIG_BYTES', 8 << 20)
        # control block: flag rows + per-CTA launch counters, in a heap of its own
        self._flag_bytes = int(self.lib.mgw_flag_block_bytes())
        self.arena = SymmArena(self.lib)
        ctl_bytes = 3 * (self._flag_bytes + 4 * _lib.MAX_CTAS + 2 * _ALIGN)
        self._ctl: Block = self.arena.alloc(ctl_bytes)               # first block of a fresh (zeroed) heap
        top = [0]

        def carve(n):
            off = top[0]
            top[0] = (off + n + _ALIGN - 1) // _ALIGN * _ALIGN
            return off
        self._flag_off = carve(self._flag_bytes)
        self._epoch_off = carve(4 * _lib.MAX_CTAS)
        self._gflag_off = carve(self._flag_bytes)          # flag rows / counters of the row all-gather
        self._gepoch_off = carve(4 * _lib.MAX_CTAS)
        self._rflag_off = carve(self._flag_bytes)          # ... and of the reduce-scatter weight gradients
        self._repoch_off = carve(4 * _lib.MAX_CTAS)
        assert top[0] <= ctl_bytes
        self._gather_tables = None
        status = C.POINTER(C.c_int)()
        _lib.check(self.lib.mgw_host_status_alloc(8, C.byref(status)), 'status_alloc')
        self._status = status
        self._blocks: Dict[int, List[Block]] = {}      # id(optimizer) -> blocks to give back on detach
        self._scratch = None            # block + capacities for allreduce_async_
        self._scratch_tables: Dict[Tuple[int, int], GroupTable] = {}
        self._scratch_geometry = None
        self._done_event = torch.cuda.Event()
        self._plans: Dict[int, List[_GroupPlan]] = {}
        self._hyper: Dict[int, HyperTable] = {}
        self._keepalive: List[object] = []
        self.launches = 0
        if self._world > 1 and os.environ.get('MGWFBP_BN_RESERVE', '1').strip().lower() not in ('0', 'false', 'no', 'off'):
            # the memory-bound kernels of the model are sized as one resident wave: leave the SMs that an overlapped
            # communication kernel may hold out of that wave (see ops.bn_relu.set_sm_budget)
            from ...ops.bn_relu import set_sm_budget
            sms = torch.cuda.get_device_properties(self.device).multi_processor_count
            set_sm_budget(max(sms // 2, sms - self.overlap_ctas))

    @property
    def stream(self) -> torch.cuda.Stream:
        """Where communication kernels are launched: a high-priority side stream of their own, so that they run beside
        backward; with ``MGWFBP_COMM_STREAM=main`` the stream that is current at the call, which gives up the overlap and
        keeps a captured training step a single chain of kernels."""
        return torch.cuda.current_stream(self.device) if self._on_main else self._side_stream

    @property
    def nvls_available(self) -> bool:
        """True when the symmetric heap is bound to an NVSwitch multicast object (``multimem`` instructions work)."""
        return self.arena.has_multicast

    @classmethod
    def shared(cls) -> 'NvlComm':
        if cls._shared is None:
            cls._shared = cls()
        return cls._shared

    def size(self) -> int:
        return self._world

    def rank(self) -> int:
        return self._rank

    def close(self) -> None:
        torch.cuda.synchronize()
        self.arena.close()
        self._blocks, self._plans, self._hyper, self._scratch = {}, {}, {}, None
        if self._status:
            self.lib.mgw_host_status_free(self._status)
            self._status = None
        if NvlComm._shared is self:
            NvlComm._shared = None

    # ------------------------------------------------------------------ status
    def status(self) -> Tuple[int, int, int, int, int]:
        s = self._status
        if not s:                                   # closed
            return (0, 0, 0, 0, 0)
        return (s[0], s[1], s[2], s[3], s[4])

    def check_status(self, synchronize: bool = False) -> None:
        """Raise :class:`CommTimeoutError` if a kernel gave up waiting for a peer."""
        if synchronize:
            torch.cuda.synchronize()
        code, peer, expected, observed, cta = self.status()
        if code != 0:
            raise CommTimeoutError('communication kernel on rank %d gave up (code %d): waited for rank %d, '
                                   'expected launch %d, saw %d (CTA %d)' % (self._rank, code, peer, expected, observed, cta))

    def clear_status(self) -> None:
        for i in range(8):
            self._status[i] = 0

    # ------------------------------------------------------------------ planning
    def big_algo(self) -> int:
        """The algorithm for messages beyond the one-shot range."""
        if self.nvls_available and self._world >= self.nvls_min_world:
            return _lib.ALGO_NVLS
        return _lib.ALGO_TWOSHOT

    def choose(self, n_vec: int, overlapped: bool = False) -> Tuple[int, int]:
        """Algorithm and CTA count for a message of ``n_vec`` float4 slots (same answer on every rank).
        ``overlapped``: the kernel will run beside backward, so it is given at most ``overlap_ctas`` CTAs."""
        nbytes = n_vec * 16
        forced = settings.COMM_ALGO.lower()
        if forced in _lib.ALGO_NAMES and not (forced == 'nvls' and not self.nvls_available):
            algo = _lib.ALGO_NAMES[forced]
        elif nbytes <= self.oneshot_max_bytes:
            algo = _lib.ALGO_ONESHOT
        else:
            algo = self.big_algo()
        # a CTA is worth launching for two (one-shot) / eight (two-shot) float4 slots per thread
        if algo == _lib.ALGO_ONESHOT:
            per_cta = 2 * self.n_threads
            n_ctas = max(1, min(self.max_ctas_oneshot, (n_vec + per_cta - 1) // per_cta))
        else:
            per_cta = 8 * self._threads_for(algo, n_vec)
            cap = min(self.max_ctas_twoshot, self.overlap_ctas) if overlapped else self.max_ctas_twoshot
            n_ctas = max(1, min(cap, (n_vec + per_cta - 1) // per_cta))
        return algo, n_ctas

    def _threads_for(self, algo: int, n_vec: int) -> int:
        if algo != _lib.ALGO_ONESHOT and 16 * n_vec >= self.big_bytes:
            return self.big_threads
        return self.n_threads

    def _fill_args(self, plan: _GroupPlan, block: Block, hyper_ptr: int, partials_ptr: int,
                   inbox_stride: Optional[int] = None, stage_slots: Optional[int] = None) -> None:
        a = _lib.MgwAllreduceArgs()
        a.group = plan.table.struct
        for r in range(self._world):
            a.stage[r] = block.peer(r) + plan.stage_off
            a.flags[r] = self._ctl.peer(r) + self._flag_off
        a.epoch = self._ctl.base + self._epoch_off
        a.mc_stage = (block.mc + plan.stage_off) if block.mc else None
        a.hyper = hyper_ptr or None
        a.sumsq_partials = partials_ptr or None
        a.status = C.cast(self._status, C.c_void_p).value
        a.rank, a.world = self._rank, self._world
        a.algo, a.n_ctas, a.n_threads = plan.algo, plan.n_ctas, self._threads_for(plan.algo, plan.table.n_vec)
        a.max_pieces, a.piece_slots = self.max_pieces, self.piece_slots
        a.grad_scale = 1.0
        a.mode, a.first_step = 0, 0
        a.inbox_stride = plan.table.n_vec if inbox_stride is None else inbox_stride
        a.stage_slots = plan.table.n_vec if stage_slots is None else stage_slots
        a.timeout_ns = self.timeout_ns
        plan.args = a

    def attach(self, opt) -> None:
        """Lay out staging memory and descriptor tables for every group of ``opt``'s schedule."""
        key = id(opt)
        named = opt._named_parameters
        momenta_created = False
        plans: List[_GroupPlan] = []
        total = 0
        sizes = []
        n_groups = len(opt._groups)
        late = getattr(opt, '_late_groups', frozenset())      # ready so close to the end of backward that they count as last
        for gi, names in enumerate(opt._groups):
            params = [named[n] for n in names]
            n_vec = sum((p.numel() + 3) // 4 for p in params)
            # every group but the last one of the schedule is launched while backward still runs
            algo, n_ctas = self.choose(n_vec, overlapped=gi < n_groups - 1 and gi not in late)
            nbytes = int(self.lib.mgw_stage_bytes(algo, n_vec, self._world))
            sizes.append((algo, n_ctas, nbytes))
            total += (nbytes + _ALIGN - 1) // _ALIGN * _ALIGN
        block = self.arena.alloc(total + _ALIGN)
        self._blocks.setdefault(key, []).append(block)
        stage_top = 0
        hyper = HyperTable(self.device)
        self._hyper[key] = hyper
        n_partials = sum(s[1] for s in sizes)
        # one sum of squares per CTA of every group kernel, plus (clipping only) those of the weights whose gradient
        # arrives through the reduce-scatter GEMM: their norm is taken by one extra kernel in finish_step
        scatter = list(getattr(opt, '_scatter', []))
        opt._rs_sumsq_ctas = 64 if (scatter and opt._norm_clip is not None) else 0
        opt._rs_partials_off = n_partials
        partials = torch.zeros(max(n_partials + opt._rs_sumsq_ctas, 1), dtype=torch.float32, device=self.device)
        clip_out = torch.ones(2, dtype=torch.float32, device=self.device)
        opt._nvl_partials, opt._nvl_clip_out = partials, clip_out
        p_off = 0
        for names, (algo, n_ctas, nbytes) in zip(opt._groups, sizes):
            params = [named[n] for n in names]
            if opt._base_is_sgd:
                momenta, created = ensure_momentum_buffers(opt, params)
                momenta_created = momenta_created or created
                pgi = param_group_index(opt, params)
            else:
                momenta, pgi = [None] * len(params), [0] * len(params)
            plan = _GroupPlan()
            plan.params = params
            plan.table = GroupTable(params, pgi, momenta, self.device)
            plan.algo, plan.n_ctas = algo, n_ctas
            plan.stage_off = stage_top
            stage_top += (nbytes + _ALIGN - 1) // _ALIGN * _ALIGN
            plan.partials_off = p_off
            plan.block = block
            plan.overlapped = len(plans) < n_groups - 1 and len(plans) not in late
            plan.copy_pack = bool(self.pack_mode == 'copy' and plan.overlapped and algo != _lib.ALGO_ONESHOT)
            plan.stage_views = None
            self._fill_args(plan, block, hyper.data_ptr(), partials.data_ptr() + 4 * p_off)
            p_off += n_ctas
            plans.append(plan)
        self._plans[key] = plans
        if any(pl.copy_pack for pl in plans):
            self.arena.zero(block)        # pad lanes between tensors are never written by the copies: they must hold zeros
        opt._nvl_first_step = momenta_created
        opt._nvl_all = None
        if opt._base_is_sgd:
            gathered = {id(p) for _n, p, _m in getattr(opt, '_external', [])}      # updated by their own GEMM epilogue
            allp = [p for g in opt.param_groups for p in g['params'] if p.requires_grad and id(p) not in gathered]
            mom, _ = ensure_momentum_buffers(opt, allp)
            opt._nvl_all = GroupTable(allp, param_group_index(opt, allp), mom, self.device)
        mode = 0
        if opt._fused_update:
            mode |= _lib.MODE_UPDATE
            if settings.WRITE_BACK_GRADS:          # off by default: the update consumed the gradient, nobody reads it again
                mode |= _lib.MODE_WRITEBACK
        else:
            mode |= _lib.MODE_WRITEBACK
            if opt._norm_clip is not None:
                mode |= _lib.MODE_SUMSQ
        opt._nvl_mode = mode
        # Deferred update: the two-shot / NVLS kernels leave the averaged gradient in their staging area (mode 0: no
        # pass over parameters, momenta or gradient tensors while backward runs) and ONE multi-tensor SGD kernel reads
        # it there after backward.  One-shot groups (small) sum their inbox rows into p.grad as usual.
        deferred = bool(getattr(opt, '_deferred_update', False)) and opt._base_is_sgd and opt._norm_clip is None
        opt._nvl_deferred_ptrs = None
        for plan in plans:
            plan.mode = mode
            if deferred:
                plan.mode = _lib.MODE_WRITEBACK if plan.algo == _lib.ALGO_ONESHOT else 0
        if deferred:
            where = {}
            for plan in plans:
                for ti, p in enumerate(plan.params):
                    where[id(p)] = None if plan.algo == _lib.ALGO_ONESHOT else \
                        plan.block.base + plan.stage_off + 16 * int(plan.table.voff_host[ti])
            opt._nvl_deferred_ptrs = [where.get(id(p)) for p in opt._nvl_all.params]
        opt._nvl_held = []
        if getattr(opt, '_external', None):
            self._attach_external(opt)
        if scatter:
            self._attach_scatter(opt)
        algos = {0: 0, 1: 0, 2: 0}
        for pl in plans:
            algos[pl.algo] += 1
        logger.info('NvlComm: %d groups (%d one-shot, %d two-shot, %d nvls), %.1f MB staging, fused update: %s',
                    len(plans), algos[0], algos[1], algos[2], total / 1e6, opt._fused_update)

    def detach(self, opt) -> None:
        """Forget ``opt`` (collective): its staging blocks go back to the arena once no rank uses them any more."""
        key = id(opt)
        if key not in self._plans and key not in self._blocks:
            return
        torch.cuda.synchronize()
        runtime.barrier()
        for block in self._blocks.pop(key, []):
            self.arena.free(block)
        self._plans.pop(key, None)
        self._hyper.pop(key, None)
        for st in getattr(opt, '_ext_state', {}).values():
            st['bufs'] = None
        for _name, _p, module in getattr(opt, '_external', []):
            module._exchange = None                 # the layer behaves like nn.Linear again
        for _name, p in getattr(opt, '_scatter', []):
            p._mgw_rs_sink = None
        opt._rs_state = {}

    # ------------------------------------------------------------------ hot path
    def launch_group(self, opt, gi: int) -> None:
        plan = self._plans[id(opt)][gi]
        grads = [p.grad for p in plan.params]
        for g, p in zip(grads, plan.params):
            if g.stride() != p.stride():
                raise RuntimeError('gradient layout differs from parameter layout; fused kernels need them equal')
        compute = torch.cuda.current_stream()
        ready = torch.cuda.Event()
        ready.record(compute)
        self.stream.wait_event(ready)
        if plan.copy_pack:
            self._copy_pack(plan, grads)
        else:
            plan.table.refresh_grads(grads, self.stream)
        if not opt._groups_pending and not torch.cuda.is_current_stream_capturing():
            # first group of this iteration: hyper-parameters may have moved (inside a graph capture the
            # table is refreshed by the caller before every replay instead)
            self._hyper[id(opt)].sync(opt.param_groups, self.stream)
        a = plan.args
        a.mode = plan.mode
        a.skip_pack = int(plan.copy_pack)
        a.first_step = int(opt._nvl_first_step)
        a.grad_scale = float(getattr(opt, '_grad_scale', 1.0))
        _lib.check(self.lib.mgw_allreduce_group(C.byref(a), self.stream.cuda_stream), 'allreduce_group')
        opt._nvl_held.append(grads)
        self.launches += 1
        counters.bump('allreduce_fused')

    def _copy_pack(self, plan: _GroupPlan, grads) -> None:
        """Queue one device-to-device copy per gradient tensor into the group's staging area (side stream)."""
        if plan.stage_views is None:
            base = plan.block.base + plan.stage_off
            views = []
            for ti, p in enumerate(plan.params):
                flat = _wrap_device_memory(base + 16 * int(plan.table.voff_host[ti]), p.numel(), self.device)
                views.append(torch.as_strided(flat, p.size(), p.stride()))      # same layout as the gradient: a plain memcpy
            plan.stage_views = views
        with torch.cuda.stream(self.stream):
            for dst, g in zip(plan.stage_views, grads):
                dst.copy_(g, non_blocking=True)

    def wait_groups(self, opt, pending: Sequence[int]) -> None:
        self._done_event.record(self.stream)
        torch.cuda.current_stream().wait_event(self._done_event)
        opt._nvl_held = []
        if opt._fused_update:
            opt._nvl_first_step = False
        self.check_status()

    def finish_step(self, opt, closure=None):
        loss = closure() if closure is not None else None
        if opt._fused_update:
            if getattr(opt, '_scatter', None):
                # every other weight was updated inside its group's kernel; these got an averaged gradient from the
                # reduce-scatter GEMM and take one multi-tensor SGD launch of their own
                table: GroupTable = opt._rs_table
                table.refresh_grads([p.grad for p in table.params])
                if not torch.cuda.is_current_stream_capturing():
                    self._hyper[id(opt)].sync(opt.param_groups)
                n_ctas = max(1, min(296, (table.n_vec + 2047) // 2048))
                _lib.check(self.lib.mgw_multi_tensor_sgd(C.byref(table.struct), self._hyper[id(opt)].data_ptr(), None, 1.0,
                                                         int(opt._rs_first), _lib.MODE_UPDATE, None, n_ctas,
                                                         torch.cuda.current_stream().cuda_stream), 'multi_tensor_sgd')
                opt._rs_first = False
                self.launches += 1
                counters.bump('multi_tensor_sgd')
            return loss
        if opt._base_is_sgd and opt._nvl_all is not None:
            table: GroupTable = opt._nvl_all
            grads = [p.grad for p in table.params]
            if all(g is not None and g.stride() == p.stride() for g, p in zip(grads, table.params)):
                staged = opt._nvl_deferred_ptrs
                if staged is not None:
                    # averaged gradients wait in the staging areas (already scaled); the rest was summed into p.grad
                    table.refresh_grad_ptrs([s if s is not None else g.data_ptr() for s, g in zip(staged, grads)])
                else:
                    table.refresh_grads(grads)
                if not torch.cuda.is_current_stream_capturing():
                    self._hyper[id(opt)].sync(opt.param_groups)
                s = torch.cuda.current_stream().cuda_stream
                clip_ptr = None
                if opt._norm_clip is not None:
                    part = opt._nvl_partials
                    if opt._rs_sumsq_ctas:
                        rs: GroupTable = opt._rs_table
                        rs.refresh_grads([p.grad for p in rs.params])
                        _lib.check(self.lib.mgw_group_sumsq(C.byref(rs.struct), part.data_ptr() + 4 * opt._rs_partials_off,
                                                            opt._rs_sumsq_ctas, s), 'group_sumsq')
                        counters.bump('group_sumsq')
                    _lib.check(self.lib.mgw_clip_coef(part.data_ptr(), part.numel(), float(opt._norm_clip),
                                                      opt._nvl_clip_out.data_ptr(), s), 'clip_coef')
                    clip_ptr = opt._nvl_clip_out.data_ptr() + 4
                    counters.bump('clip_coef')
                n_ctas = max(1, min(296, (table.n_vec + 2047) // 2048))
                _lib.check(self.lib.mgw_multi_tensor_sgd(C.byref(table.struct), self._hyper[id(opt)].data_ptr(), clip_ptr,
                                                         1.0, int(opt._nvl_first_step), _lib.MODE_UPDATE, None, n_ctas, s),
                           'multi_tensor_sgd')
                opt._nvl_first_step = False
                self.launches += 1
                counters.bump('multi_tensor_sgd')
                return loss
        if opt._norm_clip is not None:
            torch.nn.utils.clip_grad_norm_([p for p in opt._requires_update], opt._norm_clip)
        opt._base_cls.step(opt)
        return loss

    # ------------------------------------------------------------------ gathered weight gradients
    def _attach_external(self, opt) -> None:
        """Wire the layers whose weights are updated from gathered activations (opt._external)."""
        opt._ext_state = {}
        for name, p, module in opt._external:
            mom, created = ensure_momentum_buffers(opt, [p])
            opt._ext_state[id(module)] = dict(name=name, param=p, mom=mom[0], pg=param_group_index(opt, [p])[0],
                                              first=created, bufs=None, opt_key=id(opt))
            module._exchange = (lambda m, dy, x, _o=opt: self.exchange_external(_o, m, dy, x))

    # ------------------------------------------------------------------ reduce-scatter weight gradients
    def _attach_scatter(self, opt) -> None:
        """Staging slots, symmetric gradient tensors and sinks for the weights in ``opt._scatter``: their gradient GEMM stores
        every tile into the owner rank's slot, owners add the slots up and broadcast the sums (csrc/wgrad_gemm_sm100.cu)."""
        from ...ops import wgrad
        lib = wgrad._lib_ready()
        w = self._world
        opt._rs_state = {}
        flags = torch.tensor([self._ctl.peer(r) + self._rflag_off for r in range(w)], dtype=torch.int64, device=self.device)
        for name, p in opt._scatter:
            m, n = p.shape
            stage_bytes = 4 * int(lib.mgw_wgrad_scatter_stage_floats(m, n, w))
            sblock, gblock = self.arena.alloc(stage_bytes), self.arena.alloc(4 * m * n)
            self._blocks.setdefault(id(opt), []).extend([sblock, gblock])
            tab = lambda blk: torch.tensor([blk.peer(r) for r in range(w)], dtype=torch.int64, device=self.device)   # noqa: E731
            grad = _wrap_device_memory(gblock.base, m * n, self.device).view(m, n)
            opt._rs_state[id(p)] = dict(name=name, param=p, m=m, n=n, tab_stage=tab(sblock), tab_grad=tab(gblock), flags=flags,
                                        grad=grad, n_ctas=max(1, min(_env_int('MGWFBP_SCATTER_CTAS', 128), (m * n) // (128 * 128 * w))))
            p._mgw_rs_sink = (lambda dy, x, _o=opt, _p=p: self.scatter_wgrad(_o, _p, dy, x))
        params = [p for _n, p in opt._scatter]
        if opt._base_is_sgd:
            mom, created = ensure_momentum_buffers(opt, params)
            opt._rs_table = GroupTable(params, param_group_index(opt, params), mom, self.device)
            opt._rs_first = created
        else:
            opt._rs_table = GroupTable(params, [0] * len(params), [None] * len(params), self.device)
            opt._rs_first = False

    def scatter_wgrad(self, opt, p, dy: torch.Tensor, x: torch.Tensor) -> None:
        """Called from backward where a weight gradient ``dy^T x`` is due: tensor-core GEMM whose epilogue scatters the
        tiles to their owner ranks, then the owners' sums broadcast into every rank's gradient tensor; ``p.grad`` is that
        tensor (symmetric memory) afterwards.  Runs on the side stream behind what produced ``dy`` and ``x``."""
        from ...ops import wgrad
        lib = wgrad._lib_ready()
        st = opt._rs_state[id(p)]
        w, r = self._world, self._rank
        k = dy.shape[0]
        compute = torch.cuda.current_stream()
        ready = torch.cuda.Event()
        ready.record(compute)
        self.stream.wait_event(ready)
        s = self.stream.cuda_stream
        scale = float(getattr(opt, '_grad_scale', 1.0)) / w
        _lib.check(lib.mgw_wgrad_gemm_scatter(dy.data_ptr(), x.data_ptr(), st['m'], st['n'], k, scale, st['tab_stage'].data_ptr(), r, w,
                                              wgrad._status(dy.device).data_ptr(), s), 'wgrad_gemm_scatter')
        _lib.check(lib.mgw_wgrad_reduce_finish(st['tab_stage'].data_ptr(), st['tab_grad'].data_ptr(), st['flags'].data_ptr(),
                                               self._ctl.base + self._repoch_off, C.cast(self._status, C.c_void_p).value, r, w,
                                               st['m'], st['n'], st['n_ctas'], self.timeout_ns, s), 'wgrad_reduce_finish')
        counters.bump('wgrad_gemm_sm100')
        counters.bump('wgrad_reduce_finish')
        p.grad = st['grad']
        opt._nvl_held.append((dy, x))
        opt._synchronized = False
        self.launches += 2

    def _gather_buffers(self, st, rows: int, m: int, n: int):
        """Symmetric [W*rows, m] and [W*rows, n] buffers of one layer (collective on first use)."""
        if st['bufs'] is not None and st['bufs']['rows'] == rows:
            return st['bufs']
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError('gathered weight-gradient buffers must exist before CUDA graph capture (run eager steps first)')
        w = self._world
        nbytes = 4 * w * rows * (m + n)
        block = self.arena.alloc(nbytes + 2 * _ALIGN)
        self._blocks.setdefault(st['opt_key'], []).append(block)
        off_dy = 0
        off_x = (4 * w * rows * m + _ALIGN - 1) // _ALIGN * _ALIGN

        def ptr_table(off):
            return torch.tensor([block.peer(r) + off for r in range(w)], dtype=torch.int64, device=self.device)
        flags = torch.tensor([self._ctl.peer(r) + self._gflag_off for r in range(w)], dtype=torch.int64, device=self.device)
        st['bufs'] = dict(rows=rows, block=block, off_dy=off_dy, off_x=off_x, tab_dy=ptr_table(off_dy), tab_x=ptr_table(off_x),
                          flags=flags, dy_all=block.base + off_dy, x_all=block.base + off_x)
        return st['bufs']

    def exchange_external(self, opt, module, dy: torch.Tensor, x: torch.Tensor) -> None:
        """Called from the layer's backward: all-gather (dy, x) rows over NVLink, then one tensor-core
        GEMM whose epilogue applies the averaged gradient to the layer's weight and momentum."""
        from ...ops import wgrad
        st = opt._ext_state[id(module)]
        rows, m = dy.shape
        n = x.shape[1]
        w, r = self._world, self._rank
        bufs = self._gather_buffers(st, rows, m, n)
        lib = wgrad._lib_ready()
        compute = torch.cuda.current_stream()
        ready = torch.cuda.Event()
        ready.record(compute)
        self.stream.wait_event(ready)
        if not opt._groups_pending and not torch.cuda.is_current_stream_capturing():
            self._hyper[id(opt)].sync(opt.param_groups, self.stream)
        s = self.stream.cuda_stream
        status = C.cast(self._status, C.c_void_p).value
        epoch = self._ctl.base + self._gepoch_off
        with torch.cuda.stream(self.stream):
            for src, base, cols, tab in ((dy, bufs['dy_all'], m, bufs['tab_dy']), (x, bufs['x_all'], n, bufs['tab_x'])):
                block = rows * cols
                dst = _wrap_device_memory(base + 4 * r * block, block, self.device)
                dst.copy_(src.reshape(-1), non_blocking=True)
                n_ctas = max(1, min(16, block // 16384))
                _lib.check(lib.mgw_allgather_rows(tab.data_ptr(), bufs['flags'].data_ptr(), epoch, status, r, w, block, n_ctas,
                                                  self.timeout_ns, s), 'allgather_rows')
                counters.bump('allgather_rows')
            dy_all = _wrap_device_memory(bufs['dy_all'], w * rows * m, self.device).view(w * rows, m)
            x_all = _wrap_device_memory(bufs['x_all'], w * rows * n, self.device).view(w * rows, n)
            grad_out = None
            if settings.WRITE_BACK_GRADS:
                p = st['param']
                if p.grad is None or p.grad.shape != p.shape:
                    p.grad = torch.empty_like(p)
                grad_out = p.grad
            wgrad.wgrad_sgd_(dy_all, x_all, st['param'].data, st['mom'], self._hyper[id(opt)].data_ptr(), st['pg'],
                             scale=float(getattr(opt, '_grad_scale', 1.0)) / w, first_step=bool(st['first']), grad_out=grad_out, stream=self.stream)
        st['first'] = False
        opt._nvl_held.append((dy, x))
        opt._synchronized = False
        self.launches += 3

    def sync_hyper(self, opt) -> None:
        """Upload ``opt``'s current learning rates etc. (call before replaying a captured step)."""
        # On the CURRENT stream, the one that replays the captured step: the upload is then ordered after every
        # kernel of the previous replay (which still reads the table) and before every kernel of the next one.
        # The side stream is idle between replays, so an upload there could land in the middle of a replay.
        self._hyper[id(opt)].sync(opt.param_groups)

    # ------------------------------------------------------------------ generic tensor all-reduce
    def _ensure_scratch(self, n_vec: int) -> None:
        """Scratch staging for :meth:`allreduce_async_`: a one-shot inbox with a fixed row stride and
        a separate two-shot buffer.  The two regions never overlap: a peer may still be reading its
        two-shot buffer when the next launch's one-shot stores arrive."""
        sc = self._scratch
        if sc is not None and sc['ts_cap'] >= n_vec:
            return
        ts_cap = max(n_vec, 1 << 16)
        os_cap = self.oneshot_max_bytes // 16 + 1
        os_bytes = int(self.lib.mgw_stage_bytes(_lib.ALGO_ONESHOT, os_cap, self._world))
        ts_bytes = int(self.lib.mgw_stage_bytes(_lib.ALGO_TWOSHOT, ts_cap, self._world))
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError('the all-reduce scratch area must exist before CUDA graph capture (call once eagerly first)')
        if sc is not None:
            # every rank grows at the same call: drain, meet, and give the old block back before taking a larger one
            torch.cuda.synchronize()
            runtime.barrier()
            self.arena.free(sc['block'])
            self._scratch_geometry = None
        os_al = (os_bytes + _ALIGN - 1) // _ALIGN * _ALIGN
        block = self.arena.alloc(os_al + ts_bytes + _ALIGN)
        self._scratch = dict(block=block, os_off=0, os_cap=os_cap, ts_off=os_al, ts_cap=ts_cap)

    def allreduce_async_(self, tensor: torch.Tensor, average: bool = True, name: Optional[str] = None,
                         algo: Optional[str] = None, n_ctas: Optional[int] = None):
        """In-place all-reduce of an arbitrary dense float32 CUDA tensor (collective: every rank
        must call it with the same shape).  Horovod-shaped; used by the communication profiler."""
        if tensor.dtype != torch.float32 or not tensor.is_cuda:
            raise ValueError('NvlComm.allreduce_async_ needs a float32 CUDA tensor')
        flat = tensor.view(-1)
        n_vec = (flat.numel() + 3) // 4
        self._ensure_scratch(n_vec)
        sc = self._scratch
        key = (flat.data_ptr(), flat.numel())
        table = self._scratch_tables.get(key)
        if table is None:
            if len(self._scratch_tables) > 256:
                self._scratch_tables.clear()
            table = GroupTable([flat], [0], [None], self.device)
            self._scratch_tables[key] = table
        plan = _GroupPlan()
        plan.table, plan.params, plan.block = table, [flat], sc['block']
        plan.algo, plan.n_ctas = self.choose(n_vec)
        if algo is not None:
            plan.algo = _lib.ALGO_NAMES[algo]
            plan.n_ctas = self.choose(n_vec)[1]
        if plan.algo == _lib.ALGO_ONESHOT and n_vec > sc['os_cap']:
            raise ValueError('message of %d bytes is too large for the one-shot inbox' % (n_vec * 16))
        if n_ctas is not None:
            plan.n_ctas = n_ctas
        plan.stage_off = sc['os_off'] if plan.algo == _lib.ALGO_ONESHOT else sc['ts_off']
        geometry = (plan.algo, n_vec, plan.n_ctas)
        if geometry != self._scratch_geometry:
            # Calls of different shapes cut the shared scratch area into different per-CTA chunks, and the
            # flag protocol only orders a CTA against the SAME CTA of its peers.  Every rank sees the change at
            # the same call, so all of them drain their queues and meet here before the area is reused.
            if not torch.cuda.is_current_stream_capturing():
                torch.cuda.synchronize()
                runtime.barrier()
            self._scratch_geometry = geometry
        self._fill_args(plan, sc['block'], 0, 0, inbox_stride=sc['os_cap'], stage_slots=sc['ts_cap'])
        compute = torch.cuda.current_stream()
        ready = torch.cuda.Event()
        ready.record(compute)
        self.stream.wait_event(ready)
        table.refresh_grads([flat], self.stream)
        plan.args.mode = _lib.MODE_WRITEBACK
        _lib.check(self.lib.mgw_allreduce_group(C.byref(plan.args), self.stream.cuda_stream), 'allreduce_group')
        self.launches += 1
        counters.bump('allreduce_fused')
        done = torch.cuda.Event()
        done.record(self.stream)
        return (done, tensor, None if average else float(self._world))

    def synchronize(self, handle):
        first, tensor, extra = handle
        if isinstance(first, torch.cuda.Event):
            torch.cuda.current_stream().wait_event(first)
            if extra is not None:
                tensor.mul_(extra)
        elif first is not None:
            first.wait()
        return tensor

    def broadcast_async_(self, tensor, root_rank, name=None):
        import torch.distributed as dist
        work = dist.broadcast(tensor, src=root_rank, group=runtime.data_group(), async_op=True)
        return (work, tensor, None)
