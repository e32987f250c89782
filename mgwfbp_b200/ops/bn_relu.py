# -*- coding: utf-8 -*-
"""Fused BatchNorm (+ residual add) (+ ReLU) for channels-last activations (``csrc/bn_relu.cu``).

``FusedBatchNorm2d`` / ``FusedBatchNorm1d`` are drop-in subclasses of the torch modules: same
parameters, buffers and ``state_dict`` keys (``weight, bias, running_mean, running_var,
num_batches_tracked``), same numerics (biased variance for normalisation, unbiased for the running
estimate, momentum and eps as configured).  In training mode on a CUDA device with a dense
channels-innermost input they run this package's kernels; ``forward(x, residual=None)`` optionally
adds a residual before the ReLU, which covers the tail of a ResNet block in one pass.  The
reference gets the same math from separate cuDNN BatchNorm, add and ReLU kernels
(``models/resnet.py:29-39``, torchvision ``Bottleneck``).
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import _lib, counters


def _as_rows(x: torch.Tensor):
    """View a dense channels-innermost tensor as (M, C); returns None when the layout does not fit."""
    if x.dim() == 2:
        return (x.shape[0], x.shape[1]) if x.is_contiguous() else None
    if x.dim() == 4 and x.is_contiguous(memory_format=torch.channels_last):
        n, c, h, w = x.shape
        return n * h * w, c
    return None


def _row_layout(x: torch.Tensor):
    """``(M, C, ld)`` for an input the kernels can read in place: a dense channels-innermost tensor (``ld == C``), or the
    first channels of a wider channels-last tensor (``x = wide[:, :C]``: rows ``ld = C_wide`` floats apart), 16-byte
    aligned with ``ld % 4 == 0`` when the vector path applies.  ``None`` otherwise."""
    rows = _as_rows(x)
    if rows is not None:
        return rows[0], rows[1], rows[1]
    if x.dim() != 4:
        return None
    n, c, h, w = x.shape
    ld = x.stride(3)
    if min(n, c, h, w) < 1 or w < 2 or x.stride(1) != 1 or ld <= c or x.stride(2) != w * ld or x.stride(0) != h * w * ld:
        return None
    if c % 4 == 0 and (ld % 4 != 0 or x.data_ptr() % 16 != 0):
        return None
    return n * h * w, c, ld


_declared = False


def _declare(lib) -> None:
    global _declared
    if _declared:
        return
    lib.mgw_bn_partials_floats.restype = C.c_size_t
    lib.mgw_bn_partials_floats.argtypes = [C.c_longlong, C.c_int]
    lib.mgw_bn_relu_fwd.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_longlong, C.c_int, C.c_void_p, C.c_void_p,
                                    C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_float, C.c_int, C.c_void_p,
                                    C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.mgw_bn_relu_bwd.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_longlong, C.c_int,
                                    C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p,
                                    C.c_void_p, C.c_void_p, C.c_void_p]
    # the same with a row stride for x, and (backward) a row stride and an accumulate flag for dx
    lib.mgw_bn_relu_fwd_ld.argtypes = [C.c_void_p, C.c_longlong] + list(lib.mgw_bn_relu_fwd.argtypes[1:])
    lib.mgw_bn_relu_bwd_ld.argtypes = (list(lib.mgw_bn_relu_bwd.argtypes[:4]) + [C.c_longlong] +
                                       list(lib.mgw_bn_relu_bwd.argtypes[4:6]) + [C.c_longlong, C.c_int] +
                                       list(lib.mgw_bn_relu_bwd.argtypes[6:]))
    lib.mgw_bn_launches.argtypes = [C.c_longlong, C.c_int, C.c_int]
    lib.mgw_bn_set_sm_budget.argtypes = [C.c_int]
    lib.mgw_bn_cluster_supported.argtypes = [C.c_longlong, C.c_int]
    lib.mgw_bn_relu_fwd_cluster.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_longlong, C.c_int, C.c_void_p, C.c_void_p,
                                            C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_float, C.c_int, C.c_void_p,
                                            C.c_void_p, C.c_void_p, C.c_void_p]
    lib.mgw_bn_relu_bwd_cluster.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_longlong,
                                            C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p,
                                            C.c_void_p, C.c_void_p, C.c_void_p]
    _declared = True


# Small activations (at most 8192 rows, at most 288 channels in multiples of 16) take the one-launch cluster kernels
# (csrc/bn_relu_cluster.cu); MGWFBP_BN_CLUSTER=0 keeps everything on the three-launch kernels.
_CLUSTER = os.environ.get('MGWFBP_BN_CLUSTER', '1').strip().lower() not in ('0', 'false', 'no', 'off', '')


def set_sm_budget(sms: int) -> int:
    """Size the BatchNorm grids for ``sms`` SMs from now on (0: all of them); returns the previous budget.

    The kernels run as exactly one resident wave.  A job whose communication kernels hold a few SMs beside backward
    (``NvlComm.overlap_ctas``) lowers the budget by that many, so the wave still fits while such a kernel is running;
    call it before the training step is captured in a CUDA graph."""
    lib = _lib.load(allow_build=False)
    _declare(lib)
    return int(lib.mgw_bn_set_sm_budget(int(sms)))


def _use_cluster(lib, M: int, Cc: int) -> bool:
    return _CLUSTER and bool(lib.mgw_bn_cluster_supported(M, Cc))


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


class _BNReLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, running_mean, running_var, num_batches_tracked, residual, relu, momentum, eps, dual):
        lib = _lib.load(allow_build=False)
        _declare(lib)
        M, Cc, ld = _row_layout(x)
        y = torch.empty_like(x) if ld == Cc else torch.empty(x.shape, dtype=x.dtype, device=x.device, memory_format=torch.channels_last)
        mean = torch.empty(Cc, dtype=torch.float32, device=x.device)
        invstd = torch.empty(Cc, dtype=torch.float32, device=x.device)
        s = torch.cuda.current_stream().cuda_stream
        # With a residual the ReLU mask cannot be rebuilt from x alone.  The forward kernel then records it as
        # one byte per float4 (1/16 of the tensor) and backward reads that instead of the output tensor; when
        # the channel count is not a multiple of 4 the output itself is kept.
        needs_mask = bool(relu and residual is not None)
        bits = torch.empty((M * Cc) // 4, dtype=torch.uint8, device=x.device) if (needs_mask and Cc % 4 == 0) else None
        if ld == Cc and _use_cluster(lib, M, Cc):
            _lib.check(lib.mgw_bn_relu_fwd_cluster(x.data_ptr(), _ptr(residual), y.data_ptr(), M, Cc, _ptr(weight), _ptr(bias),
                                                   _ptr(running_mean), _ptr(running_var), _ptr(num_batches_tracked),
                                                   float(momentum), float(eps), int(relu), mean.data_ptr(), invstd.data_ptr(),
                                                   _ptr(bits), s), 'bn_relu_fwd_cluster')
            counters.bump('bn_relu_fwd_cluster', 1)
        else:
            partials = torch.empty(lib.mgw_bn_partials_floats(M, Cc), dtype=torch.float32, device=x.device)
            if ld == Cc:
                _lib.check(lib.mgw_bn_relu_fwd(x.data_ptr(), _ptr(residual), y.data_ptr(), M, Cc, _ptr(weight), _ptr(bias),
                                               _ptr(running_mean), _ptr(running_var), _ptr(num_batches_tracked),
                                               float(momentum), float(eps), int(relu), mean.data_ptr(), invstd.data_ptr(),
                                               partials.data_ptr(), _ptr(bits), s), 'bn_relu_fwd')
            else:       # a channel slice of a wider tensor, read in place
                _lib.check(lib.mgw_bn_relu_fwd_ld(x.data_ptr(), ld, _ptr(residual), y.data_ptr(), M, Cc, _ptr(weight), _ptr(bias),
                                                  _ptr(running_mean), _ptr(running_var), _ptr(num_batches_tracked),
                                                  float(momentum), float(eps), int(relu), mean.data_ptr(), invstd.data_ptr(),
                                                  partials.data_ptr(), _ptr(bits), s), 'bn_relu_fwd_ld')
                counters.bump('note:bn_relu_fwd_strided', 1)
            counters.bump('bn_relu_fwd', lib.mgw_bn_launches(M, Cc, 0))
        ctx.save_for_backward(x, y if (needs_mask and bits is None) else None, weight, bias, mean, invstd, bits)
        ctx.relu, ctx.has_residual, ctx.rows, ctx.ld = bool(relu), residual is not None, (M, Cc), ld
        # A caller that sums the gradients of several consumers of x in one buffer (models/dense_block.py) leaves a dict
        # on the input tensor; when backward runs, its 'target' entry is where this layer's input gradient is ADDED.
        ctx.grad_cell = getattr(x, '_mgw_grad_cell', None)
        ctx.mark_non_differentiable(*[t for t in (running_mean, running_var, num_batches_tracked) if t is not None])
        if dual:
            # two handles on the same output: each consumer's gradient then reaches backward() separately
            # and the kernel sums them while loading, instead of autograd launching an add kernel
            return y, y.view_as(y)
        return y

    @staticmethod
    def backward(ctx, dy, dy2=None):
        lib = _lib.load(allow_build=False)
        if dy is None:
            dy, dy2 = dy2, None
        x, y, weight, bias, mean, invstd, bits = ctx.saved_tensors
        M, Cc = ctx.rows
        ld = ctx.ld
        four_d = x.dim() == 4
        # where the input gradient goes: a dense tensor of its own, or -- added -- the caller's wider gradient buffer
        target = ctx.grad_cell.get('target') if (ctx.grad_cell is not None and not ctx.has_residual) else None
        if target is not None:
            t_layout = _row_layout(target)
            if target.shape != x.shape or target.dtype != x.dtype or t_layout is None:
                target = None
        if target is None:
            dx = torch.empty_like(x) if ld == Cc else torch.empty(x.shape, dtype=x.dtype, device=x.device,
                                                                  memory_format=torch.channels_last)
            dense_stride = dx.stride()
        else:
            dx = None
            n_, c_, h_, w_ = x.shape
            dense_stride = (h_ * w_ * c_, 1, w_ * c_, c_)
        if _as_rows(dy) is None or dy.stride() != dense_stride:
            dy = dy.contiguous(memory_format=torch.channels_last) if four_d else dy.contiguous()
        if dy2 is not None and (_as_rows(dy2) is None or dy2.stride() != dense_stride):
            dy2 = dy2.contiguous(memory_format=torch.channels_last) if four_d else dy2.contiguous()
        dz = torch.empty_like(dx) if ctx.has_residual else None     # only a residual needs the masked gradient itself
        dgamma = torch.empty(Cc, dtype=torch.float32, device=x.device)
        dbeta = torch.empty(Cc, dtype=torch.float32, device=x.device)
        s = torch.cuda.current_stream().cuda_stream
        if target is None and ld == Cc and _use_cluster(lib, M, Cc):
            _lib.check(lib.mgw_bn_relu_bwd_cluster(dy.data_ptr(), _ptr(dy2), _ptr(y), x.data_ptr(), _ptr(dz), dx.data_ptr(), M, Cc,
                                                   _ptr(weight), _ptr(bias), mean.data_ptr(), invstd.data_ptr(), int(ctx.relu),
                                                   dgamma.data_ptr(), dbeta.data_ptr(), _ptr(bits), s), 'bn_relu_bwd_cluster')
            counters.bump('bn_relu_bwd_cluster', 1)
        else:
            partials = torch.empty(lib.mgw_bn_partials_floats(M, Cc), dtype=torch.float32, device=x.device)
            if target is not None:      # dx is added into the caller's buffer and never exists by itself
                _lib.check(lib.mgw_bn_relu_bwd_ld(dy.data_ptr(), _ptr(dy2), _ptr(y), x.data_ptr(), ld, None, target.data_ptr(),
                                                  t_layout[2], 1, M, Cc, _ptr(weight), _ptr(bias), mean.data_ptr(),
                                                  invstd.data_ptr(), int(ctx.relu), dgamma.data_ptr(), dbeta.data_ptr(),
                                                  partials.data_ptr(), _ptr(bits), s), 'bn_relu_bwd_ld(accumulate)')
                counters.bump('note:bn_relu_bwd_accumulate', 1)
            elif ld == Cc:
                _lib.check(lib.mgw_bn_relu_bwd(dy.data_ptr(), _ptr(dy2), _ptr(y), x.data_ptr(), _ptr(dz), dx.data_ptr(), M, Cc,
                                               _ptr(weight), _ptr(bias), mean.data_ptr(), invstd.data_ptr(), int(ctx.relu),
                                               dgamma.data_ptr(), dbeta.data_ptr(), partials.data_ptr(), _ptr(bits), s), 'bn_relu_bwd')
            else:
                _lib.check(lib.mgw_bn_relu_bwd_ld(dy.data_ptr(), _ptr(dy2), _ptr(y), x.data_ptr(), ld, _ptr(dz), dx.data_ptr(), Cc, 0,
                                                  M, Cc, _ptr(weight), _ptr(bias), mean.data_ptr(), invstd.data_ptr(), int(ctx.relu),
                                                  dgamma.data_ptr(), dbeta.data_ptr(), partials.data_ptr(), _ptr(bits), s),
                           'bn_relu_bwd_ld')
            counters.bump('bn_relu_bwd', lib.mgw_bn_launches(M, Cc, 1))
        need = ctx.needs_input_grad
        return (dx if need[0] else None, dgamma if (weight is not None and need[1]) else None,
                dbeta if need[2] else None, None, None, None, dz if (ctx.has_residual and need[6]) else None,
                None, None, None, None)


def bn_relu(x, weight, bias, running_mean, running_var, num_batches_tracked, residual=None, relu=True,
            momentum=0.1, eps=1e-5, dual=False):
    """Functional form: training-mode batch norm over all but the channel dimension, optional
    residual add, optional ReLU.  ``x`` must be CUDA float32, dense, channels innermost."""
    if not x.is_cuda or x.dtype != torch.float32:
        raise ValueError('bn_relu needs a float32 CUDA tensor')
    _declare(_lib.load(allow_build=False))
    layout = _row_layout(x)
    if layout is None:
        raise ValueError('bn_relu needs a dense channels-last (or 2-D) tensor, or the first channels of a wider channels-last one')
    if residual is not None and (residual.shape != x.shape or _as_rows(residual) is None or
                                 (layout[2] == layout[1] and residual.stride() != x.stride())):
        residual = residual.contiguous(memory_format=torch.channels_last) if x.dim() == 4 else residual.contiguous()
    return _BNReLU.apply(x, weight, bias, running_mean, running_var, num_batches_tracked, residual, relu, momentum, eps, dual)


class _FusedBNMixin:
    fused_relu = False

    def _native_ok(self, x: torch.Tensor) -> bool:
        if not _declared and x.is_cuda:
            _declare(_lib.load(allow_build=False))           # also settles which input layouts the library reads in place
        return (self.training and x.is_cuda and x.dtype == torch.float32 and self.momentum is not None
                and self.track_running_stats and x.numel() > 0 and _row_layout(x) is not None)

    def forward(self, x, residual=None, dual=False):
        """``dual=True`` returns the output twice (two handles on one tensor) for a consumer pair such as
        the next block's first convolution and its shortcut; see :func:`bn_relu`."""
        if self._native_ok(x):
            return bn_relu(x, self.weight, self.bias, self.running_mean, self.running_var, self.num_batches_tracked,
                           residual, self.fused_relu, self.momentum, self.eps, dual)
        if x.is_cuda and x.dim() == 4 and self.training and not x.is_contiguous(memory_format=torch.channels_last) \
                and x.dtype == torch.float32 and self.momentum is not None and self.track_running_stats:
            # keep the native path: one layout conversion is cheaper than leaving the fused kernels
            return self.forward(x.contiguous(memory_format=torch.channels_last),
                                None if residual is None else residual.contiguous(memory_format=torch.channels_last), dual)
        out = super().forward(x)
        if residual is not None:
            out = out + residual
        out = F.relu(out) if self.fused_relu else out
        return (out, out) if dual else out

    def extra_repr(self):
        return super().extra_repr() + ', fused_relu=%s' % self.fused_relu


class FusedBatchNorm2d(_FusedBNMixin, nn.BatchNorm2d):
    pass


class FusedBatchNorm1d(_FusedBNMixin, nn.BatchNorm1d):
    pass


# --------------------------------------------------------------------------------------------------
# BatchNorm + ReLU + MaxPool(3, stride 2, padding 1): the ResNet / DenseNet stem in two passes over x
# --------------------------------------------------------------------------------------------------
_pool_declared = False


def _declare_pool(lib) -> None:
    global _pool_declared
    if not _pool_declared:
        lib.mgw_bn_relu_maxpool_fwd.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p,
                                                C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_float, C.c_void_p,
                                                C.c_void_p, C.c_void_p, C.c_void_p]
        lib.mgw_bn_relu_maxpool_bwd.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                                C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                                C.c_void_p]
        _pool_declared = True


class _BNReLUMaxPool(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, running_mean, running_var, num_batches_tracked, momentum, eps):
        lib = _lib.load(allow_build=False)
        _declare(lib)
        _declare_pool(lib)
        n, c, h, w = x.shape
        oh, ow = (h - 1) // 2 + 1, (w - 1) // 2 + 1
        y = torch.empty((n, c, oh, ow), dtype=x.dtype, device=x.device, memory_format=torch.channels_last)
        idx = torch.empty((n, oh, ow, c), dtype=torch.uint8, device=x.device)
        mean = torch.empty(c, dtype=torch.float32, device=x.device)
        invstd = torch.empty(c, dtype=torch.float32, device=x.device)
        partials = torch.empty(lib.mgw_bn_partials_floats(n * h * w, c), dtype=torch.float32, device=x.device)
        s = torch.cuda.current_stream().cuda_stream
        _lib.check(lib.mgw_bn_relu_maxpool_fwd(x.data_ptr(), y.data_ptr(), idx.data_ptr(), n, h, w, c, _ptr(weight), _ptr(bias),
                                               _ptr(running_mean), _ptr(running_var), _ptr(num_batches_tracked), float(momentum),
                                               float(eps), mean.data_ptr(), invstd.data_ptr(), partials.data_ptr(), s),
                   'bn_relu_maxpool_fwd')
        counters.bump('bn_relu_maxpool_fwd', 3)
        ctx.save_for_backward(x, idx, weight, bias, mean, invstd)
        ctx.mark_non_differentiable(*[t for t in (running_mean, running_var, num_batches_tracked) if t is not None])
        return y

    @staticmethod
    def backward(ctx, dp):
        lib = _lib.load(allow_build=False)
        x, idx, weight, bias, mean, invstd = ctx.saved_tensors
        n, c, h, w = x.shape
        if not dp.is_contiguous(memory_format=torch.channels_last):
            dp = dp.contiguous(memory_format=torch.channels_last)
        dx = torch.empty_like(x)
        dgamma = torch.empty(c, dtype=torch.float32, device=x.device)
        dbeta = torch.empty(c, dtype=torch.float32, device=x.device)
        partials = torch.empty(lib.mgw_bn_partials_floats(n * h * w, c), dtype=torch.float32, device=x.device)
        s = torch.cuda.current_stream().cuda_stream
        _lib.check(lib.mgw_bn_relu_maxpool_bwd(dp.data_ptr(), idx.data_ptr(), x.data_ptr(), dx.data_ptr(), n, h, w, c, _ptr(weight),
                                               _ptr(bias), mean.data_ptr(), invstd.data_ptr(), dgamma.data_ptr(), dbeta.data_ptr(),
                                               partials.data_ptr(), s), 'bn_relu_maxpool_bwd')
        counters.bump('bn_relu_maxpool_bwd', 3)
        need = ctx.needs_input_grad
        return (dx if need[0] else None, dgamma if (weight is not None and need[1]) else None, dbeta if need[2] else None,
                None, None, None, None, None)


def bn_relu_maxpool(bn: torch.nn.BatchNorm2d, pool: torch.nn.MaxPool2d, x: torch.Tensor) -> torch.Tensor:
    """``pool(relu(bn(x)))`` for a training-mode BatchNorm and a 3x3 / stride 2 / padding 1 max-pool, without ever
    writing the full-resolution normalised tensor; any other configuration runs the modules one after the other."""
    def _pair(v):
        return tuple(v) if isinstance(v, (tuple, list)) else (v, v)
    fusable = (isinstance(bn, _FusedBNMixin) and bn._native_ok(x) and x.dim() == 4 and _as_rows(x) is not None and x.shape[1] % 4 == 0
               and _pair(pool.kernel_size) == (3, 3) and _pair(pool.stride) == (2, 2) and _pair(pool.padding) == (1, 1)
               and _pair(pool.dilation) == (1, 1) and not pool.ceil_mode and not pool.return_indices)
    if not fusable:
        out = bn(x)
        if not getattr(bn, 'fused_relu', False):
            out = F.relu(out)
        return pool(out)
    return _BNReLUMaxPool.apply(x, bn.weight, bn.bias, bn.running_mean, bn.running_var, bn.num_batches_tracked,
                                bn.momentum, bn.eps)
