# -*- coding: utf-8 -*-
"""Tensor-core weight-gradient GEMM with an optimizer epilogue (``csrc/wgrad_gemm_sm100.cu``).

``wgrad_gemm(dy, x)`` returns ``dy^T @ x`` (TF32 inputs, fp32 accumulation in tensor memory).
``wgrad_sgd_(dy, x, weight, momentum_buffer, hyper, ...)`` applies the same product straight to the
weights: the gradient tile never makes a round trip through HBM.  ``GatheredWgradLinear`` uses it
for data-parallel training of large fully-connected layers whose batch is small: ranks exchange
their activations and output gradients (a few MB) instead of all-reducing the weight gradient
(hundreds of MB for the 25088 -> 4096 VGG layer, ``torchvision vgg16.classifier``).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib, counters

MODE_STORE, MODE_SGD = 1, 2
_declared = False


def _lib_ready():
    global _declared
    lib = _lib.load(allow_build=False)
    if not _declared:
        lib.mgw_wgrad_gemm_supported.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int]
        lib.mgw_wgrad_gemm.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_float, C.c_int, C.c_void_p,
                                       C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        lib.mgw_allgather_rows.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_longlong,
                                           C.c_int, C.c_ulonglong, C.c_void_p]
        lib.mgw_wgrad_scatter_stage_floats.restype = C.c_size_t
        lib.mgw_wgrad_scatter_stage_floats.argtypes = [C.c_int, C.c_int, C.c_int]
        lib.mgw_wgrad_gemm_scatter.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_float, C.c_void_p, C.c_int,
                                               C.c_int, C.c_void_p, C.c_void_p]
        lib.mgw_wgrad_reduce_finish.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                                C.c_int, C.c_int, C.c_int, C.c_ulonglong, C.c_void_p]
        _declared = True
    return lib


_status_cache = {}


def _status(device) -> torch.Tensor:
    """One status word per device in pinned host memory (device-visible under unified addressing): the kernels
    record a failed bounded wait there and the host can look at it without synchronising."""
    t = _status_cache.get(device)
    if t is None:
        t = _status_cache[device] = torch.zeros(8, dtype=torch.int32).pin_memory()
    return t


def set_persistent(form) -> None:
    """Choose the GEMM kernel: ``1`` / ``True`` the persistent one with one CTA of 16 epilogue warps per SM (CTAs walk
    over the tiles; loads and MMAs of the next tile overlap the epilogue of the current one), ``2`` the persistent one
    with two CTAs of 8 epilogue warps per SM, ``0`` / ``False`` one tile per CTA, ``None`` what
    ``MGWFBP_WGRAD_PERSISTENT`` says (default 1)."""
    lib = _lib_ready()
    lib.mgw_wgrad_set_persistent.restype = None
    lib.mgw_wgrad_set_persistent.argtypes = [C.c_int]
    lib.mgw_wgrad_set_persistent(-1 if form is None else int(form))


def supported(dy: torch.Tensor, x: torch.Tensor) -> bool:
    if not (dy.is_cuda and x.is_cuda and dy.dtype == torch.float32 and x.dtype == torch.float32):
        return False
    if dy.dim() != 2 or x.dim() != 2 or dy.shape[0] != x.shape[0] or not dy.is_contiguous() or not x.is_contiguous():
        return False
    return bool(_lib_ready().mgw_wgrad_gemm_supported(dy.data_ptr(), x.data_ptr(), dy.shape[1], x.shape[1], dy.shape[0]))


def check_status_nosync(device=None) -> None:
    """Raise if a GEMM CTA of a launch that has already finished gave up on one of its bounded waits."""
    for dev, t in _status_cache.items():
        if device is None or dev == device:
            code = int(t[0])
            if code != 0:
                t.zero_()
                raise RuntimeError('wgrad_gemm kernel reported wait failure code %d' % code)


def check_status(device=None) -> None:
    """As :func:`check_status_nosync`, after waiting for every launch issued so far."""
    if _status_cache:
        torch.cuda.synchronize()
    check_status_nosync(device)


def wgrad_gemm(dy: torch.Tensor, x: torch.Tensor, scale: float = 1.0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``scale * dy^T @ x`` for ``dy [K, M]`` and ``x [K, N]`` (row-major fp32)."""
    if not supported(dy, x):
        raise ValueError('wgrad_gemm needs contiguous fp32 CUDA matrices with M and N multiples of 4')
    lib = _lib_ready()
    K, M = dy.shape
    N = x.shape[1]
    if out is None:
        out = torch.empty(M, N, dtype=torch.float32, device=dy.device)
    _lib.check(lib.mgw_wgrad_gemm(dy.data_ptr(), x.data_ptr(), M, N, K, float(scale), MODE_STORE, out.data_ptr(), None, None,
                                  None, 0, 0, _status(dy.device).data_ptr(), torch.cuda.current_stream().cuda_stream), 'wgrad_gemm')
    counters.bump('wgrad_gemm_sm100')
    return out


def wgrad_sgd_(dy: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, momentum_buffer: Optional[torch.Tensor],
               hyper_ptr: int, pg: int = 0, scale: float = 1.0, first_step: bool = False,
               grad_out: Optional[torch.Tensor] = None, stream: Optional[torch.cuda.Stream] = None) -> None:
    """In-place SGD update of ``weight [M, N]`` with the gradient ``scale * dy^T @ x``; the
    hyper-parameters are read from the device table at ``hyper_ptr`` (entry ``pg``)."""
    if not supported(dy, x) or not weight.is_contiguous() or tuple(weight.shape) != (dy.shape[1], x.shape[1]):
        raise ValueError('wgrad_sgd_ needs contiguous fp32 CUDA operands of matching shapes')
    lib = _lib_ready()
    K, M = dy.shape
    N = x.shape[1]
    mode = MODE_SGD | (MODE_STORE if grad_out is not None else 0)
    s = (stream or torch.cuda.current_stream()).cuda_stream
    _lib.check(lib.mgw_wgrad_gemm(dy.data_ptr(), x.data_ptr(), M, N, K, float(scale), mode,
                                  None if grad_out is None else grad_out.data_ptr(), weight.data_ptr(),
                                  None if momentum_buffer is None else momentum_buffer.data_ptr(), hyper_ptr, pg,
                                  int(first_step), _status(dy.device).data_ptr(), s), 'wgrad_gemm(sgd)')
    counters.bump('wgrad_gemm_sm100')


# --------------------------------------------------------------------------------------------------
# Data-parallel linear layer whose weight gradient is never all-reduced
# --------------------------------------------------------------------------------------------------
class _GatheredLinearFn(torch.autograd.Function):
    """``y = x W^T + b`` whose backward hands ``(dy, x)`` to the communicator instead of forming ``dW``."""

    @staticmethod
    def forward(ctx, x, weight, bias, module):
        ctx.save_for_backward(x, weight)
        ctx.module = module
        ctx.has_bias = bias is not None
        return torch.nn.functional.linear(x, weight, bias)

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        x2 = x.reshape(-1, x.shape[-1])
        dx = (dy2 @ weight).reshape(x.shape) if ctx.needs_input_grad[0] else None
        db = dy2.sum(0) if ctx.has_bias else None
        sink = getattr(ctx.module.weight, '_mgw_rs_sink', None)
        if sink is not None:
            sink(dy2.contiguous(), x2.contiguous())        # GEMM with the reduce-scatter epilogue + owners' sums, side stream
        else:
            ctx.module._exchange(ctx.module, dy2.contiguous(), x2.contiguous())     # gather + GEMM + update on the side stream
        return dx, None, db, None


class GatheredWgradLinear(torch.nn.Linear):
    """``nn.Linear`` (same parameters and ``state_dict`` keys) for large layers fed by small batches.

    Under a fused data-parallel optimizer the weight takes no part in the gradient all-reduce:
    during backward every rank publishes its ``dy`` and ``x`` rows, pulls the other ranks' rows over
    NVLink, and applies ``(1/W) * dY_all^T X_all`` to its weights with the tensor-core GEMM whose
    epilogue is the SGD update.  Traffic is ``W*B*(in+out)`` floats instead of ``in*out``.  Without
    such an optimizer (single process, CPU, other optimizers) it behaves exactly like ``nn.Linear``.
    """
    batch_rows_hint: Optional[int] = None      # rows of x per step and rank, set by the trainer

    def gathered_is_profitable(self, world: int) -> bool:
        rows = self.batch_rows_hint
        if rows is None or world < 1:
            return False
        m, n = self.out_features, self.in_features
        return (m % 4 == 0 and n % 4 == 0 and world * rows * (m + n) * 2 <= m * n)

    def forward(self, x):
        external = getattr(self, '_exchange', None) is not None or getattr(self.weight, '_mgw_rs_sink', None) is not None
        if external and self.training and torch.is_grad_enabled() and x.is_cuda:
            return _GatheredLinearFn.apply(x, self.weight, self.bias, self)
        return super().forward(x)


def convert_large_linears(net: torch.nn.Module, min_params: int = 8 * 1024 * 1024) -> int:
    """Swap every ``nn.Linear`` with at least ``min_params`` weights for :class:`GatheredWgradLinear`
    (in place: parameters, buffers and names are untouched).  Returns how many were converted."""
    n = 0
    for m in net.modules():
        if type(m) is torch.nn.Linear and m.in_features * m.out_features >= min_params:
            m.__class__ = GatheredWgradLinear
            m.weight._mgw_gathered = m
            n += 1
    return n
