# -*- coding: utf-8 -*-
"""DenseNet blocks without the quadratic number of gradient additions.

torchvision's ``_DenseBlock`` (the reference builds its DenseNets from torchvision, ``dl_trainer.py:221-231``) keeps a
list of feature maps and lets every layer concatenate all of them.  In backward every feature map then receives one
gradient slice from each later layer of its block, and autograd adds them up one slice at a time: L (L - 1) / 2 small
strided additions per block, 1815 kernels of about 3 us per step for DenseNet-201 (6 + 12 + 48 + 32 layers) -- 5.4 ms
of a 24 ms step on a B200, all of it launch latency.

Here a block owns ONE buffer ``[N, C_total, H, W]``: layer *l* reads its first ``C_l`` channels and writes its
``growth`` new channels behind them, so the buffer is also the block's output and the final concatenation disappears.
Backward walks the layers in reverse over one gradient buffer of the same shape: the gradient of layer *l*'s output
is complete when its turn comes (every later layer has already added its share), the layer's own graph is run by a
nested ``torch.autograd.backward`` (parameter gradients accumulate as usual, so gradient hooks fire in the usual
order) and its input gradient is added to the first ``C_l`` channels in ONE kernel.  L additions instead of
L (L - 1) / 2, moving the same bytes.  On the GPU the first BatchNorm of a layer reads its channel slice of the buffer
in place (row stride = total channels) and its backward kernel adds the input gradient into the gradient buffer
directly (``ops/bn_relu.py``), so neither a concatenated copy nor a separate addition kernel remains.

Parameters, buffers and ``state_dict`` keys are untouched: :func:`fuse_dense_blocks` only binds a new ``forward``.
"""
from __future__ import annotations

import os

import torch
import torch.nn.functional as F
from torch.autograd.function import once_differentiable

_ENABLED = os.environ.get('MGWFBP_DENSE_BLOCK', '1').strip().lower() not in ('0', 'false', 'no', 'off')


class _Tap(torch.autograd.Function):
    """Identity in forward; in backward it hands the gradient to a callback instead of passing it on."""

    @staticmethod
    def forward(ctx, x, cell):
        ctx.cell = cell
        ctx.set_materialize_grads(False)        # no gradient (the consumer added it to the buffer itself) stays None
        return x.view_as(x)

    @staticmethod
    @once_differentiable
    def backward(ctx, grad):
        if grad is not None:
            ctx.cell['sink'](grad)
        return None, None


def _alias(view: torch.Tensor) -> torch.Tensor:
    """The same memory as ``view`` under a version counter of its own: the block buffer is written again (behind the
    channels ``view`` covers) after ``view`` has been saved for backward, which must not look like an in-place change."""
    out = torch.empty(0, dtype=view.dtype, device=view.device)
    out.set_(view.untyped_storage(), view.storage_offset(), view.size(), view.stride())
    return out


def _layer_body(layer, x):
    """``_DenseLayer`` on an already concatenated input (fused BatchNorm+ReLU modules carry their ReLU themselves)."""
    out = layer.norm1(x)
    if not getattr(layer.norm1, 'fused_relu', False):
        out = layer.relu1(out)
    out = layer.norm2(layer.conv1(out))
    if not getattr(layer.norm2, 'fused_relu', False):
        out = layer.relu2(out)
    out = layer.conv2(out)
    if layer.drop_rate > 0:
        out = F.dropout(out, p=layer.drop_rate, training=layer.training)
    return out


class _DenseBlockFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x0, block):
        layers = list(block.values())
        c0 = x0.shape[1]
        total = c0 + sum(l.conv2.out_channels for l in layers)
        channels_last = x0.dim() == 4 and x0.is_contiguous(memory_format=torch.channels_last) and not x0.is_contiguous()
        buf = torch.empty((x0.shape[0], total) + tuple(x0.shape[2:]), dtype=x0.dtype, device=x0.device,
                          memory_format=torch.channels_last if channels_last else torch.contiguous_format)
        buf[:, :c0].copy_(x0)
        steps, c = [], c0
        for layer in layers:
            cell = {}
            with torch.enable_grad():
                xin = _alias(buf[:, :c]).requires_grad_(True)
                tapped = _Tap.apply(xin, cell)
                tapped._mgw_grad_cell = cell         # the fused BatchNorm adds its input gradient to cell['target'] itself
                out = _layer_body(layer, tapped)
            g = out.shape[1]
            buf[:, c:c + g].copy_(out.detach())
            steps.append((c, g, cell, out))          # `out` keeps the layer's autograd graph alive until backward
            c += g
        ctx.steps, ctx.c0 = steps, c0
        return buf

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_out):
        steps, ctx.steps = ctx.steps, None
        if steps is None:
            raise RuntimeError('a dense block can run backward once per forward: the graphs of its layers are freed by it')
        grad = grad_out.clone(memory_format=torch.preserve_format)        # accumulated in place below
        for c, g, cell, out in reversed(steps):
            head = grad[:, :c]
            cell['sink'], cell['target'] = head.add_, head
            g_out = grad[:, c:c + g]
            if g_out.dtype != out.dtype:          # mixed precision: the layer ran in a narrower type than the buffer holds
                g_out = g_out.to(out.dtype)
            torch.autograd.backward(out, g_out)
            cell.clear()
        return grad[:, :ctx.c0], None


def _plain_forward(self, init_features):
    features = [init_features]
    for layer in self.values():
        features.append(layer(features))
    return torch.cat(features, 1)


def _block_forward(self, init_features):
    if (_ENABLED and self.training and torch.is_grad_enabled() and torch.is_tensor(init_features) and init_features.requires_grad
            and not any(getattr(l, 'memory_efficient', False) for l in self.values())):
        return _DenseBlockFn.apply(init_features, self)
    return _plain_forward(self, init_features)


def fuse_dense_blocks(net: torch.nn.Module) -> int:
    """Bind the single-buffer forward to every torchvision ``_DenseBlock`` of ``net``; returns how many were found."""
    try:
        from torchvision.models.densenet import _DenseBlock
    except Exception:      # pragma: no cover - torchvision is optional
        return 0
    from .fuse import _bind
    n = 0
    for m in net.modules():
        if isinstance(m, _DenseBlock):
            _bind(m, _block_forward)
            n += 1
    return n
