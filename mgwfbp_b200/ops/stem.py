# -*- coding: utf-8 -*-
"""The ImageNet stem convolution (7x7, stride 2, padding 3, 3 input channels) as a 4x4 / stride 1
convolution over the 2x2 space-to-depth input (12 channels).

A 3-channel channels-last input is the worst case for tensor-core convolution kernels: on B200 cuDNN pads
it, converts its layout and runs legacy kernels (0.85 ms forward + weight gradient at batch 64, 7 % of a
ResNet-50 step).  The same arithmetic on the rearranged input runs on the regular implicit-GEMM kernels.
The module keeps the canonical ``[O, 3, 7, 7]`` weight as its parameter (state-dict compatible with
``torch.nn.Conv2d``); the ``[O, 12, 4, 4]`` view of it is rebuilt every forward pass through autograd
ops on a 9 K-element tensor, the input is rearranged by one kernel (``csrc/stem_s2d.cu``).

Index algebra: output row ``r`` reads input rows ``2r + k - 3``, ``k = 0..6``.  With ``h = 2j + p`` (``p`` the
row parity) and four zero rows on top, tap ``k`` lands on cell offset ``a = (k + 1 - p) / 2`` of a 4-tap kernel,
i.e. ``k = 2a + p - 1``; ``k = -1`` is a zero tap.  Same for columns.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import _lib, counters


def s2d_weight(w: torch.Tensor) -> torch.Tensor:
    """``[O, 3, 7, 7]`` -> ``[O, 12, 4, 4]`` with input-channel index ``p * 6 + q * 3 + c`` (differentiable)."""
    o = w.shape[0]
    wp = F.pad(w, (1, 0, 1, 0))                       # index k + 1; the new first row / column is the zero tap
    wp = wp.view(o, 3, 4, 2, 4, 2)                    # [o, c, a, p, b, q]
    return wp.permute(0, 3, 5, 1, 2, 4).reshape(o, 12, 4, 4)


def s2d_input_reference(x: torch.Tensor) -> torch.Tensor:
    """The rearranged input with plain tensor ops (any device); what the kernel computes."""
    n, _, h, w = x.shape
    xp = F.pad(x, (4, 2, 4, 2)).view(n, 3, h // 2 + 3, 2, w // 2 + 3, 2)      # [n, c, j, p, i, q]
    return xp.permute(0, 3, 5, 1, 2, 4).reshape(n, 12, h // 2 + 3, w // 2 + 3)


def s2d_input(x: torch.Tensor) -> torch.Tensor:
    """``x``: channels-last ``[N, 3, H, W]`` float32 CUDA tensor, H and W even -> channels-last ``[N, 12, H/2+3, W/2+3]``."""
    n, _, h, w = x.shape
    out = torch.empty((n, 12, h // 2 + 3, w // 2 + 3), device=x.device, dtype=x.dtype, memory_format=torch.channels_last)
    lib = _lib.load(allow_build=False)
    _lib.check(lib.mgw_s2d_stem_input(x.data_ptr(), out.data_ptr(), n, h, w, torch.cuda.current_stream().cuda_stream),
               's2d_stem_input')
    counters.bump('s2d_stem_input')
    return out


class S2DStemConv2d(nn.Conv2d):
    """Drop-in for ``nn.Conv2d(3, O, 7, stride=2, padding=3)``; any other configuration or input runs the parent."""

    def _rearranged_ok(self, x: torch.Tensor) -> bool:
        return (x.is_cuda and x.dtype == torch.float32 and x.dim() == 4 and x.shape[1] == 3 and not x.requires_grad
                and x.shape[2] % 2 == 0 and x.shape[3] % 2 == 0 and x.shape[2] >= 8 and x.shape[3] >= 8
                and x.is_contiguous(memory_format=torch.channels_last)
                and tuple(self.weight.shape[1:]) == (3, 7, 7) and self.stride == (2, 2) and self.padding == (3, 3)
                and self.dilation == (1, 1) and self.groups == 1 and self.padding_mode == 'zeros')

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not self._rearranged_ok(x):
            return super().forward(x)
        ws = s2d_weight(self.weight).contiguous(memory_format=torch.channels_last)
        return F.conv2d(s2d_input(x), ws, self.bias, 1, 0)


def convert_stem(conv: nn.Conv2d) -> nn.Conv2d:
    """``conv`` re-typed as :class:`S2DStemConv2d` sharing its parameters when it is an ImageNet stem; else unchanged."""
    if (type(conv) is nn.Conv2d and conv.in_channels == 3 and conv.kernel_size == (7, 7) and conv.stride == (2, 2)
            and conv.padding == (3, 3) and conv.dilation == (1, 1) and conv.groups == 1 and conv.padding_mode == 'zeros'):
        new = S2DStemConv2d(3, conv.out_channels, 7, stride=2, padding=3, bias=conv.bias is not None)
        new.weight = conv.weight
        new.bias = conv.bias
        return new
    return conv
