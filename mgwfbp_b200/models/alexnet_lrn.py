# -*- coding: utf-8 -*-
"""Original (two-tower, local-response-normalised) AlexNet.

Same layer stack and state-dict layout as reference ``models/alexnet.py:9-87`` (``features.{0,4,8,10,12}``,
``classifier.{0,3,6}``); the registry uses torchvision's AlexNet for the ``alexnet`` key, as the reference does
(``dl_trainer.py:121-123``), and this class remains available as ``models.AlexNet``.  The network is assembled
from a layer table, and the normalisation is written with ``avg_pool`` calls on a view instead of pooling modules.
"""
from __future__ import annotations

from typing import List

import torch
import torch.nn as nn
import torch.nn.functional as F


class LRN(nn.Module):
    """``x / (1 + alpha * mean_window(x^2)) ** beta``; the window runs over neighbouring channels
    (``ACROSS_CHANNELS``) or over a square neighbourhood inside each channel."""

    def __init__(self, local_size: int = 1, alpha: float = 1.0, beta: float = 0.75, ACROSS_CHANNELS: bool = True):
        super().__init__()
        self.local_size, self.alpha, self.beta = int(local_size), float(alpha), float(beta)
        self.ACROSS_CHANNELS = bool(ACROSS_CHANNELS)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        k, pad = self.local_size, (self.local_size - 1) // 2
        squares = x * x
        if self.ACROSS_CHANNELS:
            # average over a window of k channels: treat the channel axis as the depth of a 3-D pooling
            window_mean = F.avg_pool3d(squares[:, None], (k, 1, 1), stride=1, padding=(pad, 0, 0))[:, 0]
        else:
            window_mean = F.avg_pool2d(squares, k, stride=1, padding=pad)
        return x * torch.pow(1.0 + self.alpha * window_mean, -self.beta)

    def extra_repr(self) -> str:
        return 'local_size=%d, alpha=%g, beta=%g, across_channels=%s' % (self.local_size, self.alpha, self.beta, self.ACROSS_CHANNELS)


# (out channels, kernel, stride, padding, groups, followed by LRN, followed by max-pool)
_CONV_TABLE = (
    (96, 11, 4, 0, 1, True, True),
    (256, 5, 1, 2, 2, True, True),
    (384, 3, 1, 1, 1, False, False),
    (384, 3, 1, 1, 2, False, False),
    (256, 3, 1, 1, 2, False, True),
)


class AlexNet(nn.Module):
    def __init__(self, num_classes: int = 1000):
        super().__init__()
        self.name = 'alexnet'
        stack: List[nn.Module] = []
        channels = 3
        for out, kernel, stride, padding, groups, norm, pool in _CONV_TABLE:
            stack += [nn.Conv2d(channels, out, kernel, stride, padding, groups=groups), nn.ReLU(inplace=True)]
            if norm:
                stack.append(LRN(local_size=5, alpha=1e-4, beta=0.75))
            if pool:
                stack.append(nn.MaxPool2d(kernel_size=3, stride=2))
            channels = out
        self.features = nn.Sequential(*stack)
        head: List[nn.Module] = []
        width = channels * 6 * 6
        for hidden in (4096, 4096):
            head += [nn.Linear(width, hidden), nn.ReLU(inplace=True), nn.Dropout()]
            width = hidden
        head.append(nn.Linear(width, num_classes))
        self.classifier = nn.Sequential(*head)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.classifier(torch.flatten(self.features(x), 1))


def alexnet(pretrained: bool = False, **kwargs) -> AlexNet:
    if pretrained:
        raise RuntimeError('pretrained weights are not available offline')
    return AlexNet(**kwargs)
