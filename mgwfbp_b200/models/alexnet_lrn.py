# -*- coding: utf-8 -*-
"""Original (two-tower, local-response-normalised) AlexNet.

Layer stack of reference ``models/alexnet.py:9-87``; the registry uses torchvision's AlexNet for
the ``alexnet`` key, as the reference does (``dl_trainer.py:121-123``), and this class remains
available as ``models.AlexNet``.
"""
import torch
import torch.nn as nn


class LRN(nn.Module):
    """``x / (1 + alpha * mean_{window}(x^2)) ** beta`` across channels or within a channel."""

    def __init__(self, local_size=1, alpha=1.0, beta=0.75, ACROSS_CHANNELS=True):
        super().__init__()
        self.ACROSS_CHANNELS = ACROSS_CHANNELS
        pad = int((local_size - 1.0) / 2)
        if ACROSS_CHANNELS:
            self.average = nn.AvgPool3d(kernel_size=(local_size, 1, 1), stride=1, padding=(pad, 0, 0))
        else:
            self.average = nn.AvgPool2d(kernel_size=local_size, stride=1, padding=pad)
        self.alpha, self.beta = alpha, beta

    def forward(self, x):
        sq = x.pow(2)
        mean = self.average(sq.unsqueeze(1)).squeeze(1) if self.ACROSS_CHANNELS else self.average(sq)
        return x / mean.mul(self.alpha).add(1.0).pow(self.beta)


class AlexNet(nn.Module):
    def __init__(self, num_classes=1000):
        super().__init__()
        self.name = 'alexnet'
        def lrn():
            return LRN(local_size=5, alpha=0.0001, beta=0.75)
        self.features = nn.Sequential(
            nn.Conv2d(3, 96, kernel_size=11, stride=4, padding=0), nn.ReLU(inplace=True), lrn(), nn.MaxPool2d(3, 2),
            nn.Conv2d(96, 256, kernel_size=5, padding=2, groups=2), nn.ReLU(inplace=True), lrn(), nn.MaxPool2d(3, 2),
            nn.Conv2d(256, 384, kernel_size=3, padding=1), nn.ReLU(inplace=True),
            nn.Conv2d(384, 384, kernel_size=3, padding=1, groups=2), nn.ReLU(inplace=True),
            nn.Conv2d(384, 256, kernel_size=3, padding=1, groups=2), nn.ReLU(inplace=True), nn.MaxPool2d(3, 2))
        self.classifier = nn.Sequential(
            nn.Linear(256 * 6 * 6, 4096), nn.ReLU(inplace=True), nn.Dropout(),
            nn.Linear(4096, 4096), nn.ReLU(inplace=True), nn.Dropout(), nn.Linear(4096, num_classes))

    def forward(self, x):
        return self.classifier(self.features(x).flatten(1))


def alexnet(pretrained=False, **kwargs):
    if pretrained:
        raise RuntimeError('pretrained weights are not available offline')
    return AlexNet(**kwargs)
