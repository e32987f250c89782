# -*- coding: utf-8 -*-
"""ResNet-18/34/50/101/152 for 32x32 inputs (3x3 stem, no max-pool, projection shortcuts).

Counterpart of the reference's top-level ``resnet.py``, which its registry never reaches; kept for users who
import it directly.  Parameter names match the reference's checkpoints
(``conv1, bn1, layer{1..4}.{i}.conv{k}/bn{k}/shortcut.{0,1}, linear``), the construction does not: both block types
are one class driven by a table of ``(kernel, width factor, carries the stride)`` rows, and the depth variants are
rows of ``_DEPTHS``.
"""
from __future__ import annotations

from typing import Dict, Sequence, Tuple

import torch
import torch.nn as nn

# (kernel size, output width as a multiple of `planes`, whether this convolution carries the block's stride)
_BASIC: Tuple[Tuple[int, int, bool], ...] = ((3, 1, True), (3, 1, False))
_BOTTLENECK: Tuple[Tuple[int, int, bool], ...] = ((1, 1, False), (3, 1, True), (1, 4, False))


class _ResidualUnit(nn.Module):
    """conv-bn(-relu) chain described by ``plan`` plus an identity or 1x1-projection shortcut."""
    plan: Tuple[Tuple[int, int, bool], ...] = ()
    expansion = 1

    def __init__(self, in_planes: int, planes: int, stride: int = 1):
        super().__init__()
        width = in_planes
        for idx, (kernel, factor, strided) in enumerate(self.plan, start=1):
            out_width = planes * factor
            setattr(self, 'conv%d' % idx, nn.Conv2d(width, out_width, kernel, stride if strided else 1, kernel // 2, bias=False))
            setattr(self, 'bn%d' % idx, nn.BatchNorm2d(out_width))
            width = out_width
        project = stride != 1 or in_planes != width
        self.shortcut = nn.Sequential(nn.Conv2d(in_planes, width, 1, stride, bias=False), nn.BatchNorm2d(width)) if project \
            else nn.Sequential()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        out = x
        last = len(self.plan)
        for idx in range(1, last + 1):
            out = getattr(self, 'bn%d' % idx)(getattr(self, 'conv%d' % idx)(out))
            if idx < last:
                out = torch.relu(out)
        return torch.relu(out + self.shortcut(x))


class BasicBlock(_ResidualUnit):
    plan = _BASIC
    expansion = 1


class Bottleneck(_ResidualUnit):
    plan = _BOTTLENECK
    expansion = 4


class ResNet(nn.Module):
    STAGE_WIDTHS = (64, 128, 256, 512)

    def __init__(self, block, num_blocks: Sequence[int], num_classes: int = 10):
        super().__init__()
        self.conv1 = nn.Conv2d(3, self.STAGE_WIDTHS[0], 3, 1, 1, bias=False)
        self.bn1 = nn.BatchNorm2d(self.STAGE_WIDTHS[0])
        width = self.STAGE_WIDTHS[0]
        for stage, (planes, depth) in enumerate(zip(self.STAGE_WIDTHS, num_blocks), start=1):
            units = []
            for i in range(depth):
                units.append(block(width, planes, 2 if (i == 0 and stage > 1) else 1))
                width = planes * block.expansion
            setattr(self, 'layer%d' % stage, nn.Sequential(*units))
        self.linear = nn.Linear(width, num_classes)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        out = torch.relu(self.bn1(self.conv1(x)))
        for stage in range(1, len(self.STAGE_WIDTHS) + 1):
            out = getattr(self, 'layer%d' % stage)(out)
        return self.linear(nn.functional.avg_pool2d(out, 4).flatten(1))


_DEPTHS: Dict[str, Tuple[type, Tuple[int, int, int, int]]] = {
    'resnet18c': (BasicBlock, (2, 2, 2, 2)),
    'resnet34c': (BasicBlock, (3, 4, 6, 3)),
    'resnet50c': (Bottleneck, (3, 4, 6, 3)),
    'resnet101c': (Bottleneck, (3, 4, 23, 3)),
    'resnet152c': (Bottleneck, (3, 8, 36, 3)),
}


def model_builder(dnn: str, num_classes: int = 10) -> ResNet:
    """Name -> network of this file (the reference's ``model_builder.py`` is an empty stub)."""
    if dnn not in _DEPTHS:
        raise ValueError('unknown network %s' % dnn)
    block, depths = _DEPTHS[dnn]
    return ResNet(block, depths, num_classes)


def ResNet18():
    return model_builder('resnet18c')


def ResNet34():
    return model_builder('resnet34c')


def ResNet50():
    return model_builder('resnet50c')


def ResNet101():
    return model_builder('resnet101c')


def ResNet152():
    return model_builder('resnet152c')
