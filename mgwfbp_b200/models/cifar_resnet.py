# -*- coding: utf-8 -*-
"""CIFAR-style residual networks (3 stages, 16/32/64 channels).

Architectures and parameter names (``conv_1_3x3``, ``bn_1``, ``stage_k.i.conv_a`` ...) match
reference ``models/resnet.py:9-147`` (post-activation), ``models/preresnet.py`` (pre-activation),
``models/resnet_mod.py`` (post-activation returning intermediate features) and
``models/resnext.py`` so that checkpoints are interchangeable.  The shortcut of a stride-2 stage
is the parameter-free "option A": sub-sample by 2 and pad the new channels with zeros
(``models/res_utils.py:4-13``).
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F


class DownsampleA(nn.Module):
    """Stride-2 spatial sub-sampling followed by doubling the channels with zeros."""

    def __init__(self, n_in: int, n_out: int, stride: int):
        super().__init__()
        if stride != 2:
            raise ValueError('option-A shortcut only exists for stride 2')
        self.avg = nn.AvgPool2d(kernel_size=1, stride=stride)

    def forward(self, x):
        x = self.avg(x)
        return torch.cat((x, torch.zeros_like(x)), 1)


class DownsampleC(nn.Module):
    def __init__(self, n_in: int, n_out: int, stride: int):
        super().__init__()
        self.conv = nn.Conv2d(n_in, n_out, kernel_size=1, stride=stride, padding=0, bias=False)

    def forward(self, x):
        return self.conv(x)


class DownsampleD(nn.Module):
    def __init__(self, n_in: int, n_out: int, stride: int):
        super().__init__()
        self.conv = nn.Conv2d(n_in, n_out, kernel_size=2, stride=stride, padding=0, bias=False)
        self.bn = nn.BatchNorm2d(n_out)

    def forward(self, x):
        return self.bn(self.conv(x))


def _conv3x3(cin, cout, stride=1):
    return nn.Conv2d(cin, cout, kernel_size=3, stride=stride, padding=1, bias=False)


class ResNetBasicblock(nn.Module):
    expansion = 1

    def __init__(self, inplanes, planes, stride=1, downsample=None):
        super().__init__()
        self.conv_a = _conv3x3(inplanes, planes, stride)
        self.bn_a = nn.BatchNorm2d(planes)
        self.conv_b = _conv3x3(planes, planes)
        self.bn_b = nn.BatchNorm2d(planes)
        self.downsample = downsample

    def forward(self, x):
        out = F.relu(self.bn_a(self.conv_a(x)), inplace=True)
        out = self.bn_b(self.conv_b(out))
        shortcut = x if self.downsample is None else self.downsample(x)
        return F.relu(shortcut + out, inplace=True)


class PreActBasicblock(nn.Module):
    expansion = 1

    def __init__(self, inplanes, planes, stride, downsample, kind):
        super().__init__()
        if kind not in ('both_preact', 'normal'):
            raise ValueError('unknown block type %s' % kind)
        self.Type = kind
        self.bn_a = nn.BatchNorm2d(inplanes)
        self.conv_a = _conv3x3(inplanes, planes, stride)
        self.bn_b = nn.BatchNorm2d(planes)
        self.conv_b = _conv3x3(planes, planes)
        self.relu = nn.ReLU(inplace=True)
        self.downsample = downsample

    def forward(self, x):
        pre = self.relu(self.bn_a(x))
        shortcut = pre if self.Type == 'both_preact' else x
        out = self.conv_b(self.relu(self.bn_b(self.conv_a(pre))))
        if self.downsample is not None:
            shortcut = self.downsample(shortcut)
        return shortcut + out


def _init_cifar(module: nn.Module, conv_uniform: bool) -> None:
    for m in module.modules():
        if isinstance(m, nn.Conv2d):
            n = m.kernel_size[0] * m.kernel_size[1] * m.out_channels
            if conv_uniform:
                bound = 1.0 / math.sqrt(n)
                nn.init.uniform_(m.weight, -bound, bound)
            else:
                nn.init.normal_(m.weight, 0.0, math.sqrt(2.0 / n))
        elif isinstance(m, nn.BatchNorm2d):
            nn.init.ones_(m.weight)
            nn.init.zeros_(m.bias)
        elif isinstance(m, nn.Linear):
            nn.init.kaiming_normal_(m.weight)
            nn.init.zeros_(m.bias)


class CifarResNet(nn.Module):
    """Post-activation ResNet-(6n+2) for 32x32 inputs."""

    def __init__(self, block, depth: int, num_classes: int, conv_uniform: bool = True):
        super().__init__()
        if (depth - 2) % 6 != 0:
            raise ValueError('depth should be one of 20, 32, 44, 56, 110')
        n = (depth - 2) // 6
        self.name = 'resnet%d' % depth
        self.num_classes = num_classes
        self.conv_1_3x3 = _conv3x3(3, 16)
        self.bn_1 = nn.BatchNorm2d(16)
        self.inplanes = 16
        self.stage_1 = self._make_stage(block, 16, n, 1)
        self.stage_2 = self._make_stage(block, 32, n, 2)
        self.stage_3 = self._make_stage(block, 64, n, 2)
        self.avgpool = nn.AvgPool2d(8)
        self.classifier = nn.Linear(64 * block.expansion, num_classes)
        _init_cifar(self, conv_uniform)

    def _make_stage(self, block, planes, blocks, stride):
        down = None
        if stride != 1 or self.inplanes != planes * block.expansion:
            down = DownsampleA(self.inplanes, planes * block.expansion, stride)
        layers = [block(self.inplanes, planes, stride, down)]
        self.inplanes = planes * block.expansion
        layers += [block(self.inplanes, planes) for _ in range(1, blocks)]
        return nn.Sequential(*layers)

    def forward(self, x):
        x = F.relu(self.bn_1(self.conv_1_3x3(x)), inplace=True)
        x = self.stage_3(self.stage_2(self.stage_1(x)))
        x = self.avgpool(x)
        return self.classifier(x.view(x.size(0), -1))


class CifarResNetMod(CifarResNet):
    """Same network; ``forward_features`` additionally returns every block's two BN outputs
    (the list-in/list-out mode of reference ``models/resnet_mod.py``)."""

    def __init__(self, block, depth, num_classes):
        super().__init__(block, depth, num_classes, conv_uniform=False)
        self.name = 'resnet_mod%d' % depth

    def forward_features(self, x):
        feats = []
        x = F.relu(self.bn_1(self.conv_1_3x3(x)), inplace=True)
        for stage in (self.stage_1, self.stage_2, self.stage_3):
            for blk in stage:
                bn_a = blk.bn_a(blk.conv_a(x))
                bn_b = blk.bn_b(blk.conv_b(F.relu(bn_a)))
                shortcut = x if blk.downsample is None else blk.downsample(x)
                x = F.relu(shortcut + bn_b)
                feats += [bn_a, bn_b]
        x = self.avgpool(x)
        return self.classifier(x.view(x.size(0), -1)), feats

    def forward(self, x):
        if isinstance(x, list):
            if len(x) != 1:
                raise ValueError('The length of inputs must be one vs %d' % len(x))
            return self.forward_features(x[0])
        return super().forward(x)


class CifarPreResNet(nn.Module):
    def __init__(self, block, depth: int, num_classes: int):
        super().__init__()
        if (depth - 2) % 6 != 0:
            raise ValueError('depth should be one of 20, 32, 44, 56, 110')
        n = (depth - 2) // 6
        self.name = 'preresnet%d' % depth
        self.num_classes = num_classes
        self.conv_3x3 = _conv3x3(3, 16)
        self.inplanes = 16
        self.stage_1 = self._make_stage(block, 16, n, 1)
        self.stage_2 = self._make_stage(block, 32, n, 2)
        self.stage_3 = self._make_stage(block, 64, n, 2)
        self.lastact = nn.Sequential(nn.BatchNorm2d(64 * block.expansion), nn.ReLU(inplace=True))
        self.avgpool = nn.AvgPool2d(8)
        self.classifier = nn.Linear(64 * block.expansion, num_classes)
        _init_cifar(self, conv_uniform=False)

    def _make_stage(self, block, planes, blocks, stride):
        down = None
        if stride != 1 or self.inplanes != planes * block.expansion:
            down = DownsampleA(self.inplanes, planes * block.expansion, stride)
        layers = [block(self.inplanes, planes, stride, down, 'both_preact')]
        self.inplanes = planes * block.expansion
        layers += [block(self.inplanes, planes, 1, None, 'normal') for _ in range(1, blocks)]
        return nn.Sequential(*layers)

    def forward(self, x):
        x = self.stage_3(self.stage_2(self.stage_1(self.conv_3x3(x))))
        x = self.avgpool(self.lastact(x))
        return self.classifier(x.view(x.size(0), -1))


class ResNeXtBottleneck(nn.Module):
    """ResNeXt type-C bottleneck: 1x1 reduce, grouped 3x3, 1x1 expand."""
    expansion = 4

    def __init__(self, inplanes, planes, cardinality, base_width, stride=1, downsample=None):
        super().__init__()
        width = int(math.floor(planes * (base_width / 64.0))) * cardinality
        self.conv_reduce = nn.Conv2d(inplanes, width, 1, 1, 0, bias=False)
        self.bn_reduce = nn.BatchNorm2d(width)
        self.conv_conv = nn.Conv2d(width, width, 3, stride, 1, groups=cardinality, bias=False)
        self.bn = nn.BatchNorm2d(width)
        self.conv_expand = nn.Conv2d(width, planes * 4, 1, 1, 0, bias=False)
        self.bn_expand = nn.BatchNorm2d(planes * 4)
        self.downsample = downsample

    def forward(self, x):
        out = F.relu(self.bn_reduce(self.conv_reduce(x)), inplace=True)
        out = F.relu(self.bn(self.conv_conv(out)), inplace=True)
        out = self.bn_expand(self.conv_expand(out))
        shortcut = x if self.downsample is None else self.downsample(x)
        return F.relu(shortcut + out, inplace=True)


class CifarResNeXt(nn.Module):
    def __init__(self, block, depth, cardinality, base_width, num_classes):
        super().__init__()
        if (depth - 2) % 9 != 0:
            raise ValueError('depth should be one of 29, 38, 47, 56, 101')
        n = (depth - 2) // 9
        self.cardinality, self.base_width, self.num_classes = cardinality, base_width, num_classes
        self.conv_1_3x3 = nn.Conv2d(3, 64, 3, 1, 1, bias=False)
        self.bn_1 = nn.BatchNorm2d(64)
        self.inplanes = 64
        self.stage_1 = self._make_stage(block, 64, n, 1)
        self.stage_2 = self._make_stage(block, 128, n, 2)
        self.stage_3 = self._make_stage(block, 256, n, 2)
        self.avgpool = nn.AvgPool2d(8)
        self.classifier = nn.Linear(256 * block.expansion, num_classes)
        _init_cifar(self, conv_uniform=False)

    def _make_stage(self, block, planes, blocks, stride):
        down = None
        if stride != 1 or self.inplanes != planes * block.expansion:
            down = nn.Sequential(nn.Conv2d(self.inplanes, planes * block.expansion, 1, stride, bias=False),
                                 nn.BatchNorm2d(planes * block.expansion))
        layers = [block(self.inplanes, planes, self.cardinality, self.base_width, stride, down)]
        self.inplanes = planes * block.expansion
        layers += [block(self.inplanes, planes, self.cardinality, self.base_width) for _ in range(1, blocks)]
        return nn.Sequential(*layers)

    def forward(self, x):
        x = F.relu(self.bn_1(self.conv_1_3x3(x)), inplace=True)
        x = self.avgpool(self.stage_3(self.stage_2(self.stage_1(x))))
        return self.classifier(x.view(x.size(0), -1))


def _factory(cls, block, depth, **extra):
    def build(num_classes=10):
        return cls(block, depth, num_classes=num_classes, **extra)
    build.__doc__ = '%s, depth %d, for CIFAR-10 by default.' % (cls.__name__, depth)
    return build


resnet20, resnet32, resnet44, resnet56, resnet110 = (
    _factory(CifarResNet, ResNetBasicblock, d) for d in (20, 32, 44, 56, 110))
resnet_mod20, resnet_mod32, resnet_mod44, resnet_mod56, resnet_mod110 = (
    _factory(CifarResNetMod, ResNetBasicblock, d) for d in (20, 32, 44, 56, 110))
preresnet20, preresnet32, preresnet44, preresnet56, preresnet110 = (
    _factory(CifarPreResNet, PreActBasicblock, d) for d in (20, 32, 44, 56, 110))


def resnext29_16_64(num_classes=10):
    return CifarResNeXt(ResNeXtBottleneck, 29, 16, 64, num_classes)


def resnext29_8_64(num_classes=10):
    return CifarResNeXt(ResNeXtBottleneck, 29, 8, 64, num_classes)
