# -*- coding: utf-8 -*-
"""GoogLeNet (BatchNorm-free variant) and Inception-v4.

Topologies and ``state_dict`` keys follow reference ``models/googlenet.py:53-233`` (the
torchvision GoogLeNet with its BatchNorm layers disabled, auxiliary heads off, truncated-normal
initialisation) and ``models/inceptionv4.py:35-337`` (conv + BN(eps=1e-3) + ReLU units).  Both
are written table-first: each mixed block is a list of branches, each branch a list of
convolution specs.
"""
from __future__ import annotations

from typing import Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F


# --------------------------------------------------------------------------- GoogLeNet
class _ConvReLU(nn.Module):
    """``conv`` (no bias) followed by ReLU; the reference comments its BatchNorm out."""

    def __init__(self, cin, cout, **kw):
        super().__init__()
        self.conv = nn.Conv2d(cin, cout, bias=False, **kw)

    def forward(self, x):
        return F.relu(self.conv(x), inplace=True)


class Inception(nn.Module):
    def __init__(self, cin, c1, c3r, c3, c5r, c5, cp):
        super().__init__()
        self.branch1 = _ConvReLU(cin, c1, kernel_size=1)
        self.branch2 = nn.Sequential(_ConvReLU(cin, c3r, kernel_size=1), _ConvReLU(c3r, c3, kernel_size=3, padding=1))
        # the "5x5" branch uses a 3x3 kernel, as torchvision does
        self.branch3 = nn.Sequential(_ConvReLU(cin, c5r, kernel_size=1), _ConvReLU(c5r, c5, kernel_size=3, padding=1))
        self.branch4 = nn.Sequential(nn.MaxPool2d(kernel_size=3, stride=1, padding=1, ceil_mode=True),
                                     _ConvReLU(cin, cp, kernel_size=1))

    def forward(self, x):
        return torch.cat([self.branch1(x), self.branch2(x), self.branch3(x), self.branch4(x)], 1)


class InceptionAux(nn.Module):
    def __init__(self, cin, num_classes):
        super().__init__()
        self.conv = _ConvReLU(cin, 128, kernel_size=1)
        self.fc1 = nn.Linear(2048, 1024)
        self.fc2 = nn.Linear(1024, num_classes)

    def forward(self, x):
        x = self.conv(F.adaptive_avg_pool2d(x, (4, 4))).flatten(1)
        x = F.dropout(F.relu(self.fc1(x), inplace=True), 0.7, training=self.training)
        return self.fc2(x)


_GOOGLENET_BLOCKS = (
    ('inception3a', (192, 64, 96, 128, 16, 32, 32)), ('inception3b', (256, 128, 128, 192, 32, 96, 64)),
    ('maxpool3', None),
    ('inception4a', (480, 192, 96, 208, 16, 48, 64)), ('inception4b', (512, 160, 112, 224, 24, 64, 64)),
    ('inception4c', (512, 128, 128, 256, 24, 64, 64)), ('inception4d', (512, 112, 144, 288, 32, 64, 64)),
    ('inception4e', (528, 256, 160, 320, 32, 128, 128)),
    ('maxpool4', None),
    ('inception5a', (832, 256, 160, 320, 32, 128, 128)), ('inception5b', (832, 384, 192, 384, 48, 128, 128)),
)


class GoogLeNet(nn.Module):
    def __init__(self, num_classes=1000, aux_logits=False, transform_input=False, init_weights=True):
        super().__init__()
        self.name = 'googlenet'
        self.aux_logits = aux_logits
        self.transform_input = transform_input
        self.conv1 = _ConvReLU(3, 64, kernel_size=7, stride=2, padding=3)
        self.maxpool1 = nn.MaxPool2d(3, stride=2, ceil_mode=True)
        self.conv2 = _ConvReLU(64, 64, kernel_size=1)
        self.conv3 = _ConvReLU(64, 192, kernel_size=3, padding=1)
        self.maxpool2 = nn.MaxPool2d(3, stride=2, ceil_mode=True)
        for name, spec in _GOOGLENET_BLOCKS:
            if spec is None:
                k = 3 if name == 'maxpool3' else 2
                setattr(self, name, nn.MaxPool2d(k, stride=2, ceil_mode=True))
            else:
                setattr(self, name, Inception(*spec))
        if aux_logits:
            self.aux1 = InceptionAux(512, num_classes)
            self.aux2 = InceptionAux(528, num_classes)
        self.avgpool = nn.AdaptiveAvgPool2d((1, 1))
        self.dropout = nn.Dropout(0.2)
        self.fc = nn.Linear(1024, num_classes)
        if init_weights:
            self._initialize_weights()

    def _initialize_weights(self):
        for m in self.modules():
            if isinstance(m, (nn.Conv2d, nn.Linear)):
                nn.init.trunc_normal_(m.weight, mean=0.0, std=0.01, a=-0.02, b=0.02)
            elif isinstance(m, nn.BatchNorm2d):
                nn.init.ones_(m.weight)
                nn.init.zeros_(m.bias)

    def forward(self, x):
        if self.transform_input:
            scale = x.new_tensor([0.229 / 0.5, 0.224 / 0.5, 0.225 / 0.5]).view(1, 3, 1, 1)
            shift = x.new_tensor([(0.485 - 0.5) / 0.5, (0.456 - 0.5) / 0.5, (0.406 - 0.5) / 0.5]).view(1, 3, 1, 1)
            x = x * scale + shift
        x = self.maxpool2(self.conv3(self.conv2(self.maxpool1(self.conv1(x)))))
        aux = []
        for name, _ in _GOOGLENET_BLOCKS:
            x = getattr(self, name)(x)
            if self.training and self.aux_logits and name in ('inception4a', 'inception4d'):
                aux.append((self.aux1 if name == 'inception4a' else self.aux2)(x))
        x = self.fc(self.dropout(self.avgpool(x).flatten(1)))
        if self.training and self.aux_logits:
            return x, aux[1], aux[0]
        return x


def googlenet(pretrained=False, progress=True, **kwargs):
    if pretrained:
        raise RuntimeError('pretrained weights are not available offline')
    return GoogLeNet(**kwargs)


# --------------------------------------------------------------------------- Inception-v4
class BasicConv2d(nn.Module):
    def __init__(self, cin, cout, kernel_size, stride=1, padding=0):
        super().__init__()
        self.conv = nn.Conv2d(cin, cout, kernel_size=kernel_size, stride=stride, padding=padding, bias=False)
        self.bn = nn.BatchNorm2d(cout, eps=0.001, momentum=0.1, affine=True)
        self.relu = nn.ReLU(inplace=True)

    def forward(self, x):
        return self.relu(self.bn(self.conv(x)))


def _chain(cin: int, specs: Sequence[tuple]):
    """specs: (cout, kernel, stride, padding) per conv; returns one unit or a Sequential."""
    units = []
    for cout, k, s, p in specs:
        units.append(BasicConv2d(cin, cout, kernel_size=k, stride=s, padding=p))
        cin = cout
    return units[0] if len(units) == 1 else nn.Sequential(*units)


class _Concat(nn.Module):
    """Run named branches on the same input and concatenate along channels."""
    order: Sequence[str] = ()

    def forward(self, x):
        return torch.cat([getattr(self, n)(x) for n in self.order], 1)


class Mixed_3a(_Concat):
    order = ('maxpool', 'conv')

    def __init__(self):
        super().__init__()
        self.maxpool = nn.MaxPool2d(3, stride=2)
        self.conv = BasicConv2d(64, 96, kernel_size=3, stride=2)


class Mixed_4a(_Concat):
    order = ('branch0', 'branch1')

    def __init__(self):
        super().__init__()
        self.branch0 = _chain(160, [(64, 1, 1, 0), (96, 3, 1, 0)])
        self.branch1 = _chain(160, [(64, 1, 1, 0), (64, (1, 7), 1, (0, 3)), (64, (7, 1), 1, (3, 0)), (96, 3, 1, 0)])


class Mixed_5a(_Concat):
    order = ('conv', 'maxpool')

    def __init__(self):
        super().__init__()
        self.conv = BasicConv2d(192, 192, kernel_size=3, stride=2)
        self.maxpool = nn.MaxPool2d(3, stride=2)


def _pool_proj(cin, cout):
    return nn.Sequential(nn.AvgPool2d(3, stride=1, padding=1, count_include_pad=False),
                         BasicConv2d(cin, cout, kernel_size=1, stride=1))


class Inception_A(_Concat):
    order = ('branch0', 'branch1', 'branch2', 'branch3')

    def __init__(self):
        super().__init__()
        self.branch0 = _chain(384, [(96, 1, 1, 0)])
        self.branch1 = _chain(384, [(64, 1, 1, 0), (96, 3, 1, 1)])
        self.branch2 = _chain(384, [(64, 1, 1, 0), (96, 3, 1, 1), (96, 3, 1, 1)])
        self.branch3 = _pool_proj(384, 96)


class Reduction_A(_Concat):
    order = ('branch0', 'branch1', 'branch2')

    def __init__(self):
        super().__init__()
        self.branch0 = _chain(384, [(384, 3, 2, 0)])
        self.branch1 = _chain(384, [(192, 1, 1, 0), (224, 3, 1, 1), (256, 3, 2, 0)])
        self.branch2 = nn.MaxPool2d(3, stride=2)


class Inception_B(_Concat):
    order = ('branch0', 'branch1', 'branch2', 'branch3')

    def __init__(self):
        super().__init__()
        self.branch0 = _chain(1024, [(384, 1, 1, 0)])
        self.branch1 = _chain(1024, [(192, 1, 1, 0), (224, (1, 7), 1, (0, 3)), (256, (7, 1), 1, (3, 0))])
        self.branch2 = _chain(1024, [(192, 1, 1, 0), (192, (7, 1), 1, (3, 0)), (224, (1, 7), 1, (0, 3)),
                                     (224, (7, 1), 1, (3, 0)), (256, (1, 7), 1, (0, 3))])
        self.branch3 = _pool_proj(1024, 128)


class Reduction_B(_Concat):
    order = ('branch0', 'branch1', 'branch2')

    def __init__(self):
        super().__init__()
        self.branch0 = _chain(1024, [(192, 1, 1, 0), (192, 3, 2, 0)])
        self.branch1 = _chain(1024, [(256, 1, 1, 0), (256, (1, 7), 1, (0, 3)), (320, (7, 1), 1, (3, 0)), (320, 3, 2, 0)])
        self.branch2 = nn.MaxPool2d(3, stride=2)


class Inception_C(nn.Module):
    def __init__(self):
        super().__init__()
        self.branch0 = BasicConv2d(1536, 256, kernel_size=1, stride=1)
        self.branch1_0 = BasicConv2d(1536, 384, kernel_size=1, stride=1)
        self.branch1_1a = BasicConv2d(384, 256, kernel_size=(1, 3), stride=1, padding=(0, 1))
        self.branch1_1b = BasicConv2d(384, 256, kernel_size=(3, 1), stride=1, padding=(1, 0))
        self.branch2_0 = BasicConv2d(1536, 384, kernel_size=1, stride=1)
        self.branch2_1 = BasicConv2d(384, 448, kernel_size=(3, 1), stride=1, padding=(1, 0))
        self.branch2_2 = BasicConv2d(448, 512, kernel_size=(1, 3), stride=1, padding=(0, 1))
        self.branch2_3a = BasicConv2d(512, 256, kernel_size=(1, 3), stride=1, padding=(0, 1))
        self.branch2_3b = BasicConv2d(512, 256, kernel_size=(3, 1), stride=1, padding=(1, 0))
        self.branch3 = _pool_proj(1536, 256)

    def forward(self, x):
        b1 = self.branch1_0(x)
        b2 = self.branch2_2(self.branch2_1(self.branch2_0(x)))
        return torch.cat([self.branch0(x), self.branch1_1a(b1), self.branch1_1b(b1),
                          self.branch2_3a(b2), self.branch2_3b(b2), self.branch3(x)], 1)


class InceptionV4(nn.Module):
    def __init__(self, num_classes=1001):
        super().__init__()
        self.name = 'inceptionv4'
        self.input_space, self.input_size, self.mean, self.std = None, (299, 299, 3), None, None
        stem = [BasicConv2d(3, 32, kernel_size=3, stride=2), BasicConv2d(32, 32, kernel_size=3, stride=1),
                BasicConv2d(32, 64, kernel_size=3, stride=1, padding=1), Mixed_3a(), Mixed_4a(), Mixed_5a()]
        body = ([Inception_A() for _ in range(4)] + [Reduction_A()] + [Inception_B() for _ in range(7)]
                + [Reduction_B()] + [Inception_C() for _ in range(3)])
        self.features = nn.Sequential(*(stem + body))
        self.last_linear = nn.Linear(1536, num_classes)

    def logits(self, features):
        x = F.avg_pool2d(features, kernel_size=features.shape[2])   # any input resolution
        return self.last_linear(x.flatten(1))

    def forward(self, x):
        return self.logits(self.features(x))


def inceptionv4(num_classes=1000, pretrained=None):
    if pretrained:
        raise RuntimeError('pretrained weights are not available offline')
    return InceptionV4(num_classes=num_classes)
