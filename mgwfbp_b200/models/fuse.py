# -*- coding: utf-8 -*-
"""Swap BatchNorm(+ReLU)(+residual add) patterns for the fused CUDA modules, keeping every
parameter, buffer and ``state_dict`` key where it was.

* any ``nn.Sequential`` containing ``BatchNorm2d`` directly followed by ``ReLU``: the BatchNorm
  becomes ``FusedBatchNorm2d(fused_relu=True)`` and the ReLU an ``Identity`` (indices unchanged);
* known block classes get a forward that calls the fused modules explicitly: torchvision
  ``Bottleneck`` / ``BasicBlock`` / ResNet stem, torchvision DenseNet layers and transitions,
  Inception ``BasicConv2d`` units, this package's CIFAR blocks;
* every remaining ``BatchNorm2d`` / ``BatchNorm1d`` is swapped for its fused subclass without ReLU.

Class swaps are done in place (``module.__class__ = ...``), so optimizers, hooks and checkpoints
that reference the original modules stay valid.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops.bn_relu import FusedBatchNorm1d, FusedBatchNorm2d, bn_relu_maxpool
from ..ops.stem import convert_stem


def _to_fused(bn: nn.Module, relu: bool) -> nn.Module:
    if isinstance(bn, (FusedBatchNorm2d, FusedBatchNorm1d)):
        bn.fused_relu = bn.fused_relu or relu
        return bn
    if type(bn) is nn.BatchNorm2d:
        bn.__class__ = FusedBatchNorm2d
    elif type(bn) is nn.BatchNorm1d:
        bn.__class__ = FusedBatchNorm1d
    else:
        return bn
    bn.fused_relu = relu
    return bn


# ---- forwards for known blocks ------------------------------------------------------------------
def _split(x):
    """A block receives either one tensor or the previous block's (main, shortcut) pair of handles."""
    return x if isinstance(x, tuple) else (x, x)


def _tv_bottleneck_forward(self, x):
    x_main, x_id = _split(x)
    out = self.bn1(self.conv1(x_main))
    out = self.bn2(self.conv2(out))
    identity = x_id if self.downsample is None else self.downsample(x_id)
    return self.bn3(self.conv3(out), identity, dual=True)        # (output, same output) for the next block


def _tv_basicblock_forward(self, x):
    x_main, x_id = _split(x)
    out = self.bn1(self.conv1(x_main))
    identity = x_id if self.downsample is None else self.downsample(x_id)
    return self.bn2(self.conv2(out), identity, dual=True)


def _tv_resnet_forward_impl(self, x):
    x = bn_relu_maxpool(self.bn1, self.maxpool, self.conv1(x))       # stem: BN + ReLU + pool in two passes over x
    x = self.layer4(self.layer3(self.layer2(self.layer1(x))))
    x = x[0] if isinstance(x, tuple) else x
    return self.fc(torch.flatten(self.avgpool(x), 1))


def _tv_denselayer_forward(self, input):
    prev = [input] if torch.is_tensor(input) else input
    x = torch.cat(prev, 1)
    out = self.conv1(self.norm1(x))
    out = self.conv2(self.norm2(out))
    if self.drop_rate > 0:
        out = F.dropout(out, p=self.drop_rate, training=self.training)
    return out


def _tv_densenet_forward(self, x):
    f = self.features
    out = bn_relu_maxpool(f.norm0, f.pool0, f.conv0(x))            # stem: BN + ReLU + pool fused
    for name, module in f.named_children():
        if name not in ('conv0', 'norm0', 'relu0', 'pool0'):
            out = module(out)                                      # norm5 carries the final ReLU
    out = torch.flatten(F.adaptive_avg_pool2d(out, (1, 1)), 1)
    return self.classifier(out)


def _basicconv_forward(self, x):
    return self.bn(self.conv(x))


def _cifar_block_forward(self, x):
    x_main, x_id = _split(x)
    out = self.bn_a(self.conv_a(x_main))
    shortcut = x_id if self.downsample is None else self.downsample(x_id)
    return self.bn_b(self.conv_b(out), shortcut, dual=True)


def _cifar_resnet_forward(self, x):
    x = self.bn_1(self.conv_1_3x3(x))
    x = self.stage_3(self.stage_2(self.stage_1(x)))
    x = x[0] if isinstance(x, tuple) else x
    x = self.avgpool(x)
    return self.classifier(x.reshape(x.size(0), -1))


_bound_classes = {}


def _bind(module, fn):
    """Give ``module`` the forward ``fn`` by moving it to a subclass of its class that defines it.  (An instance
    attribute ``module.forward = MethodType(fn, module)`` would be copied by ``nn.DataParallel``'s replication still bound
    to the original module, so every replica would run on the original's parameters.)"""
    base = type(module)
    if base.__dict__.get('_mgw_bound_forward') is fn:
        return
    key = (base, fn)
    cls = _bound_classes.get(key)
    if cls is None:
        cls = type(base.__name__, (base,), {'forward': fn, '_mgw_bound_forward': fn, '__module__': base.__module__})
        _bound_classes[key] = cls
    module.__class__ = cls


def fuse_model(net: nn.Module) -> nn.Module:
    try:
        import torchvision.models as tvm
        from torchvision.models.resnet import Bottleneck, BasicBlock, ResNet
        from torchvision.models.densenet import DenseNet, _DenseLayer, _Transition
        from torchvision.models.inception import BasicConv2d as TvBasicConv2d
    except Exception:  # pragma: no cover - torchvision is optional
        Bottleneck = BasicBlock = ResNet = DenseNet = _DenseLayer = _Transition = TvBasicConv2d = ()
    from .cifar_resnet import CifarResNet, CifarResNetMod, ResNetBasicblock
    from .inception import BasicConv2d as V4BasicConv2d

    for m in list(net.modules()):
        if isinstance(m, nn.Sequential):
            names = list(m._modules.keys())
            for a, b in zip(names, names[1:]):
                if type(m._modules[a]) in (nn.BatchNorm2d, FusedBatchNorm2d) and type(m._modules[b]) is nn.ReLU:
                    _to_fused(m._modules[a], relu=True)
                    m._modules[b] = nn.Identity()
        if Bottleneck and isinstance(m, Bottleneck):
            _to_fused(m.bn1, True), _to_fused(m.bn2, True), _to_fused(m.bn3, True)
            _bind(m, _tv_bottleneck_forward)
        elif BasicBlock and isinstance(m, BasicBlock):
            _to_fused(m.bn1, True), _to_fused(m.bn2, True)
            _bind(m, _tv_basicblock_forward)
        elif ResNet and isinstance(m, ResNet):
            _to_fused(m.bn1, True)
            m.conv1 = convert_stem(m.conv1)          # 7x7 / stride 2 on 3 channels as 4x4 on the space-to-depth input
            _bind(m, _tv_resnet_forward_impl)
        elif _DenseLayer and isinstance(m, _DenseLayer) and not m.memory_efficient:
            _to_fused(m.norm1, True), _to_fused(m.norm2, True)
            _bind(m, _tv_denselayer_forward)
        elif DenseNet and isinstance(m, DenseNet):
            _to_fused(m.features.norm0, True)
            m.features.conv0 = convert_stem(m.features.conv0)
            m.features.relu0 = nn.Identity()
            _to_fused(m.features.norm5, True)
            _bind(m, _tv_densenet_forward)
        elif (TvBasicConv2d and isinstance(m, TvBasicConv2d)) or isinstance(m, V4BasicConv2d):
            _to_fused(m.bn, True)
            _bind(m, _basicconv_forward)
        elif isinstance(m, ResNetBasicblock):
            _to_fused(m.bn_a, True), _to_fused(m.bn_b, True)
            _bind(m, _cifar_block_forward)
        elif isinstance(m, CifarResNet) and not isinstance(m, CifarResNetMod):
            _to_fused(m.bn_1, True)
            _bind(m, _cifar_resnet_forward)
    for m in net.modules():
        if type(m) in (nn.BatchNorm2d, nn.BatchNorm1d):
            _to_fused(m, relu=False)
    from .dense_block import fuse_dense_blocks
    fuse_dense_blocks(net)            # one buffer per dense block: L gradient additions instead of L (L - 1) / 2
    return net
