# -*- coding: utf-8 -*-
"""Model zoo and the ``--dnn`` registry.

``create_net(num_classes, dnn, **kw) -> (net, ext)`` resolves the 22 names the reference accepts
(``dl_trainer.py:45,87-135``): CIFAR ResNets, the CIFAR VGG-16-BN, GoogLeNet, Inception-v4, the
PTB LSTM, the AN4 acoustic model and the MNIST nets are defined in this package; ImageNet
ResNets / DenseNets / Inception-v3 / VGG-16 (``vgg16i``) / AlexNet come from torchvision, as in
the reference.  ``vgg19`` is listed by the reference but has no constructor branch there; here it
builds the CIFAR VGG-19-BN.  ``fuse=True`` swaps BatchNorm+ReLU pairs and LSTMs for this
package's fused CUDA modules without changing any ``state_dict`` key.
"""
from __future__ import annotations

import torch.nn as nn

from .cifar_resnet import (resnet20, resnet32, resnet44, resnet56, resnet110,  # noqa: F401
                           preresnet20, preresnet32, preresnet44, preresnet56, preresnet110,
                           resnet_mod20, resnet_mod32, resnet_mod44, resnet_mod56, resnet_mod110,
                           resnext29_8_64, resnext29_16_64, DownsampleA, DownsampleC, DownsampleD)
from .small import (MnistNet, FCN5Net, LinearRegression, LeNet, VGG, caffe_cifar, densenet100_12)  # noqa: F401
from .inception import googlenet, GoogLeNet, inceptionv4, InceptionV4  # noqa: F401
from .alexnet_lrn import AlexNet  # noqa: F401
from .cifar_resnet_tv import ResNet18, ResNet34, ResNet50, ResNet101, ResNet152, model_builder  # noqa: F401
from .lstm import lstm, repackage_hidden  # noqa: F401
from .deepspeech import DeepSpeech, create_net as LSTMAN4  # noqa: F401

_support_datasets = ['imagenet', 'cifar10', 'an4', 'ptb', 'mnist']
_support_dnns = ['resnet50', 'resnet101', 'resnet152', 'densenet121', 'densenet161', 'densenet201', 'resnet20',
                 'resnet56', 'resnet110', 'vgg19', 'vgg16', 'alexnet', 'lstman4', 'lstm', 'googlenet', 'inceptionv4',
                 'inceptionv3', 'vgg16i', 'mnistnet', 'fcn5net', 'lenet', 'lr']

_TORCHVISION = {'resnet50': 'resnet50', 'resnet101': 'resnet101', 'resnet152': 'resnet152',
                'densenet121': 'densenet121', 'densenet161': 'densenet161', 'densenet201': 'densenet201',
                'inceptionv3': 'inception_v3', 'vgg16i': 'vgg16', 'alexnet': 'alexnet',
                'resnet18': 'resnet18', 'resnet34': 'resnet34'}


def _torchvision_model(key: str, num_classes: int):
    import torchvision
    ctor = getattr(torchvision.models, _TORCHVISION[key])
    kwargs = {'num_classes': num_classes}
    if key == 'inceptionv3':
        kwargs.update(init_weights=True)
    if key == 'alexnet':
        kwargs = {}                      # the reference builds the 1000-class AlexNet unconditionally
    net = ctor(**kwargs)
    net.name = key
    return net


# ImageNet ResNets under the names reference models/__init__.py:24 exports
def resnet18(num_classes=1000):
    return _torchvision_model('resnet18', num_classes)


def resnet34(num_classes=1000):
    return _torchvision_model('resnet34', num_classes)


def resnet50(num_classes=1000):
    return _torchvision_model('resnet50', num_classes)


def resnet101(num_classes=1000):
    return _torchvision_model('resnet101', num_classes)


def resnet152(num_classes=1000):
    return _torchvision_model('resnet152', num_classes)


def create_net(num_classes, dnn='resnet20', fuse=False, channels_last=False, **kwargs):
    """Build the network registered under ``dnn``; returns ``(net, ext)`` where ``ext`` carries
    model-specific extras (audio configuration for ``lstman4``), else ``None``."""
    ext = None
    if dnn in ('resnet20', 'resnet32', 'resnet44', 'resnet56', 'resnet110'):
        net = globals()[dnn](num_classes=num_classes)
    elif dnn in _TORCHVISION:
        net = _torchvision_model(dnn, num_classes)
    elif dnn == 'inceptionv4':
        net = inceptionv4(num_classes=num_classes)
    elif dnn == 'googlenet':
        net = googlenet()
    elif dnn == 'mnistnet':
        net = MnistNet()
    elif dnn == 'fcn5net':
        net = FCN5Net()
    elif dnn == 'lenet':
        net = LeNet()
    elif dnn == 'lr':
        net = LinearRegression()
    elif dnn in ('vgg16', 'vgg19'):
        net = VGG(dnn.upper())
    elif dnn == 'lstman4':
        net, ext = LSTMAN4(datapath=kwargs.get('datapath'))
    elif dnn == 'lstm':
        net = lstm(vocab_size=kwargs['vocab_size'], batch_size=kwargs['batch_size'],
                   num_steps=kwargs.get('num_steps', 35), fused=kwargs.get('fused_lstm', False))
    else:
        raise ValueError('Unsupport neural network %s' % dnn)
    if not hasattr(net, 'name'):
        net.name = dnn
    if fuse and dnn not in ('lstm',):
        from .fuse import fuse_model
        net = fuse_model(net)
    from .. import settings as _settings
    if fuse and not _settings.FP16:
        # large fully-connected layers: exchange activations instead of all-reducing the weight gradient
        # (fp32 / TF32 kernels; under FP16 autocast the layers stay torch.nn.Linear)
        from ..ops.wgrad import convert_large_linears
        convert_large_linears(net)
    if channels_last:
        import torch
        net = net.to(memory_format=torch.channels_last)
    return net, ext
