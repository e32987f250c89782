# -*- coding: utf-8 -*-
"""Small MNIST / CIFAR networks.

``MnistNet`` (reference ``dl_trainer.py:65-82``), ``FCN5Net`` and ``LinearRegression``
(``models/fcn.py:9-35``), ``LeNet`` (``models/lenet.py:5-24``), the CIFAR VGG-BN family
(``models/vgg.py:14-38``), ``CifarCaffeNet`` (``models/caffe_cifar.py``) and the CIFAR DenseNet
(``models/densenet.py``).  Parameter names follow the reference so checkpoints load either way.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F


class MnistNet(nn.Module):
    def __init__(self):
        super().__init__()
        self.conv1 = nn.Conv2d(1, 10, kernel_size=5)
        self.conv2 = nn.Conv2d(10, 20, kernel_size=5)
        self.conv2_drop = nn.Dropout2d()
        self.fc1 = nn.Linear(320, 50)
        self.fc2 = nn.Linear(50, 10)
        self.name = 'mnistnet'

    def forward(self, x):
        x = F.relu(F.max_pool2d(self.conv1(x), 2))
        x = F.relu(F.max_pool2d(self.conv2_drop(self.conv2(x)), 2))
        x = F.relu(self.fc1(x.flatten(1)))
        x = F.dropout(x, training=self.training)
        return self.fc2(x)


class FCN5Net(nn.Module):
    def __init__(self, sparse=False, sparsity=None):
        super().__init__()
        self.fc1 = nn.Linear(28 * 28, 200)
        self.fc2 = nn.Linear(200, 200)
        self.fc3 = nn.Linear(200, 10)
        self.name = 'fcn5net'

    def forward(self, x):
        x = x.reshape(-1, 28 * 28)
        return self.fc3(F.relu(self.fc2(F.relu(self.fc1(x)))))


class LinearRegression(nn.Module):
    def __init__(self):
        super().__init__()
        self.fc1 = nn.Linear(28 * 28, 10)
        self.name = 'lr'

    def forward(self, x):
        return self.fc1(x.reshape(-1, 28 * 28))


class LeNet(nn.Module):
    """LeNet-5 on 32x32 single-channel inputs."""

    def __init__(self):
        super().__init__()
        self.conv1 = nn.Conv2d(1, 6, 5)
        self.conv2 = nn.Conv2d(6, 16, 5)
        self.fc1 = nn.Linear(16 * 5 * 5, 120)
        self.fc2 = nn.Linear(120, 84)
        self.fc3 = nn.Linear(84, 10)
        self.name = 'lenet'

    def forward(self, x):
        x = F.max_pool2d(F.relu(self.conv1(x)), 2)
        x = F.max_pool2d(F.relu(self.conv2(x)), 2)
        x = x.flatten(1)
        return self.fc3(F.relu(self.fc2(F.relu(self.fc1(x)))))


VGG_CFG = {
    'VGG11': [64, 'M', 128, 'M', 256, 256, 'M', 512, 512, 'M', 512, 512, 'M'],
    'VGG13': [64, 64, 'M', 128, 128, 'M', 256, 256, 'M', 512, 512, 'M', 512, 512, 'M'],
    'VGG16': [64, 64, 'M', 128, 128, 'M', 256, 256, 256, 'M', 512, 512, 512, 'M', 512, 512, 512, 'M'],
    'VGG19': [64, 64, 'M', 128, 128, 'M', 256, 256, 256, 256, 'M', 512, 512, 512, 512, 'M', 512, 512, 512, 512, 'M'],
}


class VGG(nn.Module):
    """VGG with BatchNorm for 32x32 inputs and a single 512->10 classifier."""

    def __init__(self, vgg_name: str, num_classes: int = 10):
        super().__init__()
        self.name = vgg_name.lower()
        layers, cin = [], 3
        for item in VGG_CFG[vgg_name]:
            if item == 'M':
                layers.append(nn.MaxPool2d(kernel_size=2, stride=2))
            else:
                layers += [nn.Conv2d(cin, item, kernel_size=3, padding=1), nn.BatchNorm2d(item), nn.ReLU(inplace=True)]
                cin = item
        layers.append(nn.AvgPool2d(kernel_size=1, stride=1))
        self.features = nn.Sequential(*layers)
        self.fc = nn.Linear(512, num_classes)

    def forward(self, x):
        return self.fc(self.features(x).flatten(1))


class CifarCaffeNet(nn.Module):
    def __init__(self, num_classes: int):
        super().__init__()
        self.num_classes = num_classes
        self.block_1 = nn.Sequential(nn.Conv2d(3, 32, 3, 1, 1), nn.MaxPool2d(3, 2), nn.ReLU(), nn.BatchNorm2d(32))
        self.block_2 = nn.Sequential(nn.Conv2d(32, 32, 3, 1, 1), nn.Conv2d(32, 64, 3, 1, 1), nn.ReLU(),
                                     nn.AvgPool2d(3, 2), nn.BatchNorm2d(64))
        self.block_3 = nn.Sequential(nn.Conv2d(64, 64, 3, 1, 1), nn.Conv2d(64, 128, 3, 1, 1), nn.ReLU(),
                                     nn.AvgPool2d(3, 2), nn.BatchNorm2d(128))
        self.classifier = nn.Linear(128 * 9, num_classes)
        for m in self.modules():
            if isinstance(m, nn.Conv2d):
                n = m.kernel_size[0] * m.kernel_size[1] * m.out_channels
                nn.init.normal_(m.weight, 0.0, math.sqrt(2.0 / n))
            elif isinstance(m, nn.BatchNorm2d):
                nn.init.ones_(m.weight)
                nn.init.zeros_(m.bias)
            elif isinstance(m, nn.Linear):
                nn.init.kaiming_normal_(m.weight)
                nn.init.zeros_(m.bias)

    def forward(self, x):
        x = self.block_3(self.block_2(self.block_1(x)))
        return self.classifier(x.flatten(1))


def caffe_cifar(num_classes=10):
    return CifarCaffeNet(num_classes)


class _DenseBottleneck(nn.Module):
    def __init__(self, cin, growth):
        super().__init__()
        self.bn1 = nn.BatchNorm2d(cin)
        self.conv1 = nn.Conv2d(cin, 4 * growth, kernel_size=1, bias=False)
        self.bn2 = nn.BatchNorm2d(4 * growth)
        self.conv2 = nn.Conv2d(4 * growth, growth, kernel_size=3, padding=1, bias=False)

    def forward(self, x):
        out = self.conv1(F.relu(self.bn1(x)))
        out = self.conv2(F.relu(self.bn2(out)))
        return torch.cat((x, out), 1)


class _DenseSingle(nn.Module):
    def __init__(self, cin, growth):
        super().__init__()
        self.bn1 = nn.BatchNorm2d(cin)
        self.conv1 = nn.Conv2d(cin, growth, kernel_size=3, padding=1, bias=False)

    def forward(self, x):
        return torch.cat((x, self.conv1(F.relu(self.bn1(x)))), 1)


class _DenseTransition(nn.Module):
    def __init__(self, cin, cout):
        super().__init__()
        self.bn1 = nn.BatchNorm2d(cin)
        self.conv1 = nn.Conv2d(cin, cout, kernel_size=1, bias=False)

    def forward(self, x):
        return F.avg_pool2d(self.conv1(F.relu(self.bn1(x))), 2)


class CifarDenseNet(nn.Module):
    """DenseNet for CIFAR (three dense blocks); outputs log-probabilities like the reference."""

    def __init__(self, growth, depth, reduction, num_classes, bottleneck):
        super().__init__()
        n = (depth - 4) // (6 if bottleneck else 3)
        unit = _DenseBottleneck if bottleneck else _DenseSingle
        ch = 2 * growth
        self.conv1 = nn.Conv2d(3, ch, kernel_size=3, padding=1, bias=False)

        def dense(c):
            layers = []
            for _ in range(n):
                layers.append(unit(c, growth))
                c += growth
            return nn.Sequential(*layers), c
        self.dense1, ch = dense(ch)
        out = int(math.floor(ch * reduction))
        self.trans1, ch = _DenseTransition(ch, out), out
        self.dense2, ch = dense(ch)
        out = int(math.floor(ch * reduction))
        self.trans2, ch = _DenseTransition(ch, out), out
        self.dense3, ch = dense(ch)
        self.bn1 = nn.BatchNorm2d(ch)
        self.fc = nn.Linear(ch, num_classes)
        for m in self.modules():
            if isinstance(m, nn.Conv2d):
                k = m.kernel_size[0] * m.kernel_size[1] * m.out_channels
                nn.init.normal_(m.weight, 0.0, math.sqrt(2.0 / k))
            elif isinstance(m, nn.BatchNorm2d):
                nn.init.ones_(m.weight)
                nn.init.zeros_(m.bias)
            elif isinstance(m, nn.Linear):
                nn.init.zeros_(m.bias)

    def forward(self, x):
        x = self.trans1(self.dense1(self.conv1(x)))
        x = self.dense3(self.trans2(self.dense2(x)))
        x = F.avg_pool2d(F.relu(self.bn1(x)), 8).flatten(1)
        return F.log_softmax(self.fc(x), dim=1)


def densenet100_12(num_classes=10):
    return CifarDenseNet(12, 100, 0.5, num_classes, False)
