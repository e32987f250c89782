# -*- coding: utf-8 -*-
"""Drop-in module for ``import resnet`` (CIFAR-sized ResNet-18 ... 152)."""
from mgwfbp_b200.models.cifar_resnet_tv import BasicBlock, Bottleneck, ResNet, ResNet18, ResNet34, ResNet50, ResNet101, ResNet152  # noqa: F401
