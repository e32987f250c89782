# -*- coding: utf-8 -*-
"""Drop-in module for ``import model_builder``."""
from mgwfbp_b200.models.small import MnistNet  # noqa: F401
from mgwfbp_b200.models.cifar_resnet_tv import model_builder  # noqa: F401
