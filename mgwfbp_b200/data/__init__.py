# -*- coding: utf-8 -*-
"""Datasets: ImageNet (HDF5), CIFAR-10, MNIST, Penn Treebank, AN4 -- and synthetic stand-ins."""
from .synthetic import SyntheticImages, SyntheticTokens, SyntheticLoader, NOMINAL_LENGTH  # noqa: F401
from .hdf5 import DatasetHDF5  # noqa: F401
from . import ptb as ptb_reader  # noqa: F401
