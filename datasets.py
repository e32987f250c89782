# -*- coding: utf-8 -*-
"""Drop-in module for ``from datasets import DatasetHDF5``."""
from mgwfbp_b200.data.hdf5 import DatasetHDF5, create_hdf5, read_label_mapping  # noqa: F401
