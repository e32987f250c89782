# -*- coding: utf-8 -*-
"""Drop-in module for ``from compression import compressors``."""
from mgwfbp_b200.utils.compression import NoneCompressor, compressors  # noqa: F401
