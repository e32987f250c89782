# -*- coding: utf-8 -*-
"""Drop-in module for ``from profiling import benchmark``."""
from mgwfbp_b200.utils.profiling import Profiling, benchmark, CommunicationProfiler  # noqa: F401
