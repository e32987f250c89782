# -*- coding: utf-8 -*-
"""Native operators: ctypes bindings of ``libmgwfbp_b200.so`` (``_lib``), its build (``build``), and the PyTorch-facing
wrappers of the kernels (``bn_relu``, ``stem``, ``sgd``, ``lstm``, ``wgrad``), plus ``microbench`` and launch ``counters``."""
