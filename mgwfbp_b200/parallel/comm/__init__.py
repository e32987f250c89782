# -*- coding: utf-8 -*-
"""Communicators: the data plane behind :class:`~mgwfbp_b200.parallel.optimizer.DistributedOptimizer`.

``LocalComm``      world size 1, everything is the identity.
``TorchDistComm``  ``torch.distributed`` (gloo on CPU; also usable with NCCL as the unfused
                   comparison path).  Provides the Horovod-style ``allreduce_async_`` /
                   ``synchronize`` pair the reference uses (``distributed_optimizer.py:339,375``).
``NvlComm``        this package's peer-to-peer NVLink kernels with the fused SGD update
                   (``mgwfbp_b200.parallel.comm.nvl``), imported lazily because it needs the
                   native library.
"""
from .base import Communicator, LocalComm, TorchDistComm, make_communicator  # noqa: F401
