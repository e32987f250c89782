# -*- coding: utf-8 -*-
from __future__ import annotations

from typing import Any, Dict, Optional, Tuple

import torch
import torch.distributed as dist

from .. import runtime


class CommTimeoutError(RuntimeError):
    """A peer did not show up within the bounded wait of a communication kernel."""


class Communicator:
    """Minimal asynchronous collective interface (Horovod ``mpi_ops`` shaped)."""
    fused = False

    def size(self) -> int:
        return runtime.size()

    def rank(self) -> int:
        return runtime.rank()

    def allreduce_async_(self, tensor: torch.Tensor, average: bool = True, name: Optional[str] = None):
        raise NotImplementedError

    def synchronize(self, handle) -> torch.Tensor:
        raise NotImplementedError

    def broadcast_async_(self, tensor: torch.Tensor, root_rank: int, name: Optional[str] = None):
        raise NotImplementedError

    def broadcast_(self, tensor: torch.Tensor, root_rank: int) -> torch.Tensor:
        return self.synchronize(self.broadcast_async_(tensor, root_rank))

    def close(self) -> None:
        pass


class LocalComm(Communicator):
    def size(self) -> int:
        return 1

    def rank(self) -> int:
        return 0

    def allreduce_async_(self, tensor, average=True, name=None):
        return tensor

    def synchronize(self, handle):
        return handle

    def broadcast_async_(self, tensor, root_rank, name=None):
        return tensor


class TorchDistComm(Communicator):
    """In-place all-reduce through ``torch.distributed``; handles are ``(work, tensor, scale)``."""

    def __init__(self, group=None):
        self._group = group

    def _group_for(self, tensor: torch.Tensor):
        if self._group is not None:
            return self._group
        return runtime.control_group() if tensor.device.type == 'cpu' else runtime.data_group()

    def allreduce_async_(self, tensor, average=True, name=None):
        work = dist.all_reduce(tensor, op=dist.ReduceOp.SUM, group=self._group_for(tensor), async_op=True)
        return (work, tensor, (1.0 / self.size()) if average else None)

    def synchronize(self, handle):
        work, tensor, scale = handle
        if work is not None:
            work.wait()
        if scale is not None:
            tensor.mul_(scale)
        return tensor

    def broadcast_async_(self, tensor, root_rank, name=None):
        work = dist.broadcast(tensor, src=root_rank, group=self._group_for(tensor), async_op=True)
        return (work, tensor, None)


def make_communicator(device: Optional[torch.device] = None, prefer_fused: bool = True) -> Communicator:
    """Pick the data plane for tensors living on ``device``."""
    if runtime.size() == 1:
        return LocalComm()
    from ... import settings
    if device is not None and torch.device(device).type == 'cuda' and prefer_fused and not settings.ORIGINAL_HOROVOD:
        from .nvl import NvlComm  # needs the native library
        return NvlComm.shared()
    return TorchDistComm()
