# -*- coding: utf-8 -*-
"""Process-group runtime: ``init / rank / size / local_rank / local_size / broadcast``.

Stands in for the Horovod entry points that the reference re-exports from
``horovod.torch.mpi_ops`` (``distributed_optimizer.py:21-26``) and for its mpi4py side channel
(``dist_trainer.py:22-23,46``).  One process drives one GPU.  The data plane is either this
package's NVLink kernels (GPU) or ``torch.distributed`` gloo (CPU); a gloo group always exists
as the control plane for object broadcasts, schedule agreement and timing reductions.
"""
from __future__ import annotations

import datetime
import os
from typing import Any, List, Optional

import torch
import torch.distributed as dist

from ..settings import logger

_state = {
    'initialized': False,
    'rank': 0,
    'size': 1,
    'local_rank': 0,
    'local_size': 1,
    'control_group': None,   # gloo group for CPU-side objects
    'data_group': None,      # default group (nccl on GPU boxes, gloo otherwise)
    'owns_pg': False,
    'timeout_s': 600.0,
}


def _env_int(name: str, default: int) -> int:
    try:
        return int(os.environ.get(name, default))
    except ValueError:
        return default


def init(backend: Optional[str] = None, timeout_s: Optional[float] = None, device: Optional[str] = None) -> None:
    """Join the job described by ``RANK / WORLD_SIZE / LOCAL_RANK / MASTER_ADDR / MASTER_PORT``.

    Without ``WORLD_SIZE`` (or with ``WORLD_SIZE=1``) this is a no-op single-process job, which
    mirrors the reference calling ``hvd.init()`` only when ``nworkers > 1``
    (``dist_trainer.py:132-134``).  ``timeout_s`` bounds every control-plane collective so a
    missing rank surfaces as an exception instead of a hang.
    """
    if _state['initialized']:
        return
    if timeout_s is not None:
        _state['timeout_s'] = float(timeout_s)
    world = _env_int('WORLD_SIZE', 1)
    use_cuda = torch.cuda.is_available() and (device is None or device.startswith('cuda'))
    local_rank = _env_int('LOCAL_RANK', _env_int('RANK', 0) % max(torch.cuda.device_count(), 1) if use_cuda else 0)
    if use_cuda:
        torch.cuda.set_device(local_rank % torch.cuda.device_count())
    if world <= 1 and not dist.is_initialized():
        _state.update(initialized=True, rank=0, size=1, local_rank=0, local_size=1)
        return
    timeout = datetime.timedelta(seconds=_state['timeout_s'])
    if not dist.is_initialized():
        os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
        os.environ.setdefault('MASTER_PORT', '29500')
        if backend is None:
            backend = 'nccl' if use_cuda else 'gloo'
        kwargs = {}
        if backend == 'nccl':
            kwargs['device_id'] = torch.device('cuda', torch.cuda.current_device())
        dist.init_process_group(backend=backend, timeout=timeout, **kwargs)
        _state['owns_pg'] = True
    _state['data_group'] = dist.group.WORLD
    if dist.get_backend() == 'gloo':
        _state['control_group'] = dist.group.WORLD
    else:
        _state['control_group'] = dist.new_group(backend='gloo', timeout=timeout)
    _state.update(initialized=True, rank=dist.get_rank(), size=dist.get_world_size(),
                  local_rank=local_rank, local_size=_env_int('LOCAL_WORLD_SIZE', dist.get_world_size()))
    logger.debug('runtime initialised: rank %d of %d', _state['rank'], _state['size'])


def shutdown() -> None:
    """Leave the job; safe to call twice.  A live NVLink communicator is closed first (collective: its symmetric
    memory is unmapped and, where bound, released from the NVSwitch multicast object while all ranks are still there)."""
    try:
        import sys
        nvl = sys.modules.get(__package__ + '.comm.nvl')
        comm = getattr(getattr(nvl, 'NvlComm', None), '_shared', None) if nvl is not None else None
        if comm is not None:
            comm.close()
    except Exception as e:  # pragma: no cover - teardown is best effort (e.g. a peer is already gone)
        logger.warning('closing the NVLink communicator failed: %s', e)
    if _state['initialized'] and _state['owns_pg'] and dist.is_initialized():
        try:
            dist.destroy_process_group()
        except Exception:  # pragma: no cover - teardown is best effort
            pass
    _state.update(initialized=False, rank=0, size=1, local_rank=0, local_size=1,
                  control_group=None, data_group=None, owns_pg=False)


def is_initialized() -> bool:
    return bool(_state['initialized'])


def rank() -> int:
    return int(_state['rank'])


def size() -> int:
    return int(_state['size'])


def local_rank() -> int:
    return int(_state['local_rank'])


def local_size() -> int:
    return int(_state['local_size'])


def control_group():
    return _state['control_group']


def data_group():
    return _state['data_group']


def broadcast(tensor: torch.Tensor, root_rank: int = 0, name: Optional[str] = None) -> torch.Tensor:
    """Out-of-place broadcast returning the root's value (Horovod ``broadcast`` semantics,
    used for the epoch / iteration scalars at reference ``dist_trainer.py:36-39``)."""
    if size() == 1:
        return tensor.clone()
    out = tensor.clone()
    group = _state['control_group'] if out.device.type == 'cpu' else _state['data_group']
    dist.broadcast(out, src=root_rank, group=group)
    return out


def broadcast_object(obj: Any, root_rank: int = 0) -> Any:
    """Pickle-broadcast a Python object over the control plane (replaces ``MPI.COMM_WORLD.bcast``)."""
    if size() == 1:
        return obj
    box: List[Any] = [obj if rank() == root_rank else None]
    dist.broadcast_object_list(box, src=root_rank, group=_state['control_group'])
    return box[0]


def allgather_object(obj: Any) -> List[Any]:
    if size() == 1:
        return [obj]
    out: List[Any] = [None] * size()
    dist.all_gather_object(out, obj, group=_state['control_group'])
    return out


def barrier() -> None:
    if size() > 1:
        dist.barrier(group=_state['control_group'])


def allgather_tensor(t: torch.Tensor) -> List[torch.Tensor]:
    """All ranks' copies of a CPU tensor of equal shape, in rank order, over the control plane."""
    if size() == 1:
        return [t]
    out = [torch.empty_like(t) for _ in range(size())]
    dist.all_gather(out, t.contiguous(), group=_state['control_group'])
    return out


def max_over_ranks(value: float) -> float:
    """Max of a host scalar over all ranks (multi-GPU timings are reported as the slowest rank)."""
    if size() == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=_state['control_group'])
    return float(t.item())
