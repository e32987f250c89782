"""``horovod.torch.mpi_ops`` surface consumed by the reference (``distributed_optimizer.py:21-26``),
backed by ``torch.distributed`` NCCL.  Horovod itself cannot be built offline (no MPI, no
network), so the reference's unmodified optimizer runs on this shim in the baseline arm.

The shim is kept as favourable to the reference as NCCL allows: the all-reduce is asynchronous
(NCCL's own stream), averaging is done by NCCL (``ReduceOp.AVG``, no extra kernel) and
``synchronize`` is a stream wait, not a host block.
"""
import os

import torch
import torch.distributed as dist


def init():
    if dist.is_initialized():
        return
    if int(os.environ.get('WORLD_SIZE', '1')) > 1:
        local = int(os.environ.get('LOCAL_RANK', '0'))
        torch.cuda.set_device(local)
        dist.init_process_group('nccl', device_id=torch.device('cuda', local))


def size():
    return dist.get_world_size() if dist.is_initialized() else 1


def rank():
    return dist.get_rank() if dist.is_initialized() else 0


def local_size():
    return int(os.environ.get('LOCAL_WORLD_SIZE', size()))


def local_rank():
    return int(os.environ.get('LOCAL_RANK', '0'))


def allreduce_async_(tensor, average=True, name=None):
    if size() == 1:
        return (None, tensor)
    op = dist.ReduceOp.AVG if average else dist.ReduceOp.SUM
    return (dist.all_reduce(tensor, op=op, async_op=True), tensor)


def allgather_async(tensor, name=None):
    out = [torch.empty_like(tensor) for _ in range(size())]
    work = dist.all_gather(out, tensor, async_op=True)
    return (work, out)


def broadcast_async_(tensor, root_rank, name=None):
    if size() == 1:
        return (None, tensor)
    if not tensor.is_cuda:
        dev = tensor.cuda()
        dist.broadcast(dev, src=root_rank)
        tensor.copy_(dev)
        return (None, tensor)
    return (dist.broadcast(tensor, src=root_rank, async_op=True), tensor)


def broadcast(tensor, root_rank, name=None):
    out = tensor.clone()
    synchronize(broadcast_async_(out, root_rank))
    return out


def synchronize(handle):
    work, out = handle
    if work is not None:
        work.wait()
    return torch.cat(out) if isinstance(out, list) else out
