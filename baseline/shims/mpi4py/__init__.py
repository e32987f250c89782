"""Import stub for ``from mpi4py import MPI``; ``COMM_WORLD.bcast`` goes through torch.distributed."""
import torch.distributed as dist


class _Comm(object):
    def bcast(self, obj, root=0):
        if not dist.is_initialized() or dist.get_world_size() == 1:
            return obj
        box = [obj]
        dist.broadcast_object_list(box, src=root)
        return box[0]

    def Get_rank(self):
        return dist.get_rank() if dist.is_initialized() else 0

    def Get_size(self):
        return dist.get_world_size() if dist.is_initialized() else 1


class MPI(object):
    COMM_WORLD = _Comm()
