from .mpi_ops import (allreduce_async_, allgather_async, broadcast_async_, synchronize, size, local_size, rank,  # noqa: F401
                      local_rank, init, broadcast)
