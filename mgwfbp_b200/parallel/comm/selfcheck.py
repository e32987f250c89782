# -*- coding: utf-8 -*-
"""Start-up self-check of the NVLink data plane: every all-reduce algorithm this job can use is run on a few
message sizes and compared with the sum formed on the host.

The reference relies on Horovod/NCCL being correct and checks nothing (``distributed_optimizer.py:339``).  Here the
collectives are this package's own kernels, so a job can ask them to prove themselves on the GPUs it actually got
before the first training step: ``selfcheck(comm)`` all-reduces random vectors with the one-shot, two-shot and (when
the heap is bound to a multicast object) NVLS kernels, gathers every rank's input and output over the gloo control
plane, and reports the largest deviation from the float64 mean and whether all ranks hold bitwise identical results.
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import torch

from .. import runtime


def selfcheck(comm=None, sizes: Sequence[int] = (1000, 300003, 1 << 20), tol: float = 1e-5) -> Dict[str, object]:
    """Collective.  Returns ``{'ok', 'max_abs_err', 'bitwise_equal', 'algorithms', 'sizes', 'world'}``."""
    from .nvl import NvlComm
    comm = comm or NvlComm.shared()
    world, rank = comm.size(), comm.rank()
    algos = ['oneshot', 'twoshot'] + (['nvls'] if comm.nvls_available else [])
    max_err, bitwise, ran = 0.0, True, []
    for algo in algos:
        for n in sizes:
            if algo == 'oneshot' and n * 4 > comm.oneshot_max_bytes:
                continue
            g = torch.Generator(device='cuda').manual_seed(977 * rank + n % 1009)
            x = torch.randn(n, device=comm.device, generator=g)
            mine = x.clone()
            comm.synchronize(comm.allreduce_async_(x, average=True, algo=algo))
            torch.cuda.synchronize()
            comm.check_status()
            inputs = runtime.allgather_tensor(mine.cpu())
            outputs = runtime.allgather_tensor(x.cpu())
            want = sum(t.double() for t in inputs) / world
            max_err = max(max_err, float((outputs[rank].double() - want).abs().max()))
            bitwise = bitwise and all(torch.equal(outputs[0], o) for o in outputs[1:])
            ran.append('%s/%d' % (algo, n))
    max_err = runtime.max_over_ranks(max_err)
    ok = bool(max_err <= tol and bitwise)
    return {'ok': ok, 'max_abs_err': max_err, 'bitwise_equal': bool(bitwise), 'algorithms': algos, 'cases': len(ran),
            'world': world, 'multicast_heap': bool(comm.nvls_available)}
