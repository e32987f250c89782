# -*- coding: utf-8 -*-
"""All-reduce sweep of the NVLink data plane against NCCL, one process per GPU.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29650 \
        -m mgwfbp_b200.parallel.comm.bench [--max-mb 256] [--iters 20]

For every message size: device time (CUDA events on the launching stream, max over ranks) of this
package's one-shot / two-shot / NVLS kernels (reduce + 1/N + write-back, launched on the side stream)
and of ``torch.distributed.all_reduce`` (NCCL), the algorithm bandwidth ``S / t`` and the bus
bandwidth ``2 (N-1)/N * S / t``.  The ``iters`` calls of one measurement are captured into a CUDA
graph and replayed, as the training step does with its own launches, so the figures are device
times free of the host's launch path (``--eager`` times back-to-back host launches instead).  Ends with the fitted ``alpha + beta * bytes`` per algorithm, the
quantities the MG-WFBP scheduler consumes (the reference hard-codes them for its authors' Ethernet /
InfiniBand clusters, ``distributed_optimizer.py:166-177``).  Rank 0 prints a JSON document.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from ... import settings
from .. import runtime
from ..costmodel import fit_alpha_beta


def _time(fn, iters: int, barrier) -> float:
    for _ in range(3):
        fn()
    barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return runtime.max_over_ranks(e0.elapsed_time(e1) / iters)


def _time_graph(fn, iters: int, barrier) -> float:
    """Device time per call of ``fn`` replayed from a CUDA graph; falls back to :func:`_time` when
    any rank could not capture (the decision is taken collectively, so ranks never diverge)."""
    side = torch.cuda.Stream()
    graph = None
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    try:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            for _ in range(iters):
                fn()
        graph = g
    except Exception:                                      # capture refused: time the eager launches
        graph = None
    torch.cuda.synchronize()
    if not all(runtime.allgather_object(graph is not None)):
        return _time(fn, iters, barrier)
    graph.replay()
    barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return runtime.max_over_ranks(e0.elapsed_time(e1) / iters)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument('--max-mb', type=float, default=256.0)
    ap.add_argument('--iters', type=int, default=20)
    ap.add_argument('--eager', action='store_true', help='time host-launched calls instead of a graph replay')
    ap.add_argument('--out', default=None, help='also write the JSON document to this file')
    ap.add_argument('--ctas', type=int, default=0,
                    help='also time the large-message kernels capped at this many CTAs (what a group that overlaps backward gets)')
    args = ap.parse_args(argv)
    timeit = _time if args.eager else _time_graph
    runtime.init()
    settings.logger.setLevel('WARNING')
    from .nvl import NvlComm
    comm = NvlComm.shared()
    world, rank = runtime.size(), runtime.rank()
    sizes = [1 << k for k in range(8, 31) if (1 << k) * 4 <= args.max_mb * 1e6]       # floats
    rows, samples = [], {}
    algos = ['oneshot', 'twoshot'] + (['nvls'] if comm.nvls_available else [])
    from ...utils.clocks import ClockSampler
    sampler = ClockSampler(torch.cuda.current_device()).start() if rank == 0 else None
    for n in sizes:
        x = torch.randn(n, device='cuda')
        row = {'bytes': 4 * n}
        for algo in algos:
            if algo == 'oneshot' and 4 * n > comm.oneshot_max_bytes:
                continue
            ms = timeit(lambda: comm.synchronize(comm.allreduce_async_(x, algo=algo)), args.iters, runtime.barrier)
            row[algo + '_us'] = ms * 1e3
            samples.setdefault(algo, ([], []))
            samples[algo][0].append(n)
            samples[algo][1].append(ms * 1e-3)
            if args.ctas > 0 and algo != 'oneshot' and 4 * n > comm.oneshot_max_bytes:
                cap = min(args.ctas, comm.choose((n + 3) // 4)[1])
                ms = timeit(lambda: comm.synchronize(comm.allreduce_async_(x, algo=algo, n_ctas=cap)), args.iters, runtime.barrier)
                row['%s@%d_us' % (algo, args.ctas)] = ms * 1e3
        ms = timeit(lambda: dist.all_reduce(x, op=dist.ReduceOp.AVG), args.iters, runtime.barrier)
        row['nccl_us'] = ms * 1e3
        samples.setdefault('nccl', ([], []))
        samples['nccl'][0].append(n)
        samples['nccl'][1].append(ms * 1e-3)
        best = min(v for k, v in row.items() if k.endswith('_us') and k != 'nccl_us' and '@' not in k)
        row['best_busbw_GBps'] = 2 * (world - 1) / world * 4 * n / (best * 1e-6) / 1e9
        row['nccl_busbw_GBps'] = 2 * (world - 1) / world * 4 * n / (row['nccl_us'] * 1e-6) / 1e9
        rows.append(row)
        comm.check_status(synchronize=True)
    fits = {}
    for algo, (ns, ts) in samples.items():
        if len(ns) >= 2:
            ab = fit_alpha_beta(ns, ts, 4, algo)
            fits[algo] = {'alpha_us': ab.alpha * 1e6, 'beta_s_per_byte': ab.beta,
                          'asymptotic_algbw_GBps': (1e-9 / ab.beta) if ab.beta > 0 else None}
    if rank == 0:
        doc = json.dumps({'world': world, 'heap': comm.arena.heaps[0].kind, 'multicast': comm.nvls_available,
                          'timing': 'eager' if args.eager else 'graph', 'twoshot_ctas': comm.max_ctas_twoshot,
                          'threads': comm.n_threads, 'rows': rows, 'fits': fits, 'clocks': sampler.stop()})
        print(doc)
        if args.out:
            with open(args.out, 'w') as f:
                f.write(doc)
    runtime.shutdown()


if __name__ == '__main__':
    main()
