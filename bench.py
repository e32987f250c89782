# -*- coding: utf-8 -*-
"""Headline benchmark: synchronous data-parallel training throughput on N GPUs of one node.

    python bench.py --gpus 1 --steps 30 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29600 \
        bench.py --gpus 8 --steps 30 --warmup 5
    python bench.py --impl reference ...        # the unmodified reference on a NCCL-backed Horovod shim

Default workload: ResNet-50 (torchvision bottleneck v1), batch 64 per GPU, 3x224x224 synthetic fp32 inputs,
SGD momentum 0.9 / weight decay 1e-4, fp32 storage with TF32 tensor-core math (weak scaling).  Rank 0 prints ONE
JSON line.  ``value`` is the device-timed (CUDA events, max over ranks) aggregate images/s of the training step with
inputs already on the device; ``e2e`` is the same metric through the public trainer API with, every step, the copy of
that step's inputs from pinned host memory and a device-to-host read of the step's loss.
"""
from __future__ import print_function

import argparse
import json
import os
import shutil
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))

WORKLOADS = {
    # dnn: (dataset, per-GPU batch, lr, unit, items per sample)
    'resnet50': ('imagenet', 64, 0.01, 'images/s', 1),
    'densenet201': ('imagenet', 32, 0.01, 'images/s', 1),
    'vgg16i': ('imagenet', 64, 0.01, 'images/s', 1),
    'resnet20': ('cifar10', 32, 0.1, 'images/s', 1),
    'lstm': ('ptb', 20, 22.0, 'tokens/s', 35),
}


class ClockSampler(object):
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ('index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,'
             'clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,'
             'clocks_event_reasons.sw_power_cap')

    def __init__(self, gpu_index):
        self.gpu_index, self.proc, self.path = gpu_index, None, None

    def start(self):
        exe = shutil.which('nvidia-smi')
        if exe is None:
            return
        fd, self.path = tempfile.mkstemp(suffix='.csv')
        self._out = os.fdopen(fd, 'w')
        self.proc = subprocess.Popen([exe, '-i', str(self.gpu_index), '--query-gpu=' + self.QUERY,
                                      '--format=csv,noheader,nounits', '-lms', '100'], stdout=self._out,
                                     stderr=subprocess.DEVNULL)

    def stop(self):
        if self.proc is None:
            return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': [], 'samples': 0}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self._out.close()
        sm, smax, power, reasons = [], [], [], set()
        with open(self.path) as f:
            for line in f:
                parts = [p.strip() for p in line.split(',')]
                if len(parts) < 9:
                    continue
                try:
                    sm.append(float(parts[1]))
                    smax.append(float(parts[2]))
                    power.append(float(parts[3]))
                except ValueError:
                    continue
                for name, val in zip(('hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap'), parts[5:9]):
                    if val.lower().startswith('active'):
                        reasons.add(name)
        os.unlink(self.path)
        busy = [c for c, p in zip(sm, power) if p > 0.5 * max(power)] if power else sm
        return {'sm_mhz': statistics.median(busy) if busy else None, 'sm_max_mhz': max(smax) if smax else None,
                'reasons': sorted(reasons), 'samples': len(sm), 'power_w_max': max(power) if power else None}


def _dist_env(args):
    world = int(os.environ.get('WORLD_SIZE', '1'))
    if world != args.gpus:
        if args.gpus == 1 and world == 1:
            pass
        else:
            raise SystemExit('--gpus %d but WORLD_SIZE=%d: launch with torch.distributed.run --nproc-per-node %d'
                             % (args.gpus, world, args.gpus))
    return int(os.environ.get('RANK', '0')), int(os.environ.get('LOCAL_RANK', '0')), world


def _config(args, world, bs, dataset, groups, graphed, comm):
    """The ``config`` object of the JSON line; both arms print the same keys."""
    return {'model': args.dnn, 'global_batch': world * bs, 'per_gpu_batch': bs,
            'seq_len': 35 if args.dnn == 'lstm' else None, 'parallelism': 'dp%d' % world,
            'policy': args.policy + ('(%d)' % args.threshold if args.policy == 'bucket' else ''), 'cuda_graph': bool(graphed),
            'optimizer': 'sgd momentum 0.9 wd 1e-4' if dataset != 'ptb' else 'sgd lr 22 clip 0.25',
            'groups': groups, 'comm': comm,
            'matmul': 'fp32' if args.fp32_matmul else 'tf32',
            'l2': 'per-step working set (activations + weights, > 1 GB) exceeds the 126 MB L2; no explicit flush'}


def _dtype(args):
    return 'tf32 convolutions, %s matmul (fp32 storage)' % ('fp32' if args.fp32_matmul else 'tf32')


def _time_steps(torch, dist_ok, step_fn, steps, barrier):
    """Time exactly `steps` calls of step_fn on the device; returns ms per step (this rank)."""
    barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        step_fn(i)
    e1.record()
    torch.cuda.synchronize()
    barrier()
    return e0.elapsed_time(e1) / steps


def run_ours(args):
    rank, local_rank, world = _dist_env(args)
    import torch
    if not torch.cuda.is_available():
        raise SystemExit('bench.py needs a CUDA device')
    torch.cuda.set_device(local_rank)
    torch.backends.cudnn.benchmark = True
    torch.backends.cudnn.allow_tf32 = True
    torch.backends.cuda.matmul.allow_tf32 = not args.fp32_matmul          # the same setting in both arms
    sys.path.insert(0, ROOT)
    import mgwfbp_b200 as hvd
    from mgwfbp_b200 import settings
    from mgwfbp_b200.ops import counters
    from mgwfbp_b200.trainer import DLTrainer
    from mgwfbp_b200.utils.profiling import benchmark as profile_backward

    dataset, default_bs, lr, unit, per_sample = WORKLOADS[args.dnn]
    bs = args.batch_size or default_bs
    hvd.init()
    settings.logger.setLevel('WARNING')
    settings.ADAPTIVE_MERGE = args.policy == 'mgwfbp'
    settings.ORIGINAL_HOROVOD = args.policy == 'nccl'        # the in-repo stock arm: NCCL buckets + torch's SGD.step
    trainer = DLTrainer(rank, world, dist=False, batch_size=bs, ngpus=1, data_dir='synthetic', dataset=dataset,
                        dnn=args.dnn, lr=lr, nworkers=world, prefix='allreduce', seed=0,
                        momentum=0.9 if dataset != 'ptb' else None, weight_decay=1e-4 if dataset != 'ptb' else None)
    trainer.num_batches_per_epoch = 10 ** 9          # stay inside epoch 0: no epoch-boundary work in the timed region
    seq = times = None
    if world > 1 and args.policy == 'mgwfbp':
        seq, times, _sizes = profile_backward(trainer, warmup=3, iteration=10)
        times = hvd.broadcast_object(list(times), 0)
    threshold = {'mgwfbp': 0, 'wfbp': 0, 'single': 524288000, 'bucket': args.threshold, 'nccl': 0}[args.policy]
    norm_clip = 0.25 if args.dnn == 'lstm' else None
    # start-up self-check of the communication kernels (outside every timed region)
    selfcheck = None
    if world > 1 and args.policy != 'nccl' and not args.no_selfcheck:
        from mgwfbp_b200.parallel.comm.selfcheck import selfcheck as run_selfcheck
        selfcheck = run_selfcheck()
    # cost model + interference measured on this box, schedule confirmed by timing it (engine.build_distributed_optimizer)
    from mgwfbp_b200.engine import build_distributed_optimizer
    optimizer, tuning = build_distributed_optimizer(trainer, seq_layernames=seq, layerwise_times=times, threshold=threshold,
                                                    norm_clip=norm_clip, tune=not args.no_tune, fit_comm=not args.no_comm_fit,
                                                    use_graph=not args.no_graph)

    from mgwfbp_b200.engine import TrainStep
    step = TrainStep(trainer, use_graph=not args.no_graph)
    hidden = [trainer.net.init_hidden() if args.dnn == 'lstm' else None]

    # ---- device-resident inputs: the training step alone -------------------------------------------------
    dev_batch = trainer.to_device(trainer.data_iter())

    def step_device(i):
        step.run_on_device(dev_batch)

    # ---- end to end: pinned host batch -> device, step, loss back to the host, every step ---------------
    loss_host = []

    upcoming = [trainer.data_iter()]

    def step_e2e(i):
        cur, nxt = upcoming[0], trainer.data_iter()      # the next pinned batch is copied while this step computes
        upcoming[0] = nxt
        loss_host.append(step.run(cur, next_host_batch=nxt))

    barrier = hvd.barrier
    for i in range(max(args.warmup, 3)):
        step_device(i)
    if not args.skip_e2e:
        for i in range(3):
            step_e2e(i)
    step.drain()
    torch.cuda.synchronize()

    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    counters.reset()
    if args.profiler_range:
        torch.cuda.profiler.start()
    step.replays, step.replay_host_s = 0, 0.0
    ms_dev = _time_steps(torch, world > 1, step_device, args.steps, barrier)
    host_replay_ms = 1e3 * step.replay_host_s / step.replays if step.replays else None      # host side of one graph launch
    if args.profiler_range:
        torch.cuda.profiler.stop()
    launches = counters.total()
    clocks = sampler.stop() if sampler else None
    del loss_host[:]

    def e2e_all(i):
        step_e2e(i)
        if i == args.steps - 1:
            step.drain()           # the last step's loss is read inside the timed region too
    ms_e2e = _time_steps(torch, world > 1, e2e_all, args.steps, barrier) if not args.skip_e2e else float('nan')
    ms_dev = hvd.parallel.runtime.max_over_ranks(ms_dev) if world > 1 else ms_dev
    ms_e2e = hvd.parallel.runtime.max_over_ranks(ms_e2e) if world > 1 else ms_e2e
    final_loss = step.last_loss()

    if args.timeline:
        # after the timed region: three more steps under the CUPTI activity tracer, one chrome-trace file per rank
        # (kernel name, stream, start, duration), the evidence for what overlaps what inside a replayed step
        from torch.profiler import profile, ProfilerActivity
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for i in range(3):
                step_device(i)
            torch.cuda.synchronize()
        prof.export_chrome_trace('%s.rank%d.json' % (args.timeline, rank))

    exposed = comm_ms = None
    if world > 1 and getattr(optimizer, '_fused_comm', False):
        # exposed communication = end of the last communication kernel minus end of backward (>= 0), eager steps
        from mgwfbp_b200.utils.tracing import CommTrace
        from mgwfbp_b200.engine import _tables_of
        for tbl in _tables_of(optimizer):
            tbl.invalidate()
        vals, totals = [], []
        for i in range(5 if args.dnn != 'lstm' else 0):
            trace = CommTrace(optimizer)
            optimizer.zero_grad()
            with trace:
                loss, _o, _l, _h = trainer.forward_loss(dev_batch, None, on_device=True)
                loss.backward()
                trace.mark_backward_end()
                optimizer.step()
            summ = trace.summary()
            if i >= 2:
                vals.append(summ['exposed_comm_ms'])
                totals.append(summ['comm_ms'])
        if vals:
            exposed = hvd.parallel.runtime.max_over_ranks(sum(vals) / len(vals))
            comm_ms = hvd.parallel.runtime.max_over_ranks(sum(totals) / len(totals))

    comm = getattr(optimizer, '_comm', None)
    if world == 1:
        comm_name = 'none (one GPU)'
    elif getattr(comm, 'fused', False):
        algos = sorted({p.algo for p in comm._plans.get(id(optimizer), [])})
        comm_name = 'own NVLink kernels (%s; %s heap%s)' % (
            '+'.join({0: 'one-shot', 1: 'two-shot', 2: 'NVLS multimem'}[a] for a in algos), comm.arena.heaps[0].kind,
            ', NVSwitch multicast' if comm.nvls_available else '')
    else:
        comm_name = 'NCCL via torch.distributed (stock arm)'
    if rank == 0:
        value = world * bs * per_sample / (ms_dev * 1e-3)
        e2e = world * bs * per_sample / (ms_e2e * 1e-3)
        h2d = sum(t.numel() * t.element_size() for t in trainer.data_iter() if hasattr(t, 'numel'))
        out = {
            'metric': '%s training throughput (%s, aggregate over all GPUs)' % (args.dnn, unit), 'value': value, 'unit': unit,
            'n_gpus': world, 'steps': args.steps, 'warmup': max(args.warmup, 3), 'ms_per_step': ms_dev,
            'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None, 'dtype': _dtype(args),
            'data': 'synthetic', 'impl': 'ours',
            'config': _config(args, world, bs, dataset, len(optimizer.merge_schedule.groups), step.graphed, comm_name),
            'clocks': clocks,
            'e2e': {'value': e2e, 'unit': unit, 'ms_per_step': ms_e2e, 'h2d_bytes_per_step': h2d, 'd2h_bytes_per_step': 4},
            'gpu_launches': launches, 'final_loss': final_loss,
            'exposed_comm_ms': exposed, 'comm_kernel_ms': comm_ms,
            'selfcheck': selfcheck, 'schedule_tuning': tuning,
            'sgd_stock_fallback_steps': getattr(getattr(optimizer, '_fast_sgd', None), 'fallback_steps', 0),
            'eager_steps_after_capture': step.eager_after_capture, 'host_graph_launch_ms': host_replay_ms,
        }
        print(json.dumps(out))
    hvd.shutdown()


def run_reference(args):
    """The reference's own classes (DLTrainer, profiling.benchmark, DistributedOptimizer, broadcast_parameters) from
    baseline/_ref, unmodified, on NCCL.  None of this package's code is imported on this path."""
    ref_dir = os.path.join(ROOT, 'baseline', '_ref')
    if not os.path.isfile(os.path.join(ref_dir, 'distributed_optimizer.py')):
        print(json.dumps({'impl': 'reference', 'unavailable': 'baseline/_ref is not installed (see baseline/README.md)'}))
        return
    rank, local_rank, world = _dist_env(args)
    # the reference is a flat directory of modules named settings/utils/profiling/...: make sure they win
    sys.path[:] = [ref_dir, os.path.join(ROOT, 'baseline', 'shims')] + [p for p in sys.path if os.path.abspath(p or '.') != ROOT]
    os.chdir(tempfile.mkdtemp(prefix='refbench'))
    import collections
    import collections.abc
    collections.Iterable = collections.abc.Iterable
    import torch
    if not torch.cuda.is_available():
        raise SystemExit('bench.py needs a CUDA device')
    torch.cuda.set_device(local_rank)
    torch.backends.cudnn.allow_tf32 = True                                   # torch's default, stated
    torch.backends.cuda.matmul.allow_tf32 = not args.fp32_matmul             # the same setting in both arms
    import logging
    import numpy as np
    import settings
    settings.logger.setLevel(logging.ERROR)
    import horovod.torch.mpi_ops as ops
    ops.init()
    import distributed_optimizer as hvd
    from dl_trainer import DLTrainer
    from profiling import benchmark

    dataset, default_bs, lr, unit, per_sample = WORKLOADS[args.dnn]
    bs = args.batch_size or default_bs
    settings.ADAPTIVE_MERGE = args.policy == 'mgwfbp'
    hvd.ADAPTIVE_MERGE = settings.ADAPTIVE_MERGE
    settings.CONNECTION = '56GbIB'          # the faster of the reference's two built-in cost tables
    if world not in (1, 2, 4, 8, 16) and args.policy == 'mgwfbp':
        print(json.dumps({'impl': 'reference', 'unavailable': 'reference cost tables only cover 2/4/8/16 workers'}))
        return
    if dataset == 'ptb':
        DLTrainer.vocab_size = 10000      # normally discovered by the PTB reader; no dataset is read here
    trainer = DLTrainer(rank, world, dist=False, batch_size=bs, is_weak_scaling=True, ngpus=1, data_dir=None,
                        dataset=dataset, dnn=args.dnn, lr=lr, nworkers=world, prefix='allreduce', num_steps=35)
    if dataset != 'ptb':
        for g in trainer.optimizer.param_groups:      # BASELINE's hyper-parameters instead of the imagenet defaults
            g['momentum'] = 0.9
            if g['weight_decay'] != 0:
                g['weight_decay'] = 1e-4
    trainer.num_batches_per_epoch = 10 ** 9
    if dataset == 'imagenet':
        shape, classes = (bs, 3, 224, 224), 1000
    elif dataset == 'cifar10':
        shape, classes = (bs, 3, 32, 32), 10
    else:
        shape, classes = (bs, 35), 10000
    g = torch.Generator().manual_seed(rank)
    if dataset == 'ptb':
        ring = []
        for _ in range(4):
            seq = torch.randint(0, classes, (bs, 36), generator=g)
            ring.append((seq[:, :-1].contiguous().pin_memory(), seq[:, 1:].contiguous().pin_memory()))
    else:
        ring = [(torch.randn(shape, generator=g).pin_memory(), torch.randint(0, classes, (bs,), generator=g).pin_memory())
                for _ in range(4)]

    class _Iter(object):           # the reference calls `.next()` on its iterator (Python-2 style)
        def __init__(self):
            self.i = 0

        def next(self):
            self.i += 1
            return ring[self.i % len(ring)]
    trainer.data_iterator = _Iter()
    trainer._input_shape, trainer._output_shape = shape, (bs, classes)

    seq = times = None
    if world > 1 and args.policy == 'mgwfbp':
        seq, times, sizes = benchmark(trainer)
        box = [list(times)]
        torch.distributed.broadcast_object_list(box, src=0)
        times = box[0]
    threshold = {'mgwfbp': 0, 'wfbp': 0, 'single': 524288000, 'bucket': args.threshold, 'nccl': 0}[args.policy]
    from compression import compressors
    optimizer = hvd.DistributedOptimizer(trainer.optimizer, named_parameters=trainer.net.named_parameters(),
                                         compression=compressors[None], seq_layernames=seq, layerwise_times=times,
                                         norm_clip=None, threshold=threshold)
    if world > 1:
        hvd.broadcast_parameters(trainer.net.state_dict(), root_rank=0)
    trainer.update_optimizer(optimizer)

    def barrier():
        if world > 1:
            torch.distributed.barrier()
    dev_batch = tuple(t.cuda() for t in ring[0])
    hidden = [trainer.net.init_hidden()] if args.dnn == 'lstm' else None

    def step_with(data):
        optimizer.zero_grad()
        optimizer.local = False
        if args.dnn == 'lstm':               # loop body of the reference's dist_trainer.py:85-94
            _, hidden[0] = trainer.train(1, data=data, hidden=hidden[0])
            optimizer.synchronize()
            torch.nn.utils.clip_grad_norm_(trainer.net.parameters(), 0.25)
        else:
            trainer.train(1, data=data)      # forward, backward (+ hooks), loss.item()
        trainer.update_model()               # synchronize + SGD step

    for i in range(max(args.warmup, 3)):
        step_with(dev_batch)
    for i in range(3):
        step_with(ring[i % 4])
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    ms_dev = _time_steps(torch, world > 1, lambda i: step_with(dev_batch), args.steps, barrier)
    clocks = sampler.stop() if sampler else None
    ms_e2e = _time_steps(torch, world > 1, lambda i: step_with(ring[i % 4]), args.steps, barrier)
    if world > 1:
        t = torch.tensor([ms_dev, ms_e2e], device='cuda', dtype=torch.float64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms_dev, ms_e2e = float(t[0]), float(t[1])
    if rank == 0:
        out = {
            'impl': 'reference',
            'metric': '%s training throughput (%s, aggregate over all GPUs)' % (args.dnn, unit),
            'value': world * bs * per_sample / (ms_dev * 1e-3), 'unit': unit, 'n_gpus': world, 'steps': args.steps,
            'warmup': max(args.warmup, 3), 'ms_per_step': ms_dev, 'higher_is_better': True, 'scaling': 'weak',
            'vs_baseline': None, 'dtype': _dtype(args), 'data': 'synthetic',
            'config': _config(args, world, bs, dataset, len(optimizer._groups), False,
                              'none (one GPU)' if world == 1 else 'NCCL via torch.distributed behind a horovod.torch.mpi_ops shim'),
            'clocks': clocks,
            'e2e': {'value': world * bs * per_sample / (ms_e2e * 1e-3), 'unit': unit, 'ms_per_step': ms_e2e,
                    'h2d_bytes_per_step': sum(t.numel() * t.element_size() for t in ring[0]), 'd2h_bytes_per_step': 4},
            'gpu_launches': 0,
        }
        print(json.dumps(out))
    if world > 1:
        torch.distributed.destroy_process_group()


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=30)
    ap.add_argument('--warmup', type=int, default=5)
    ap.add_argument('--impl', choices=['ours', 'reference'], default='ours')
    ap.add_argument('--dnn', choices=sorted(WORKLOADS), default='resnet50')
    ap.add_argument('--batch-size', type=int, default=None, help='per-GPU batch (default: the workload\'s)')
    ap.add_argument('--policy', choices=['mgwfbp', 'wfbp', 'single', 'bucket', 'nccl'], default='mgwfbp',
                    help="merge policy: MG-WFBP schedule, one message per tensor, one message in all, fixed-size buckets, or "
                         "the stock arm (NCCL through torch.distributed in 64 MB fusion buckets + torch's SGD.step)")
    ap.add_argument('--fp32-matmul', action='store_true', help='full-precision cuBLAS matmuls in both arms (default: TF32 in both)')
    ap.add_argument('--no-tune', action='store_true', help='do not time candidate schedules; trust the interference model')
    ap.add_argument('--no-selfcheck', action='store_true', help='skip the start-up self-check of the communication kernels')
    ap.add_argument('--threshold', type=int, default=8 * 1024 * 1024, help="bucket size in elements for --policy bucket")
    ap.add_argument('--no-graph', action='store_true', help='do not capture the training step in a CUDA graph')
    ap.add_argument('--timeline', default=None, metavar='PREFIX',
                    help='after timing, trace three steps and write PREFIX.rank<r>.json (chrome trace of every kernel)')
    ap.add_argument('--skip-e2e', action='store_true', help='profiling aid: time only the device-resident loop')
    ap.add_argument('--profiler-range', action='store_true',
                    help='profiling aid: bracket the timed device loop with cudaProfilerStart/Stop (ncu --profile-from-start off)')
    ap.add_argument('--no-comm-fit', action='store_true', help='skip the alpha-beta sweep; use the built-in NVLink table')
    args = ap.parse_args()
    if args.impl == 'reference':
        run_reference(args)
    else:
        run_ours(args)


if __name__ == '__main__':
    main()
