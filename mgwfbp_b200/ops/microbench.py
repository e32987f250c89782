# -*- coding: utf-8 -*-
"""Event-timed micro-benchmarks of this package's kernels on one GPU, with achieved fraction of the
measured roofline (``MEASURED_PEAKS.json`` at the repository root when present).

    python -m mgwfbp_b200.ops.microbench bn    --rows 200704 --channels 256
    python -m mgwfbp_b200.ops.microbench sgd   --numel 25557032
    python -m mgwfbp_b200.ops.microbench wgrad --k 64 --m 4096 --n 25088 [--sgd]
    python -m mgwfbp_b200.ops.microbench pack  --numel 25557032          # fused all-reduce kernel, world size 1
    python -m mgwfbp_b200.ops.microbench fused                            # all of ResNet-50 as one group: all-reduce + SGD

Timing: CUDA events on the launching stream, ``--warmup`` untimed launches, a write larger than L2
between timed launches, median of ``--iters``; the last line printed is the SM clock / throttle-reason
record sampled while the timings ran.  The same commands (with ``--iters 1 --warmup 1``)
are what the profiles under ``profiles/`` were captured from.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics

import torch

from . import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def peaks():
    path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.isfile(path):
        with open(path) as f:
            p = json.load(f)
        return float(p['hbm_gbs']), float(p['bf16_tflops']), 'measured'
    return 6650.0, 1590.0, 'fallback'


class Timer:
    def __init__(self, warmup: int, iters: int):
        self.warmup, self.iters = warmup, iters
        self.flush = torch.empty(256 * 1024 * 1024 // 4, device='cuda')      # 256 MB > 126 MB L2

    def __call__(self, fn) -> float:
        for _ in range(self.warmup):
            fn()
        times = []
        for _ in range(self.iters):
            self.flush.fill_(0.0)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        return statistics.median(times)


def report(name: str, ms: float, nbytes: float = 0.0, flops: float = 0.0) -> dict:
    hbm, tflops, kind = peaks()
    out = {'kernel': name, 'ms': ms}
    if nbytes:
        gbs = nbytes / ms / 1e6
        out.update(algorithmic_GB=nbytes / 1e9, GBps=gbs, frac_of_hbm_peak=gbs / hbm)
    if flops:
        tf = flops / ms / 1e9
        out.update(TFLOPs=tf)
    if nbytes or flops:
        t_mem = nbytes / (hbm * 1e9) * 1e3
        t_math = flops / (tflops * 0.5 * 1e12) * 1e3          # TF32 dense peak = half of the bf16 figure
        out.update(roofline_ms=max(t_mem, t_math), frac_of_roofline=max(t_mem, t_math) / ms, peaks=kind)
    print(json.dumps(out))
    return out


def bench_bn(args, timer):
    from .bn_relu import bn_relu
    M, Cc = args.rows, args.channels
    x = torch.randn(M, Cc, device='cuda', requires_grad=True)
    res = torch.randn(M, Cc, device='cuda') if args.residual else None
    w = torch.ones(Cc, device='cuda', requires_grad=True)
    b = torch.zeros(Cc, device='cuda', requires_grad=True)
    rm, rv, nbt = torch.zeros(Cc, device='cuda'), torch.ones(Cc, device='cuda'), torch.zeros((), dtype=torch.long, device='cuda')
    y = [None]

    def fwd():
        y[0] = bn_relu(x, w, b, rm, rv, nbt, res, True, 0.1, 1e-5)
    nb = M * Cc * 4
    report('bn_relu_fwd[%dx%d]' % (M, Cc), timer(fwd), nbytes=(3 + (1 if args.residual else 0)) * nb)
    dy = torch.randn(M, Cc, device='cuda')

    def bwd():          # autograd.grad: no accumulation into leaf .grad tensors, only the kernels under test
        torch.autograd.grad(y[0], [x, w, b], dy, retain_graph=True)
    report('bn_relu_bwd[%dx%d]' % (M, Cc), timer(bwd), nbytes=5 * nb)


def bench_sgd(args, timer):
    import mgwfbp_b200 as hvd
    sizes, left = [], args.numel
    while left > 0:                      # a ResNet-like mix of large and tiny tensors
        for n in (2359296, 1048576, 512, 65536, 2048):
            n = min(n, left)
            if n:
                sizes.append(n)
                left -= n
    params = [torch.nn.Parameter(torch.randn(n, device='cuda')) for n in sizes]
    opt = hvd.DistributedOptimizer(torch.optim.SGD(params, lr=0.1, momentum=0.9, weight_decay=1e-4),
                                   named_parameters=[('p%d' % i, p) for i, p in enumerate(params)])
    for p in params:
        p.grad = torch.randn_like(p)
    report('multi_tensor_sgd[%d tensors, %d elements]' % (len(sizes), args.numel), timer(opt.step), nbytes=5 * 4 * args.numel)


def bench_wgrad(args, timer):
    from . import wgrad
    from .tables import HyperTable
    K, M, N = args.k, args.m, args.n
    dy, x = torch.randn(K, M, device='cuda'), torch.randn(K, N, device='cuda')
    flops = 2.0 * K * M * N
    if args.sgd:
        w, mom = torch.randn(M, N, device='cuda'), torch.zeros(M, N, device='cuda')
        hyper = HyperTable(torch.device('cuda'))
        hyper.sync([{'lr': 0.01, 'weight_decay': 1e-4, 'momentum': 0.9, 'dampening': 0.0, 'nesterov': False}])
        fn = lambda: wgrad.wgrad_sgd_(dy, x, w, mom, hyper.data_ptr(), 0, scale=0.125)
        report('wgrad_gemm_sm100+sgd[K=%d M=%d N=%d]' % (K, M, N), timer(fn), nbytes=4.0 * (4 * M * N + K * (M + N)), flops=flops)
    else:
        out = torch.empty(M, N, device='cuda')
        fn = lambda: wgrad.wgrad_gemm(dy, x, out=out)
        report('wgrad_gemm_sm100[K=%d M=%d N=%d]' % (K, M, N), timer(fn), nbytes=4.0 * (M * N + K * (M + N)), flops=flops)
        prev = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = True
        report('cublas_tf32 dy^T@x[K=%d M=%d N=%d]' % (K, M, N), timer(lambda: torch.mm(dy.t(), x, out=out)),
               nbytes=4.0 * (M * N + K * (M + N)), flops=flops)
        torch.backends.cuda.matmul.allow_tf32 = prev
    wgrad.check_status()


def bench_pack(args, timer):
    from ..parallel.comm.nvl import NvlComm
    comm = NvlComm.shared()
    x = torch.randn(args.numel, device='cuda')
    for algo in ('oneshot', 'twoshot'):
        if algo == 'oneshot' and args.numel * 4 > comm.oneshot_max_bytes:
            continue
        fn = lambda: comm.synchronize(comm.allreduce_async_(x, algo=algo))
        report('allreduce_fused[%s, world 1, %d elements]' % (algo, args.numel), timer(fn), nbytes=4.0 * 4 * args.numel)
    comm.check_status(synchronize=True)


def bench_fused(args, timer):
    """The whole gradient set of ResNet-50 as ONE merged group through the fused all-reduce + SGD kernel at world
    size 1 (pack, staging, self-barriers, 1/N, update): the kernel's streaming rate without any NVLink traffic.
    Algorithmic bytes: gradient read, parameter and momentum read + write (+ gradient write-back when enabled)."""
    import torchvision
    from .. import settings
    import mgwfbp_b200 as hvd
    from ..parallel.comm.nvl import NvlComm
    comm = NvlComm.shared()
    net = torchvision.models.resnet50().cuda()
    opt = hvd.DistributedOptimizer(torch.optim.SGD(net.parameters(), lr=0.01, momentum=0.9, weight_decay=1e-4),
                                   named_parameters=net.named_parameters(), threshold=1 << 40, comm=comm)
    assert opt._fused_comm and opt._fused_update and len(opt._groups) == 1
    n = 0
    for p in net.parameters():
        p.grad = torch.randn_like(p) * 1e-3
        n += p.numel()
    plan = comm._plans[id(opt)][0]

    def fn():
        comm.launch_group(opt, 0)
        comm.wait_groups(opt, [0])
    passes = 6.0 if settings.WRITE_BACK_GRADS else 5.0
    report('allreduce_fused+sgd[%s, world 1, resnet50 %d elements, %d CTAs x %d threads]'
           % ({0: 'oneshot', 1: 'twoshot', 2: 'nvls'}[plan.algo], n, plan.n_ctas, comm.n_threads), timer(fn), nbytes=passes * 4 * n)
    comm.check_status(synchronize=True)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument('what', choices=['bn', 'sgd', 'wgrad', 'pack', 'fused'])
    ap.add_argument('--rows', type=int, default=200704)
    ap.add_argument('--channels', type=int, default=256)
    ap.add_argument('--residual', action='store_true')
    ap.add_argument('--numel', type=int, default=25557032)
    ap.add_argument('--k', type=int, default=64)
    ap.add_argument('--m', type=int, default=4096)
    ap.add_argument('--n', type=int, default=25088)
    ap.add_argument('--sgd', action='store_true')
    ap.add_argument('--iters', type=int, default=10)
    ap.add_argument('--warmup', type=int, default=3)
    args = ap.parse_args(argv)
    _lib.load(allow_build=False)
    timer = Timer(args.warmup, args.iters)
    from ..utils.clocks import ClockSampler
    sampler = ClockSampler(torch.cuda.current_device()).start()
    try:
        _run(args, timer)
    finally:
        # the SM clock seen while the kernels above were timed (median of the samples under load), read-only
        print(json.dumps({'clocks': sampler.stop()}))


def _run(args, timer):
    {'bn': bench_bn, 'sgd': bench_sgd, 'wgrad': bench_wgrad, 'pack': bench_pack, 'fused': bench_fused}[args.what](args, timer)


if __name__ == '__main__':
    main()
