# -*- coding: utf-8 -*-
"""Distributed training entry point (one process per GPU, launched by ``torchrun``; see ``dist_launch.sh``).

Same flags, log lines and phases as reference ``dist_trainer.py:29-143``: build the trainer, agree on the start
epoch / iteration, profile the backward pass layer by layer (rank 0's times are broadcast so that all ranks derive
the same merge schedule), wrap the optimizer, broadcast the model, then run epochs x iterations.  With one
micro-step per update the iteration is ``mgwfbp_b200.engine.TrainStep`` (input prefetch, asynchronous loss read,
CUDA-graph replay after three eager steps; ``--no-graph`` keeps it eager); with ``--nsteps-update > 1`` the
accumulation loop of the reference is used (``optimizer.local`` on all but the last micro-step).  ``--nworkers``
must equal the launched world size.
"""
from __future__ import annotations

import argparse
import logging
import os
import time
from typing import Optional

import numpy as np
import torch

import mgwfbp_b200 as hvd
from mgwfbp_b200 import settings
from mgwfbp_b200.engine import TrainStep, build_distributed_optimizer
from mgwfbp_b200.settings import formatter, logger
from mgwfbp_b200.trainer import DLTrainer, _support_datasets, _support_dnns
from mgwfbp_b200.utils.compression import compressors
from mgwfbp_b200.utils.misc import create_path
from mgwfbp_b200.utils.profiling import benchmark

writer = None
NORM_CLIP = {'lstm': 0.25, 'lstman4': 400}          # reference dist_trainer.py:56-65 / :89-94


class _SpeedLog:
    """``Time per iteration including communication`` every ``every`` iterations (per-worker samples per second, as
    the reference reports it, dist_trainer.py:97-100).  The host runs ahead of the device, so the interval is closed
    with a device synchronisation and divided by the iterations it contains."""

    def __init__(self, every: int, samples_per_iter: int, cuda: bool):
        self.every, self.samples, self.cuda = max(every, 1), samples_per_iter, cuda
        self.count = 0
        self.since = time.time()

    def tick(self, index_in_epoch: int) -> None:
        self.count += 1
        if index_in_epoch > 0 and index_in_epoch % self.every == 0:
            if self.cuda:
                torch.cuda.synchronize()
            now = time.time()
            mean = (now - self.since) / self.count
            logger.warning('Time per iteration including communication: %f, Speed: %f images/s', mean, self.samples / mean)
            self.count, self.since = 0, now


def _make_trainer(rank, args_like) -> DLTrainer:
    dnn, dataset, data_dir, nworkers, lr, batch_size, pretrain, num_steps = args_like
    trainer = DLTrainer(rank, nworkers, dist=False, batch_size=batch_size, is_weak_scaling=True, ngpus=1, data_dir=data_dir,
                        dataset=dataset, dnn=dnn, lr=lr, nworkers=nworkers, prefix='allreduce',
                        pretrain=pretrain if rank == 0 else None, num_steps=num_steps, tb_writer=writer)
    # only rank 0 read the checkpoint: everyone adopts its position
    epoch, iteration = hvd.broadcast_object((trainer.get_train_epoch(), trainer.get_train_iter()), 0)
    trainer.set_train_epoch(int(epoch))
    trainer.set_train_iter(int(iteration))
    return trainer


def _profile_backward(trainer, rank):
    """(names, times, sizes) in forward order with rank 0's times on every rank, or three ``None`` when off."""
    if not settings.ADAPTIVE_MERGE:
        return None, None, None
    names, times, sizes = benchmark(trainer)
    times = hvd.broadcast_object(list(times), 0)
    if rank == 0:
        logger.info('layerwise backward times: %s', list(times))
        logger.info('layerwise backward sizes: %s', list(sizes))
    logger.info('Bencharmked backward time: %f', np.sum(times))
    logger.info('Model size: %d', np.sum(sizes))
    return names, times, sizes


def _accumulating_iteration(trainer, optimizer, dnn, nsteps_update, hidden):
    optimizer.zero_grad()
    for micro in range(nsteps_update):
        optimizer.local = micro < nsteps_update - 1          # communicate on the last micro-step only
        if dnn == 'lstm':
            _, hidden = trainer.train(1, hidden=hidden)
        else:
            trainer.train(1)
    trainer.update_model()                                    # the global-norm clip happens inside step()
    return hidden


def mgwfbp(dnn, dataset, data_dir, nworkers, lr, batch_size, nsteps_update, max_epochs, nwpernode, pretrain, num_steps,
           compressor, density, threshold, gradient_path=None, max_iters=None, use_graph=True):
    rank = hvd.rank()
    if torch.cuda.is_available():
        torch.cuda.set_device(rank % max(min(nwpernode, torch.cuda.device_count()), 1))
    trainer = _make_trainer(rank, (dnn, dataset, data_dir, nworkers, lr, batch_size, pretrain, num_steps))
    names, times, _sizes = _profile_backward(trainer, rank)
    # wrap the optimizer and broadcast the model (reference dist_trainer.py:55-66).  On an NVSwitch box with the
    # adaptive policy this also fits the all-reduce cost model, measures how much an overlapped message slows backward
    # down, and keeps the candidate schedule that trains fastest; with settings.ORIGINAL_HOROVOD it builds the stock
    # arm instead (NCCL buckets through torch.distributed, torch's own SGD.step).
    optimizer, tuning = build_distributed_optimizer(trainer, seq_layernames=names, layerwise_times=times,
                                                    threshold=threshold, norm_clip=NORM_CLIP.get(dnn),
                                                    compression=compressors[compressor if density < 1 else None],
                                                    writer=writer, gradient_path=gradient_path, use_graph=use_graph)
    if rank == 0 and tuning.get('trial'):
        logger.info('merge schedule chosen by trial: %d groups; candidates %s', len(optimizer.merge_schedule.groups), tuning['trial'])

    iters_per_epoch = trainer.get_num_of_training_samples() // (nworkers * batch_size * nsteps_update)
    speed = _SpeedLog(10 if iters_per_epoch > 10 else iters_per_epoch - 1, batch_size * nsteps_update, trainer.is_cuda)
    step: Optional[TrainStep] = TrainStep(trainer, use_graph=use_graph, track_accuracy=True) if nsteps_update == 1 else None
    upcoming = trainer.data_iter() if step is not None else None
    logger.info('max_epochs: %d', max_epochs)
    done = 0
    for _epoch in range(max_epochs):
        hidden = trainer.net.init_hidden() if (dnn == 'lstm' and step is None) else None
        if step is not None:
            step.reset_state()
        for i in range(iters_per_epoch):
            if step is not None:
                current, upcoming = upcoming, trainer.data_iter()      # the next batch is copied while this one computes
                step.run(current, next_host_batch=upcoming)
            else:
                hidden = _accumulating_iteration(trainer, optimizer, dnn, nsteps_update, hidden)
            speed.tick(i)
            done += 1
            if max_iters is not None and done >= max_iters:
                if step is not None:
                    step.drain()
                return trainer
        optimizer.train_epoch += 1
    if step is not None:
        step.drain()
    return trainer


_FLAGS = (
    # name, type, default, help
    ('--batch-size', int, 32, None),
    ('--nsteps-update', int, 1, None),
    ('--nworkers', int, 1, 'Number of workers; must equal the launched world size'),
    ('--nwpernode', int, 1, 'Number of workers per node'),
    ('--data-dir', str, './data', 'Specify the data root path ("synthetic" for generated data)'),
    ('--saved-dir', str, '.', 'Specify the saved weights or gradients root path'),
    ('--lr', float, 0.1, 'Default learning rate'),
    ('--max-epochs', int, settings.MAX_EPOCHS, 'Default maximum epochs to train'),
    ('--pretrain', str, None, 'Specify the pretrain path'),
    ('--num-steps', int, 35, None),
    ('--compressor', str, 'none', "Specify the compressor if 'compression' is open"),
    ('--density', float, 1, 'Density for sparsification'),
    ('--threshold', int, 0, 'Specify the threshold for gradient merging'),
    ('--max-iters', int, None, 'Stop after this many iterations (smoke runs)'),
)


def build_parser():
    parser = argparse.ArgumentParser(description='AllReduce trainer')
    for name, kind, default, text in _FLAGS:
        parser.add_argument(name, type=kind, default=default, help=text)
    parser.add_argument('--dataset', type=str, default='imagenet', choices=_support_datasets, help='Specify the dataset for training')
    parser.add_argument('--dnn', type=str, default='resnet50', choices=_support_dnns, help='Specify the neural network for training')
    parser.add_argument('--no-graph', action='store_true', help='Do not capture the training step in a CUDA graph')
    return parser


def _log_directory(args) -> str:
    prefix = settings.PREFIX if args.density >= 1 else 'comp-%s-%s' % (args.compressor, settings.PREFIX)
    run = '%s-n%d-bs%d-lr%.4f-ns%d-ds%s' % (args.dnn, args.nworkers, args.batch_size * args.nsteps_update, args.lr,
                                            args.nsteps_update, str(args.density))
    return './logs/allreduce-%s-thres-%dkbytes/%s' % (prefix, args.threshold / 1024, run)


def main(argv=None):
    args = build_parser().parse_args(argv)
    if args.compressor not in compressors:
        args.compressor = 'none'      # the reference's default names a compressor that does not exist
    log_dir = _log_directory(args)
    create_path(log_dir)
    rank = 0
    if args.nworkers > 1:
        hvd.init()
        rank = hvd.rank()
        if hvd.size() != args.nworkers:
            raise SystemExit('--nworkers %d does not match the launched world size %d' % (args.nworkers, hvd.size()))
    handler = logging.FileHandler(os.path.join(log_dir, '%s-%d.log' % (settings.hostname, rank)))
    handler.setFormatter(formatter)
    logger.addHandler(handler)
    logger.info('Configurations: %s', args)
    try:
        mgwfbp(args.dnn, args.dataset, args.data_dir, args.nworkers, args.lr, args.batch_size, args.nsteps_update,
               args.max_epochs, args.nwpernode, args.pretrain, args.num_steps, args.compressor, args.density,
               args.threshold, None, max_iters=args.max_iters, use_graph=not args.no_graph)
    finally:
        hvd.shutdown()


if __name__ == '__main__':
    main()
