# -*- coding: utf-8 -*-
"""Distributed training entry point.

Flags and loop of reference ``dist_trainer.py:29-143``: build the trainer, agree on the start
epoch / iteration, profile the backward pass layer by layer (rank 0's times are broadcast so that
all ranks derive the same merge schedule), wrap the optimizer, broadcast the model, then run
epochs x iterations with gradient accumulation (``--nsteps-update``) and the LSTM gradient clip.
Launch one process per GPU with ``torchrun`` (see ``dist_launch.sh``); ``--nworkers`` must equal
the world size.
"""
from __future__ import print_function

import argparse
import logging
import os
import time

import numpy as np
import torch

import mgwfbp_b200 as hvd
from mgwfbp_b200 import settings
from mgwfbp_b200.settings import logger, formatter
from mgwfbp_b200.trainer import DLTrainer, _support_datasets, _support_dnns
from mgwfbp_b200.utils.compression import compressors
from mgwfbp_b200.utils.misc import create_path
from mgwfbp_b200.utils.profiling import benchmark

writer = None


def mgwfbp(dnn, dataset, data_dir, nworkers, lr, batch_size, nsteps_update, max_epochs, nwpernode, pretrain, num_steps,
           compressor, density, threshold, gradient_path=None, max_iters=None):
    rank = hvd.rank()
    if torch.cuda.is_available():
        torch.cuda.set_device(rank % max(min(nwpernode, torch.cuda.device_count()), 1))
    if rank != 0:
        pretrain = None
    trainer = DLTrainer(rank, nworkers, dist=False, batch_size=batch_size, is_weak_scaling=True, ngpus=1,
                        data_dir=data_dir, dataset=dataset, dnn=dnn, lr=lr, nworkers=nworkers, prefix='allreduce',
                        pretrain=pretrain, num_steps=num_steps, tb_writer=writer)

    start = hvd.broadcast_object((trainer.get_train_epoch(), trainer.get_train_iter()), 0)
    trainer.set_train_epoch(int(start[0]))
    trainer.set_train_iter(int(start[1]))
    if not density < 1:
        compressor = None

    seq_layernames = layerwise_times = layerwise_sizes = None
    if settings.ADAPTIVE_MERGE:
        seq_layernames, layerwise_times, layerwise_sizes = benchmark(trainer)
        layerwise_times = hvd.broadcast_object(list(layerwise_times), 0)
        if rank == 0:
            logger.info('layerwise backward times: %s', list(layerwise_times))
            logger.info('layerwise backward sizes: %s', list(layerwise_sizes))
        logger.info('Bencharmked backward time: %f', np.sum(layerwise_times))
        logger.info('Model size: %d', np.sum(layerwise_sizes))

    norm_clip = {'lstm': 0.25, 'lstman4': 400}.get(dnn)
    optimizer = hvd.DistributedOptimizer(trainer.optimizer, named_parameters=trainer.net.named_parameters(),
                                         compression=compressors[compressor], seq_layernames=seq_layernames,
                                         layerwise_times=layerwise_times, norm_clip=norm_clip, threshold=threshold,
                                         writer=writer, gradient_path=gradient_path)
    hvd.broadcast_parameters(trainer.net.state_dict(), root_rank=0)
    trainer.update_optimizer(optimizer)
    iters_per_epoch = trainer.get_num_of_training_samples() // (nworkers * batch_size * nsteps_update)

    times, done = [], 0
    logger.info('max_epochs: %d', max_epochs)
    display = 10 if iters_per_epoch > 10 else max(iters_per_epoch - 1, 1)
    for epoch in range(max_epochs):
        hidden = trainer.net.init_hidden() if dnn == 'lstm' else None
        for i in range(iters_per_epoch):
            s = time.time()
            optimizer.zero_grad()
            for j in range(nsteps_update):
                optimizer.local = nsteps_update > 1 and j < nsteps_update - 1
                if dnn == 'lstm':
                    _, hidden = trainer.train(1, hidden=hidden)
                else:
                    trainer.train(1)
            # the global-norm clip (0.25 for lstm, 400 for lstman4) is applied inside step()
            trainer.update_model()
            times.append(time.time() - s)
            done += 1
            if i % display == 0 and i > 0:
                if trainer.is_cuda:
                    torch.cuda.synchronize()
                time_per_iter = float(np.mean(times))
                logger.warning('Time per iteration including communication: %f, Speed: %f images/s',
                               time_per_iter, batch_size * nsteps_update / time_per_iter)
                times = []
            if max_iters is not None and done >= max_iters:
                return trainer
        optimizer.train_epoch += 1
    return trainer


def build_parser():
    parser = argparse.ArgumentParser(description='AllReduce trainer')
    parser.add_argument('--batch-size', type=int, default=32)
    parser.add_argument('--nsteps-update', type=int, default=1)
    parser.add_argument('--nworkers', type=int, default=1, help='Number of workers; must equal the launched world size')
    parser.add_argument('--nwpernode', type=int, default=1, help='Number of workers per node')
    parser.add_argument('--dataset', type=str, default='imagenet', choices=_support_datasets, help='Specify the dataset for training')
    parser.add_argument('--dnn', type=str, default='resnet50', choices=_support_dnns, help='Specify the neural network for training')
    parser.add_argument('--data-dir', type=str, default='./data', help='Specify the data root path ("synthetic" for generated data)')
    parser.add_argument('--saved-dir', type=str, default='.', help='Specify the saved weights or gradients root path')
    parser.add_argument('--lr', type=float, default=0.1, help='Default learning rate')
    parser.add_argument('--max-epochs', type=int, default=settings.MAX_EPOCHS, help='Default maximum epochs to train')
    parser.add_argument('--pretrain', type=str, default=None, help='Specify the pretrain path')
    parser.add_argument('--num-steps', type=int, default=35)
    parser.add_argument('--compressor', type=str, default='none', help="Specify the compressor if 'compression' is open")
    parser.add_argument('--density', type=float, default=1, help='Density for sparsification')
    parser.add_argument('--threshold', type=int, default=0, help='Specify the threshold for gradient merging')
    parser.add_argument('--max-iters', type=int, default=None, help='Stop after this many iterations (smoke runs)')
    return parser


def main(argv=None):
    args = build_parser().parse_args(argv)
    if args.compressor not in compressors:
        args.compressor = 'none'      # the reference's default names a compressor that does not exist
    batch_size = args.batch_size * args.nsteps_update
    prefix = settings.PREFIX
    if args.density < 1:
        prefix = 'comp-' + args.compressor + '-' + prefix
    logdir = 'allreduce-%s-thres-%dkbytes/%s-n%d-bs%d-lr%.4f-ns%d-ds%s' % (
        prefix, args.threshold / 1024, args.dnn, args.nworkers, batch_size, args.lr, args.nsteps_update, str(args.density))
    relative_path = './logs/%s' % logdir
    create_path(relative_path)
    rank = 0
    if args.nworkers > 1:
        hvd.init()
        rank = hvd.rank()
        if hvd.size() != args.nworkers:
            raise SystemExit('--nworkers %d does not match the launched world size %d' % (args.nworkers, hvd.size()))
    hdlr = logging.FileHandler(os.path.join(relative_path, settings.hostname + '-' + str(rank) + '.log'))
    hdlr.setFormatter(formatter)
    logger.addHandler(hdlr)
    logger.info('Configurations: %s', args)
    try:
        mgwfbp(args.dnn, args.dataset, args.data_dir, args.nworkers, args.lr, args.batch_size, args.nsteps_update,
               args.max_epochs, args.nwpernode, args.pretrain, args.num_steps, args.compressor, args.density,
               args.threshold, None, max_iters=args.max_iters)
    finally:
        hvd.shutdown()


if __name__ == '__main__':
    main()
