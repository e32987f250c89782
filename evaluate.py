# -*- coding: utf-8 -*-
"""Evaluate saved checkpoints epoch by epoch (flags of reference ``evaluate.py:59-73``).

``--model-path`` is a checkpoint directory ``<dnn>-n<N>-bs<B>-lr<lr>``; files
``<dnn>-rank0-epoch<i>.pth`` for ``i`` in ``[--start-epoch, --nepochs]`` are loaded in turn and the
best top-1 accuracy (or lowest perplexity / WER for the LSTMs) is tracked.
"""
import argparse
import logging
import os

from mgwfbp_b200.settings import logger, formatter
from mgwfbp_b200.trainer import DLTrainer
from mgwfbp_b200.utils.checkpoint import checkpoint_name, parse_checkpoint_dir


def model_average(trainers):
    """Average the weights of several trainers into the first one."""
    first = trainers[0]
    avg = {k: v.clone().float() for k, v in first.net.state_dict().items()}
    for t in trainers[1:]:
        for k, v in t.net.state_dict().items():
            avg[k] += v.float()
    ref = first.net.state_dict()
    first.net.load_state_dict({k: (v / len(trainers)).to(ref[k].dtype) for k, v in avg.items()})
    return first


def evaluate(model_path, dnn, dataset, data_dir, nepochs, allreduce=False, start_epoch=39):
    info = parse_checkpoint_dir(model_path)
    dnn = info['dnn']
    trainer = DLTrainer(0, 1, dist=False, ngpus=1, batch_size=info['batch_size'], is_weak_scaling=True, dataset=dataset,
                        dnn=dnn, data_dir=data_dir, lr=info['lr'], nworkers=1)
    lower_is_better = dnn in ('lstm', 'lstman4')
    best = None
    for epoch in range(start_epoch, nepochs + 1):
        fn = os.path.join(model_path, checkpoint_name(dnn, 0, epoch))
        if not os.path.isfile(fn):
            logger.info('skip missing checkpoint %s', fn)
            continue
        trainer.load_model_from_file(fn)
        acc = trainer.test(epoch)
        if best is None or (acc < best if lower_is_better else acc > best):
            best = acc
        logger.info('Best validation accuracy or perprexity: %f', best)
    return best


def main(argv=None):
    parser = argparse.ArgumentParser(description='model evaluater')
    parser.add_argument('--model-path', type=str, help='Saved model path')
    parser.add_argument('--dnn', type=str, default='resnet20')
    parser.add_argument('--dataset', type=str, default='cifar10')
    parser.add_argument('--data-dir', type=str, default='./data', help='Specify the data root path')
    parser.add_argument('--nepochs', type=int, default=90, help='Number of epochs to evaluate')
    parser.add_argument('--start-epoch', type=int, default=39, help='First epoch to evaluate')
    args = parser.parse_args(argv)
    hdlr = logging.FileHandler('%s/evaluate.log' % args.model_path)
    hdlr.setFormatter(formatter)
    logger.addHandler(hdlr)
    return evaluate(args.model_path, args.dnn, args.dataset, args.data_dir, args.nepochs, start_epoch=args.start_epoch)


if __name__ == '__main__':
    main()
