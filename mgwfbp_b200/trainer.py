# -*- coding: utf-8 -*-
"""``DLTrainer``: model + data + loss + learning-rate schedule + checkpoints for one worker.

Public surface of the reference's ``dl_trainer.py::DLTrainer`` (``:138-953``): ``train(n, hidden=)``,
``test(epoch)``, ``update_model()``, ``update_optimizer(opt)``, ``zero_grad()``, ``data_iter()``,
``get_data_shape()``, ``get/set_train_epoch/iter()``, ``load_model_from_file()``,
``save_checkpoint()``, ``adjust_learning_rate()``, ``update_nworker()``; same per-dataset
hyper-parameters (``:216-229``), decay / no-decay parameter groups (``:231-248``) and schedules
(``:578-709``).

What differs in mechanism: losses and accuracies stay on the device and are only read back when
they are logged (the reference's per-iteration ``loss.item()`` ends every overlap window early);
inputs are copied from pinned memory on the current stream; a synthetic-data mode exists; the
checkpoint whose file name the reference computes is actually written.
"""
from __future__ import annotations

import contextlib
import math
import os
import time
from typing import Any, List, Optional, Tuple

import numpy as np
import torch
import torch.nn as nn
import torch.optim as optim

from . import settings
from .settings import logger
from .models import create_net, repackage_hidden, _support_datasets, _support_dnns  # noqa: F401
from .parallel import runtime
from .utils import checkpoint as ckpt
from .utils.misc import create_path

NUM_CPU_THREADS = 1
SYNTHETIC = 'synthetic'


def _is_synthetic(data_dir: Optional[str]) -> bool:
    return settings.FAKE_DATA or (isinstance(data_dir, str) and data_dir.lower() == SYNTHETIC)


class DLTrainer:
    def __init__(self, rank, size, master='gpu10', dist=True, ngpus=1, batch_size=32, is_weak_scaling=True,
                 data_dir='./data', dataset='cifar10', dnn='resnet20', lr=0.04, nworkers=1, prefix=None,
                 sparsity=0.95, pretrain=None, num_steps=35, tb_writer=None, amp_handle=None,
                 fuse: Optional[bool] = None, channels_last: Optional[bool] = None, seed: Optional[int] = None,
                 weight_decay: Optional[float] = None, momentum: Optional[float] = None):
        self.size, self.rank = size, rank
        self.pretrain, self.dataset, self.prefix = pretrain, dataset, prefix
        self.num_steps, self.ngpus, self.writer, self.amp_handle = num_steps, ngpus, tb_writer, amp_handle
        self.batch_size = batch_size * ngpus if (ngpus > 0 and is_weak_scaling) else batch_size
        self.num_batches_per_epoch = -1
        self.num_classes = {'cifar10': 10, 'mnist': 10, 'imagenet': 1000, 'an4': 29, 'ptb': 10}[dataset]
        self.nworkers = nworkers
        self.data_dir = data_dir
        self.is_cuda = ngpus > 0 and torch.cuda.is_available()
        self.device = torch.device('cuda', torch.cuda.current_device()) if self.is_cuda else torch.device('cpu')
        if self.is_cuda:
            # as the reference does at import time (dl_trainer.py:19-21): let cuDNN time its algorithms per shape;
            # MGWFBP_CUDNN_BENCHMARK_LIMIT widens (0 = all) or narrows how many candidates it tries
            torch.backends.cudnn.benchmark = True
            if settings.CUDNN_BENCHMARK_LIMIT >= 0:
                torch.backends.cudnn.benchmark_limit = settings.CUDNN_BENCHMARK_LIMIT
        self.fp16 = bool(settings.FP16 and self.is_cuda)
        self.loss_scale = float(settings.LOSS_SCALE) if self.fp16 else 1.0
        self.fuse = (self.is_cuda and settings.FUSE_MODULES) if fuse is None else bool(fuse)
        self.channels_last = (self.is_cuda and settings.CHANNELS_LAST) if channels_last is None else bool(channels_last)
        if seed is not None:
            torch.manual_seed(seed)
        self.train_sampler = None
        self.trainset = self.testset = self.trainloader = self.testloader = None
        self.data_iterator = None
        self.vocab_size = 10000
        self.ext = None
        if not isinstance(dnn, str):
            self.net, self.dnn = dnn, dnn.name
            if data_dir is not None:
                self.data_prepare()
        else:
            self.dnn = dnn
            if data_dir is not None and dnn != 'lstman4':
                self.data_prepare()
            kwargs = {}
            if dnn == 'lstm':
                kwargs = dict(vocab_size=self.vocab_size, batch_size=self.batch_size, num_steps=self.num_steps,
                              fused_lstm=self.fuse and settings.FUSE_LSTM)
            elif dnn == 'lstman4':
                kwargs = dict(datapath=None if _is_synthetic(data_dir) else data_dir)
            is_conv = dnn not in ('lstm', 'lstman4', 'fcn5net', 'lr')
            self.net, self.ext = create_net(self.num_classes, dnn, fuse=self.fuse,
                                            channels_last=self.channels_last and is_conv, **kwargs)
            if data_dir is not None and dnn == 'lstman4':
                self.data_prepare()
        self.lr = self.base_lr = lr
        rows = self.batch_size * (self.num_steps if self.dnn == 'lstm' else 1)
        for m in self.net.modules():
            if hasattr(m, 'batch_rows_hint'):
                m.batch_rows_hint = rows          # rows each rank feeds a linear layer per step
        if self.is_cuda:
            if self.ngpus > 1:
                self.net = nn.DataParallel(self.net, device_ids=list(range(self.ngpus))).cuda()
            else:
                self.net.to(self.device)
        self.accuracy, self.loss_value = 0, 0.0
        self.train_iter = self.train_epoch = 0
        self.master = master
        if dist:
            runtime.init()
        if self.dataset != 'an4':
            self.criterion = nn.CrossEntropyLoss().to(self.device)
        else:
            self.criterion = nn.CTCLoss(blank=0, reduction='sum', zero_infinity=True)

        # per-dataset hyper-parameters (reference dl_trainer.py:216-229)
        wd, self.m, nesterov = 1e-4, 0.9, False
        if self.dataset == 'an4':
            self.lstman4_lr_epoch_tag = 0
        elif self.dataset == 'ptb':
            self.m, wd = 0, 0
        elif self.dataset == 'imagenet':
            self.m, wd = 0.875, 2 * 3.0517578125e-05
        if weight_decay is not None:
            wd = weight_decay
        if momentum is not None:
            self.m = momentum
        decay, no_decay = [], []
        for name, p in self.net.named_parameters():
            if not p.requires_grad:
                continue
            (no_decay if (p.dim() == 1 or 'bn' in name or 'bias' in name) else decay).append(p)
        groups = [{'params': no_decay, 'weight_decay': 0.}, {'params': decay, 'weight_decay': wd}]
        self.optimizer = optim.SGD(groups, lr=self.lr, momentum=self.m, weight_decay=wd, nesterov=nesterov)

        if self.pretrain is not None and os.path.isfile(self.pretrain):
            self.load_model_from_file(self.pretrain)

        self.sparsity, self.target_sparsities = sparsity, [1.]
        self.avg_loss_per_epoch = 0.0
        self.timer = self.forwardtime = self.backwardtime = self.iotime = 0.0
        self.epochs_info: List[float] = []
        self.train_acc_top1: List[Any] = []
        self._acc_sum_t, self._acc_steps = None, 0
        self.num_of_updates_during_comm = 0
        self._loss_t: Optional[torch.Tensor] = None       # loss of the last train() call, on device
        self._epoch_loss_t: Optional[torch.Tensor] = None
        logger.info('num_batches_per_epoch: %d' % self.num_batches_per_epoch)

    # ------------------------------------------------------------------ simple accessors
    @property
    def loss(self) -> float:
        """Mean loss of the last ``train()`` call (reads the device value on access)."""
        if self._loss_t is not None:
            self.loss_value = float(self._loss_t)
        return self.loss_value

    @loss.setter
    def loss(self, v):
        self._loss_t, self.loss_value = None, float(v)

    def get_acc(self):
        return self.accuracy

    def get_loss(self):
        return self.loss

    def get_model_state(self):
        return self.net.state_dict()

    def get_data_shape(self):
        return self._input_shape, self._output_shape

    def get_train_epoch(self):
        return self.train_epoch

    def get_train_iter(self):
        return self.train_iter

    def set_train_epoch(self, epoch):
        self.train_epoch = epoch

    def set_train_iter(self, iteration):
        self.train_iter = iteration

    def get_num_of_training_samples(self):
        return len(self.trainset)

    def update_optimizer(self, optimizer):
        self.optimizer = optimizer
        if self.loss_scale != 1.0:
            if not hasattr(optimizer, 'set_grad_scale'):
                raise ValueError('FP16 training scales the loss; wrap the optimizer in DistributedOptimizer so the update divides it out')
            optimizer.set_grad_scale(1.0 / self.loss_scale)

    def autocast(self):
        """Context of the forward pass: half-precision math when ``settings.FP16`` (reference: apex amp O2)."""
        if self.fp16:
            return torch.autocast('cuda', dtype=torch.float16)
        return contextlib.nullcontext()

    def backward(self, loss) -> None:
        """``loss.backward()`` with the static loss scale of the FP16 mode (reference dl_trainer.py:821)."""
        if self.loss_scale != 1.0:
            (loss * self.loss_scale).backward()
        else:
            loss.backward()

    def zero_grad(self):
        self.optimizer.zero_grad()

    def update_model(self):
        self.optimizer.step()

    def print_weight_gradient_ratio(self):
        """Weight histograms to the TensorBoard writer, if one was given (rank 0 only)."""
        if self.rank == 0 and self.writer is not None:
            for name, param in self.net.named_parameters():
                self.writer.add_histogram(name, param.detach().cpu().numpy(), self.train_epoch)

    def finish(self):
        if self.writer is not None:
            self.writer.close()

    # ------------------------------------------------------------------ checkpoints
    def load_model_from_file(self, filename):
        c = ckpt.load_checkpoint(filename, map_location='cpu')
        self.net.load_state_dict(c['state'])
        self.train_epoch, self.train_iter = c['epoch'], c['iter']
        logger.info('Load pretrain model: %s, start from epoch %d and iter: %d', filename, self.train_epoch, self.train_iter)

    def checkpoint_path(self, epoch: Optional[int] = None, root: str = './weights') -> str:
        d = ckpt.checkpoint_dir(self.dnn, self.nworkers, self.batch_size, self.base_lr, self.prefix, root)
        return os.path.join(d, ckpt.checkpoint_name(self.dnn, self.rank, self.train_epoch if epoch is None else epoch))

    def save_checkpoint(self, state=None, filename=None):
        """``save_checkpoint()`` writes the current model to the conventional path;
        ``save_checkpoint(state, filename)`` keeps the reference's two-argument form."""
        if state is None:
            state = {'iter': self.train_iter, 'epoch': self.train_epoch, 'state': self.get_model_state()}
        if filename is None:
            filename = self.checkpoint_path()
        return ckpt.save_checkpoint(filename, state['state'], state['epoch'], state['iter'])

    # ------------------------------------------------------------------ data
    def _loader(self, dataset, train: bool, collate=None, drop_last=False):
        sampler, shuffle = None, train
        if train and self.nworkers > 1:
            sampler = torch.utils.data.distributed.DistributedSampler(dataset, num_replicas=self.nworkers, rank=self.rank)
            sampler.set_epoch(0)
            shuffle = False
            self.train_sampler = sampler
        kw = dict(collate_fn=collate) if collate is not None else {}
        return torch.utils.data.DataLoader(dataset, batch_size=self.batch_size, shuffle=shuffle, sampler=sampler,
                                           num_workers=NUM_CPU_THREADS if train else 1, pin_memory=self.is_cuda,
                                           drop_last=drop_last, **kw)

    def _synthetic_images(self, shape, n_train, n_test):
        from .data.synthetic import SyntheticImages, SyntheticLoader, image_batch_maker
        self.trainset = SyntheticImages(shape, self.num_classes, n_train)
        self.testset = SyntheticImages(shape, self.num_classes, n_test, seed=1)
        per_epoch = max(n_train // (self.batch_size * self.nworkers), 1)
        make = image_batch_maker(self.batch_size, shape, self.num_classes)
        self.trainloader = SyntheticLoader(make, per_epoch, pin=self.is_cuda, seed=self.rank)
        self.testloader = SyntheticLoader(make, max(min(n_test // self.batch_size, 8), 1), ring=2, pin=self.is_cuda, seed=977)

    def imagenet_prepare(self):
        image_size = 224
        self._input_shape = (self.batch_size, 3, image_size, image_size)
        self._output_shape = (self.batch_size, 1000)
        if _is_synthetic(self.data_dir):
            from .data.synthetic import NOMINAL_LENGTH
            return self._synthetic_images((3, image_size, image_size), *NOMINAL_LENGTH['imagenet'])
        import torchvision.transforms as T
        from .data.hdf5 import DatasetHDF5
        norm = T.Normalize(mean=[0.485, 0.456, 0.406], std=[0.229, 0.224, 0.225])
        fn = os.path.join(self.data_dir, 'imagenet-shuffled.hdf5')
        self.trainset = DatasetHDF5(fn, 'train', T.Compose([T.ToPILImage(), T.RandomResizedCrop(image_size),
                                                            T.RandomHorizontalFlip(), T.ToTensor(), norm]))
        self.testset = DatasetHDF5(fn, 'val', T.Compose([T.ToPILImage(), T.Resize(256), T.CenterCrop(224), T.ToTensor(), norm]))
        self.trainloader = self._loader(self.trainset, True)
        self.testloader = self._loader(self.testset, False)

    def cifar10_prepare(self):
        self._input_shape = (self.batch_size, 3, 32, 32)
        self._output_shape = (self.batch_size, 10)
        if _is_synthetic(self.data_dir):
            from .data.synthetic import NOMINAL_LENGTH
            return self._synthetic_images((3, 32, 32), *NOMINAL_LENGTH['cifar10'])
        import torchvision
        import torchvision.transforms as T
        norm = T.Normalize(mean=[0.491, 0.482, 0.447], std=[0.247, 0.243, 0.262])
        self.trainset = torchvision.datasets.CIFAR10(root=self.data_dir, train=True, download=True, transform=T.Compose(
            [T.RandomCrop(32, padding=4), T.RandomHorizontalFlip(), T.ToTensor(), norm]))
        self.testset = torchvision.datasets.CIFAR10(root=self.data_dir, train=False, download=True,
                                                    transform=T.Compose([T.ToTensor(), norm]))
        self.trainloader = self._loader(self.trainset, True)
        self.testloader = self._loader(self.testset, False)
        self.classes = ('plane', 'car', 'bird', 'cat', 'deer', 'dog', 'frog', 'horse', 'ship', 'truck')

    def mnist_prepare(self):
        side = 32 if self.dnn == 'lenet' else 28
        self._input_shape = (self.batch_size, 1, side, side)
        self._output_shape = (self.batch_size, 10)
        if _is_synthetic(self.data_dir):
            from .data.synthetic import NOMINAL_LENGTH
            return self._synthetic_images((1, side, side), *NOMINAL_LENGTH['mnist'])
        import torchvision
        import torchvision.transforms as T
        steps = ([T.Resize((32, 32))] if self.dnn == 'lenet' else []) + [T.ToTensor(), T.Normalize((0.1307,), (0.3081,))]
        self.trainset = torchvision.datasets.MNIST(self.data_dir, train=True, download=True, transform=T.Compose(steps))
        self.testset = torchvision.datasets.MNIST(self.data_dir, train=False, transform=T.Compose(steps))
        self.trainloader = self._loader(self.trainset, True)
        self.testloader = self._loader(self.testset, False)

    def ptb_prepare(self):
        self._input_shape = (self.batch_size, self.num_steps)
        self._output_shape = (self.batch_size, self.num_steps)
        if _is_synthetic(self.data_dir):
            from .data.synthetic import NOMINAL_LENGTH, SyntheticTokens, SyntheticLoader, token_batch_maker
            n_train, n_test = NOMINAL_LENGTH['ptb']
            self.vocab_size = 10000
            self.trainset = SyntheticTokens(self.vocab_size, self.num_steps, n_train, self.batch_size)
            self.testset = SyntheticTokens(self.vocab_size, self.num_steps, n_test, self.batch_size, seed=1)
            make = token_batch_maker(self.batch_size, self.num_steps, self.vocab_size)
            self.trainloader = SyntheticLoader(make, max(len(self.trainset) // (self.batch_size * self.nworkers), 1),
                                               pin=self.is_cuda, seed=self.rank)
            self.testloader = SyntheticLoader(make, 4, ring=2, pin=self.is_cuda, seed=977)
            return
        from .data import ptb as ptb_reader
        train, valid, test, word_to_id, id_to_word = ptb_reader.ptb_raw_data(self.data_dir)
        self.vocab_size = len(word_to_id)
        self.trainset = ptb_reader.TrainDataset(train, self.batch_size, self.num_steps)
        self.testset = ptb_reader.TestDataset(valid, self.batch_size, self.num_steps)
        self.trainloader = self._loader(self.trainset, True, drop_last=True)
        self.testloader = self._loader(self.testset, False, drop_last=True)

    def an4_prepare(self):
        self._input_shape = (self.batch_size, 1, 161, -1)
        self._output_shape = (self.batch_size, 29)
        from .data.an4 import GreedyDecoder
        labels = self.ext['labels'] if self.ext else None
        self.decoder = GreedyDecoder(labels) if labels else None
        if _is_synthetic(self.data_dir):
            from .data.synthetic import NOMINAL_LENGTH, SyntheticLoader, spectrogram_batch_maker
            n_train, n_test = NOMINAL_LENGTH['an4']

            class _Sized:
                def __init__(self, n):
                    self.n = n

                def __len__(self):
                    return self.n
            self.trainset, self.testset = _Sized(n_train), _Sized(n_test)
            make = spectrogram_batch_maker(self.batch_size)
            self.trainloader = SyntheticLoader(make, max(n_train // (self.batch_size * self.nworkers), 1), pin=False, seed=self.rank)
            self.testloader = SyntheticLoader(make, 2, ring=2, pin=False, seed=977)
            return
        from .data.an4 import AudioDataLoader, SpectrogramDataset
        conf = self.ext['audio_conf']
        self.trainset = SpectrogramDataset(conf, os.path.join(self.data_dir, 'an4_train_manifest.csv'), labels)
        self.testset = SpectrogramDataset(conf, os.path.join(self.data_dir, 'an4_val_manifest.csv'), labels)
        sampler = None
        if self.nworkers > 1:
            sampler = torch.utils.data.distributed.DistributedSampler(self.trainset, num_replicas=self.nworkers, rank=self.rank)
            self.train_sampler = sampler
        self.trainloader = AudioDataLoader(self.trainset, batch_size=self.batch_size, num_workers=4,
                                           shuffle=sampler is None, sampler=sampler)
        self.testloader = AudioDataLoader(self.testset, batch_size=self.batch_size, num_workers=4)

    def data_prepare(self):
        prepare = {'imagenet': self.imagenet_prepare, 'cifar10': self.cifar10_prepare, 'mnist': self.mnist_prepare,
                   'an4': self.an4_prepare, 'ptb': self.ptb_prepare}.get(self.dataset)
        if prepare is None:
            raise ValueError('Unsupport dataset: %s' % self.dataset)
        prepare()
        self.data_iterator = None
        n = self.get_num_of_training_samples()
        self.num_batches_per_epoch = (n + self.batch_size * self.nworkers - 1) // (self.batch_size * self.nworkers)

    def update_nworker(self, nworkers, new_rank=-1):
        """Re-shard the training set for a changed worker count (elastic resize hook)."""
        if new_rank >= 0:
            rank = new_rank
        else:
            removed = self.nworkers - nworkers
            rank = self.rank - removed if (removed > 0 and self.rank >= removed) else self.rank
        self.rank, self.nworkers = rank, nworkers
        if self.dnn != 'lstman4' and self.trainset is not None and not _is_synthetic(self.data_dir):
            self.trainloader = self._loader(self.trainset, True)
            if self.train_sampler is not None:
                self.train_sampler.set_epoch(self.train_epoch)
        elif self.trainset is not None:
            self.data_prepare()
        self.data_iterator = None
        n = self.get_num_of_training_samples()
        self.num_batches_per_epoch = (n + self.batch_size * nworkers - 1) // (self.batch_size * nworkers)

    def data_iter(self):
        if self.data_iterator is None:
            self.data_iterator = iter(self.trainloader)
        try:
            return next(self.data_iterator)
        except StopIteration:
            self.data_iterator = iter(self.trainloader)
            return next(self.data_iterator)

    # ------------------------------------------------------------------ learning-rate schedules
    def _set_lr(self, optimizer, lr):
        self.lr = lr
        for g in optimizer.param_groups:
            g['lr'] = lr
        return lr

    def _adjust_learning_rate_lstman4(self, progress, optimizer):
        if self.lstman4_lr_epoch_tag != progress:       # anneal by 1.01 once per epoch
            self.lstman4_lr_epoch_tag = progress
            for g in optimizer.param_groups:
                g['lr'] /= 1.01
            self.lr = self.lr / 1.01
        return self.lr

    def _adjust_learning_rate_lstmptb(self, progress, optimizer):
        # boundaries 63 / 60 / 80: the x0.1 stage is unreachable, as in the reference (:595-610)
        if progress < 63:
            lr = self.base_lr
        elif progress < 60:
            lr = self.base_lr * 0.1
        elif progress < 80:
            lr = self.base_lr * 0.01
        else:
            lr = self.base_lr * 0.001
        return self._set_lr(optimizer, lr)

    def _warmup_lr(self, base_lr, first_epoch, last_epoch):
        total = (last_epoch - first_epoch) * self.num_batches_per_epoch
        lo = base_lr / total
        return lo + (base_lr - lo) / total * (self.train_iter - first_epoch * self.num_batches_per_epoch)

    def _adjust_learning_rate_general(self, progress, optimizer):
        warmup = 5
        if settings.WARMUP and progress < warmup:
            return self._set_lr(optimizer, self._warmup_lr(self.base_lr, 0, warmup))
        first, second, third = {'imagenet': (30, 60, 80), 'ptb': (24, 60, 80)}.get(self.dataset, (81, 122, 155))
        if progress < first:
            lr = self.base_lr
        elif progress < second:
            lr = self.base_lr * 0.1
        elif progress < third:
            lr = self.base_lr * 0.01
        else:
            lr = self.base_lr * 0.001
        return self._set_lr(optimizer, lr)

    def _adjust_learning_rate_vgg16(self, progress, optimizer):
        if progress > 0 and progress % 25 == 0:
            self.lr = self.base_lr / (2 ** (progress / 25))
        return self._set_lr(optimizer, self.lr)

    def _adjust_learning_rate_customized(self, progress, optimizer):
        warmup = 10
        if settings.WARMUP and progress < warmup:
            lr = self._warmup_lr(self.base_lr, 0, warmup)
        elif progress < 15:
            lr = self.base_lr
        elif progress < 25:
            lr = self.base_lr * 0.1
        elif progress < 35:
            lr = self.base_lr * 0.01
        else:
            lr = self.base_lr * 0.001
        return self._set_lr(optimizer, lr)

    def _adjust_learning_rate_cosine(self, progress, optimizer):
        warmup, max_epochs = 14, 40
        lr = self.lr
        if settings.WARMUP and progress < warmup:
            lr = self._warmup_lr(self.base_lr, 0, warmup)
        elif progress < max_epochs:
            lr = 0.5 * (1 + np.cos(np.pi * (progress - warmup) / (max_epochs - warmup))) * self.base_lr
        return self._set_lr(optimizer, lr)

    def adjust_learning_rate(self, progress, optimizer):
        if self.dnn == 'lstman4':
            return self._adjust_learning_rate_lstman4(self.train_iter // self.num_batches_per_epoch, optimizer)
        if self.dnn == 'lstm':
            return self._adjust_learning_rate_lstmptb(progress, optimizer)
        return self._adjust_learning_rate_general(progress, optimizer)

    # ------------------------------------------------------------------ forward / loss
    def cal_accuracy(self, output, target, topk=(1,)):
        with torch.no_grad():
            maxk = max(topk)
            _, pred = output.topk(maxk, 1, True, True)
            correct = pred.t().eq(target.view(1, -1))
            return [correct[:k].reshape(-1).float().sum(0, keepdim=True).mul_(100.0 / target.size(0)) for k in topk]

    def to_device(self, data):
        """Move one loader batch to the training device (non-blocking from pinned memory)."""
        if self.dataset == 'an4':
            inputs, labels_cpu, pct, tsizes = data
            return inputs.to(self.device, non_blocking=True), labels_cpu, pct, tsizes
        inputs, labels = data
        if self.dnn == 'lstm':
            inputs = inputs.to(self.device, non_blocking=True).t().contiguous()
            labels = labels.to(self.device, non_blocking=True).t().contiguous()
            return inputs, labels
        inputs = inputs.to(self.device, non_blocking=True)
        if self.channels_last and inputs.dim() == 4:
            inputs = inputs.contiguous(memory_format=torch.channels_last)
        return inputs, labels.to(self.device, non_blocking=True)

    def forward_loss(self, data, hidden=None, on_device=False):
        """Forward pass and loss for any supported model.  Returns ``(loss, outputs, labels, hidden)``."""
        batch = data if on_device else self.to_device(data)
        if self.dnn == 'lstman4':
            inputs, labels_cpu, pct, tsizes = batch
            in_sizes = pct.mul(int(inputs.size(3))).int()
            out, out_sizes = self.net(inputs, in_sizes)
            logp = out.transpose(0, 1).log_softmax(2)
            loss = self.criterion(logp, labels_cpu.long(), out_sizes.long(), tsizes.long()) / inputs.size(0)
            return loss, out, labels_cpu, None
        if self.dnn == 'lstm':
            inputs, labels = batch
            if hidden is None or (isinstance(hidden, str) and hidden == 'fresh'):
                hidden = self.net.init_hidden()
            hidden = repackage_hidden(hidden)
            with self.autocast():
                outputs, hidden = self.net(inputs, hidden)
                loss = self.criterion(outputs.view(-1, self.net.vocab_size), labels.reshape(-1))
            return loss.float(), outputs, labels, hidden
        inputs, labels = batch
        with self.autocast():
            outputs = self.net(inputs)
            if isinstance(outputs, tuple):               # inception-v3 with auxiliary logits
                loss = self.criterion(outputs[0], labels) + 0.4 * sum(self.criterion(o, labels) for o in outputs[1:])
                outputs = outputs[0]
            else:
                loss = self.criterion(outputs, labels)
        return loss.float(), outputs, labels, None

    # ------------------------------------------------------------------ training
    def _on_epoch_boundary(self):
        self.train_epoch += 1
        npe = self.num_batches_per_epoch
        logger.info('train iter: %d, num_batches_per_epoch: %d', self.train_iter, npe)
        if self._acc_sum_t is not None:           # accumulated on the device by engine.TrainStep
            acc = float(self._acc_sum_t) / max(self._acc_steps, 1)
        else:
            acc = float(torch.stack([a.reshape(()) for a in self.train_acc_top1]).mean()) if self.train_acc_top1 else float('nan')
        epoch_loss = float(self._epoch_loss_t) if self._epoch_loss_t is not None else self.avg_loss_per_epoch
        logger.info('Epoch %d, avg train acc: %f, lr: %f, avg loss: %f' % (self.train_iter // npe, acc, self.lr, epoch_loss / npe))
        if self.rank == 0 and self.writer is not None:
            self.writer.add_scalar('cross_entropy', epoch_loss / npe, self.train_epoch)
            self.writer.add_scalar('top-1_acc', acc, self.train_epoch)
        self.train_acc_top1 = []
        self._acc_sum_t, self._acc_steps = None, 0
        self.epochs_info.append(epoch_loss / npe)
        self.avg_loss_per_epoch, self._epoch_loss_t = 0.0, None
        if self.train_iter > 0 and self.rank == 0:
            self.save_checkpoint()
        if self.train_sampler is not None and self.nworkers > 1:
            self.train_sampler.set_epoch(self.train_epoch)

    def train(self, num_of_iters=1, data=None, hidden=None):
        s = time.time()
        loss_acc = None
        for _ in range(num_of_iters):
            self.adjust_learning_rate(self.train_epoch, self.optimizer)
            if self.train_iter % self.num_batches_per_epoch == 0 and self.train_iter > 0:
                self._on_epoch_boundary()
            ss = time.time()
            batch = self.to_device(data if data is not None else self.data_iter())
            self.iotime += time.time() - ss
            sf = time.time()
            loss, outputs, labels, hidden = self.forward_loss(batch, hidden, on_device=True)
            self.forwardtime += time.time() - sf
            sb = time.time()
            self.backward(loss)
            self.backwardtime += time.time() - sb
            ld = loss.detach()
            loss_acc = ld if loss_acc is None else loss_acc + ld
            self._epoch_loss_t = ld.clone() if self._epoch_loss_t is None else self._epoch_loss_t + ld
            if self.dnn not in ('lstm', 'lstman4'):
                self.train_acc_top1.append(self.cal_accuracy(outputs.detach(), labels, topk=(1,))[0])
            self.train_iter += 1
        self.num_of_updates_during_comm += 1
        self._loss_t = loss_acc / num_of_iters if loss_acc is not None else None
        self.timer += time.time() - s
        display = 40
        if self.train_iter % display == 0:
            logger.warning('[%3d][%5d/%5d][rank:%d] loss: %.3f, average forward (%f) and backward (%f) time: %f, iotime: %f ' %
                           (self.train_epoch, self.train_iter, self.num_batches_per_epoch, self.rank, self.loss,
                            self.forwardtime / display, self.backwardtime / display, self.timer / display, self.iotime / display))
            self.timer = self.iotime = self.forwardtime = self.backwardtime = 0.0
        if self.dnn == 'lstm':
            return num_of_iters, hidden
        return num_of_iters

    # ------------------------------------------------------------------ evaluation
    def test(self, epoch):
        self.net.eval()
        test_loss, costs, total_steps, total_iters, total, total_wer = 0.0, 0.0, 0, 0, 0, 0.0
        top1, top5 = [], []
        with torch.no_grad():
            for data in self.testloader:
                if self.dnn == 'lstman4':
                    inputs, labels_cpu, pct, tsizes = self.to_device(data)
                    out, out_sizes = self.net(inputs, pct.mul(int(inputs.size(3))).int())
                    decoded, _ = self.decoder.decode(out, out_sizes)
                    off = 0
                    for i, n in enumerate(tsizes.tolist()):
                        ref = self.decoder.convert_to_strings([labels_cpu[off:off + n]])[0][0]
                        off += n
                        total_wer += self.decoder.wer(decoded[i][0], ref) / float(max(len(ref.split()), 1))
                    total += inputs.size(0)
                else:
                    loss, outputs, labels, _ = self.forward_loss(data, hidden='fresh')
                    test_loss += float(loss)
                    if self.dnn == 'lstm':
                        costs += float(loss) * self.net.num_steps
                        total_steps += self.net.num_steps
                    else:
                        a1, a5 = self.cal_accuracy(outputs, labels, topk=(1, 5))
                        top1.append(float(a1))
                        top5.append(float(a5))
                    total += labels.size(0)
                total_iters += 1
        test_loss /= max(total_iters, 1)
        if self.dnn == 'lstm':
            acc, acc5 = float(np.exp(costs / max(total_steps, 1))), 0.0
        elif self.dnn == 'lstman4':
            acc, acc5 = total_wer / max(total, 1), 0.0
        else:
            acc, acc5 = float(np.mean(top1)), float(np.mean(top5))
        logger.info('Epoch %d, lr: %f, val loss: %f, val top-1 acc: %f, top-5 acc: %f' % (epoch, self.lr, test_loss, acc, acc5))
        self.net.train()
        return acc


def train_with_single(dnn, dataset, data_dir, nworkers, lr, batch_size, nsteps_update, max_epochs, num_steps=1,
                      max_iters: Optional[int] = None, use_graph: bool = True):
    """Single-GPU training loop (reference ``dl_trainer.py:956-984``): profiles the backward pass
    once, then trains, logging time per iteration and images/s."""
    from .parallel.optimizer import DistributedOptimizer
    from .utils.profiling import benchmark
    if torch.cuda.is_available():
        torch.cuda.set_device(0)
    trainer = DLTrainer(0, nworkers, dist=False, batch_size=batch_size, is_weak_scaling=True, ngpus=1, data_dir=data_dir,
                        dataset=dataset, dnn=dnn, lr=lr, nworkers=nworkers, prefix='singlegpu', num_steps=num_steps)
    iters_per_epoch = trainer.get_num_of_training_samples() // (nworkers * batch_size * nsteps_update)
    seq_layernames, layerwise_times, layerwise_sizes = benchmark(trainer)
    logger.info('Bencharmked backward time: %f', np.sum(layerwise_times))
    logger.info('Model size: %d', np.sum(layerwise_sizes))
    trainer.update_optimizer(DistributedOptimizer(trainer.optimizer, named_parameters=trainer.net.named_parameters()))
    # one micro-step per update: the graph-captured step with input prefetch; otherwise the accumulation loop
    from .engine import TrainStep
    step = TrainStep(trainer, use_graph=use_graph, track_accuracy=True) if nsteps_update == 1 else None
    if nsteps_update > 1:
        trainer.optimizer.release_external_layers()        # gradients are summed over micro-batches before the update
    upcoming = trainer.data_iter() if step is not None else None
    display = 40 if iters_per_epoch > 40 else max(iters_per_epoch - 1, 1)
    done, counted, since = 0, 0, time.time()
    for epoch in range(max_epochs):
        hidden = trainer.net.init_hidden() if (dnn == 'lstm' and step is None) else None
        if step is not None:
            step.reset_state()
        for i in range(iters_per_epoch):
            if step is not None:
                current, upcoming = upcoming, trainer.data_iter()
                step.run(current, next_host_batch=upcoming)
            else:
                trainer.optimizer.zero_grad()
                for j in range(nsteps_update):
                    if dnn == 'lstm':
                        _, hidden = trainer.train(1, hidden=hidden)
                    else:
                        trainer.train(1)
                trainer.update_model()
            done += 1
            counted += 1
            if i % display == 0 and i > 0:
                if trainer.is_cuda:
                    torch.cuda.synchronize()          # the host runs ahead of the device: close the interval first
                now = time.time()
                t = (now - since) / counted
                logger.info('Time per iteration including communication: %f. Speed: %f images/s', t, batch_size * nsteps_update / t)
                counted, since = 0, now
            if max_iters is not None and done >= max_iters:
                if step is not None:
                    step.drain()
                return trainer
    if step is not None:
        step.drain()
    return trainer
