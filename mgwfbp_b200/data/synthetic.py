# -*- coding: utf-8 -*-
"""Synthetic datasets with the shapes of the real ones.

The reference declares ``settings.FAKE_DATA`` but never implements it (``settings.py:33``); every
run there needs CIFAR/MNIST/ImageNet/PTB on disk.  Here ``data_dir='synthetic'`` (or
``MGWFBP_FAKE_DATA=1``) selects these generators: images ~ N(0,1), labels uniform, token ids
uniform, with the nominal dataset length so that epoch / iteration accounting is unchanged.

``SyntheticLoader`` serves batches from a small ring of pre-generated **pinned** host tensors, so
a training step still performs a real host-to-device copy of its inputs while the host spends no
time generating random numbers.
"""
from __future__ import annotations

from typing import Iterator, List, Optional, Sequence, Tuple

import torch
from torch.utils.data import Dataset

NOMINAL_LENGTH = {'imagenet': (1281167, 50000), 'cifar10': (50000, 10000), 'mnist': (60000, 10000),
                  'ptb': (929589 // 35, 82430 // 35), 'an4': (948, 130)}


class SyntheticImages(Dataset):
    """Deterministic per-index random images; ``len`` equals the real dataset's."""

    def __init__(self, shape: Sequence[int], num_classes: int, length: int, seed: int = 0):
        self.shape, self.num_classes, self.length, self.seed = tuple(shape), num_classes, int(length), seed

    def __len__(self):
        return self.length

    def __getitem__(self, idx):
        g = torch.Generator().manual_seed(self.seed * 1000003 + int(idx))
        return torch.randn(self.shape, generator=g), int(torch.randint(0, self.num_classes, (1,), generator=g))


class SyntheticTokens(Dataset):
    def __init__(self, vocab_size: int, num_steps: int, length: int, batch_size: int = 1, seed: int = 0):
        self.vocab_size, self.num_steps, self.seed = vocab_size, num_steps, seed
        self.length = int(length) - int(length) % max(batch_size, 1)

    def __len__(self):
        return self.length

    def __getitem__(self, idx):
        g = torch.Generator().manual_seed(self.seed * 1000003 + int(idx))
        seq = torch.randint(0, self.vocab_size, (self.num_steps + 1,), generator=g)
        return seq[:-1].numpy(), seq[1:].numpy()


class SyntheticLoader:
    """Endless-per-epoch iterator over ``ring`` pinned batches; ``len`` = batches per epoch."""

    def __init__(self, make_batch, batches_per_epoch: int, ring: int = 4, pin: Optional[bool] = None, seed: int = 0):
        pin = torch.cuda.is_available() if pin is None else pin
        self._batches: List[Tuple[torch.Tensor, ...]] = []
        g = torch.Generator().manual_seed(seed)
        for _ in range(max(ring, 1)):
            batch = make_batch(g)
            if pin:
                batch = tuple(t.pin_memory() for t in batch)
            self._batches.append(batch)
        self._n = int(batches_per_epoch)
        self.dataset = None
        self.sampler = None

    def __len__(self):
        return self._n

    def __iter__(self) -> Iterator[Tuple[torch.Tensor, ...]]:
        for i in range(self._n):
            yield self._batches[i % len(self._batches)]

    def set_epoch(self, epoch: int) -> None:
        pass


def image_batch_maker(batch_size: int, shape: Sequence[int], num_classes: int):
    def make(g):
        return (torch.randn((batch_size,) + tuple(shape), generator=g),
                torch.randint(0, num_classes, (batch_size,), generator=g, dtype=torch.int64))
    return make


def token_batch_maker(batch_size: int, num_steps: int, vocab_size: int):
    def make(g):
        seq = torch.randint(0, vocab_size, (batch_size, num_steps + 1), generator=g, dtype=torch.int64)
        return seq[:, :-1].contiguous(), seq[:, 1:].contiguous()
    return make


def spectrogram_batch_maker(batch_size: int, freq: int = 161, frames: int = 200, num_labels: int = 29, target_len: int = 20):
    def make(g):
        x = torch.randn(batch_size, 1, freq, frames, generator=g)
        targets = torch.randint(1, num_labels, (batch_size * target_len,), generator=g, dtype=torch.int32)
        pct = torch.ones(batch_size)
        sizes = torch.full((batch_size,), target_len, dtype=torch.int32)
        return x, targets, pct, sizes
    return make
