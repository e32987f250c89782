# -*- coding: utf-8 -*-
"""Penn Treebank reader.

Same behaviour as reference ``ptb_reader.py:9-102``: sentences are joined with ``<eos>``, the
vocabulary is sorted by descending frequency then alphabetically, and the datasets serve
non-overlapping windows ``(x[t:t+T], x[t+1:t+T+1])`` whose count is truncated to a multiple of
the batch size.
"""
from __future__ import annotations

import collections
import os
from typing import Dict, List, Tuple

import numpy as np
from torch.utils.data import Dataset


def _read_words(filename: str) -> List[str]:
    with open(filename, 'r') as f:
        return f.read().replace('\n', '<eos>').split()


def _build_vocab(filename: str) -> Tuple[Dict[str, int], Dict[int, str]]:
    counts = collections.Counter(_read_words(filename))
    ordered = sorted(counts.items(), key=lambda kv: (-kv[1], kv[0]))
    word_to_id = {w: i for i, (w, _) in enumerate(ordered)}
    return word_to_id, {i: w for w, i in word_to_id.items()}


def _file_to_word_ids(filename: str, word_to_id: Dict[str, int]) -> List[int]:
    return [word_to_id[w] for w in _read_words(filename) if w in word_to_id]


def ptb_raw_data(data_path: str, prefix: str = 'ptb'):
    """Returns ``(train_ids, valid_ids, test_ids, word_to_id, id_to_word)``."""
    paths = [os.path.join(data_path, '%s.%s.txt' % (prefix, split)) for split in ('train', 'valid', 'test')]
    word_to_id, id_to_word = _build_vocab(paths[0])
    train, valid, test = (_file_to_word_ids(p, word_to_id) for p in paths)
    return train, valid, test, word_to_id, id_to_word


class _WindowDataset(Dataset):
    def __init__(self, raw_data, batch_size: int, num_steps: int):
        self.raw_data = np.asarray(raw_data, dtype=np.int64)
        self.batch_size, self.num_steps = batch_size, num_steps
        self.data_len = len(self.raw_data)
        self.sample_len = self.data_len // num_steps

    def __getitem__(self, idx):
        lo, hi = self.num_steps * idx, self.num_steps * (idx + 1)
        return self.raw_data[lo:hi], self.raw_data[lo + 1:hi + 1]

    def __len__(self):
        return self.sample_len - self.sample_len % self.batch_size


class TrainDataset(_WindowDataset):
    pass


class TestDataset(_WindowDataset):
    pass
