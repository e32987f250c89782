# -*- coding: utf-8 -*-
"""Checkpoint files in the reference's layout.

A checkpoint is ``torch.save({'iter': int, 'epoch': int, 'state': net.state_dict()}, path)``
with ``path = ./weights/<prefix>/<dnn>-n<nworkers>-bs<batch>-lr<%.4f>/<dnn>-rank<r>-epoch<e>.pth``
(reference ``dl_trainer.py:769-777``; the loader at ``:307-312`` and ``evaluate.py:21-33`` define
what readers expect).  The reference computes the file name but never calls its
``save_checkpoint``; here the file is actually written.  An optional ``'optimizer'`` entry may be
added; readers that only know the three reference keys ignore it.
"""
from __future__ import annotations

import os
from typing import Any, Dict, Optional

import torch


def checkpoint_dir(dnn: str, nworkers: int, batch_size: int, base_lr: float, prefix: Optional[str] = None,
                   root: str = './weights') -> str:
    leaf = '%s-n%d-bs%d-lr%.4f' % (dnn, nworkers, batch_size, base_lr)
    return os.path.join(root, prefix, leaf) if prefix else os.path.join(root, leaf)


def checkpoint_name(dnn: str, rank: int, epoch: int) -> str:
    return '%s-rank%d-epoch%d.pth' % (dnn, rank, epoch)


def parse_checkpoint_dir(model_path: str) -> Dict[str, Any]:
    """Recover ``dnn``, ``batch_size`` and ``lr`` from a directory name (``evaluate.py:21-24``)."""
    items = os.path.basename(os.path.normpath(model_path)).split('-')
    return {'dnn': items[0], 'nworkers': int(items[1][1:]), 'batch_size': int(items[2][2:]), 'lr': float(items[-1][2:])}


def save_checkpoint(path: str, state_dict: Dict[str, torch.Tensor], epoch: int, iteration: int,
                    optimizer_state: Optional[dict] = None) -> str:
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    payload = {'iter': int(iteration), 'epoch': int(epoch),
               'state': {k: v.detach().cpu().contiguous() for k, v in state_dict.items()}}
    if optimizer_state is not None:
        payload['optimizer'] = optimizer_state
    tmp = path + '.tmp'
    torch.save(payload, tmp)
    os.replace(tmp, path)          # readers never see a half-written file
    return path


def load_checkpoint(path: str, map_location='cpu') -> Dict[str, Any]:
    ckpt = torch.load(path, map_location=map_location, weights_only=False)
    for key in ('state', 'epoch', 'iter'):
        if key not in ckpt:
            raise KeyError('%s is not a checkpoint of this format: missing %r' % (path, key))
    return ckpt
