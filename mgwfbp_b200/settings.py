# -*- coding: utf-8 -*-
"""Process-wide switches and the shared logger.

Mirrors the switch set of the reference's ``settings.py:7-53`` (``DEBUG``, ``WARMUP``,
``CONNECTION``, ``FP16``, ``ADAPTIVE_MERGE``, ``ORIGINAL_HOROVOD``, ``MAX_EPOCHS``, ``PREFIX``,
``logger``, ``formatter``, ``hostname``) so scripts written against the reference keep working,
and adds the switches that only exist here (``FAKE_DATA`` made real, fused-update control,
communication algorithm selection).  Every switch can be overridden from the environment as
``MGWFBP_<NAME>`` so launch scripts need not edit this file.
"""
from __future__ import annotations

import logging
import os
import socket


def _env_flag(name: str, default: bool) -> bool:
    raw = os.environ.get('MGWFBP_' + name)
    if raw is None:
        return default
    return raw.strip().lower() not in ('0', 'false', 'no', 'off', '')


def _env_str(name: str, default: str) -> str:
    return os.environ.get('MGWFBP_' + name, default)


DEBUG = _env_flag('DEBUG', False)

# Kept for name compatibility with the reference (unused there as well).
GPU_CONSTRUCTION = True
DELAY_COMM = 1
EXCHANGE_MODE = 'MODEL'
TENSORBOARD = False

# Linear LR warm-up over the first five epochs (reference dl_trainer.py:612-621).
WARMUP = _env_flag('WARMUP', True)

# Which alpha-beta table the scheduler falls back to when nothing was measured.
# '10GbE' and '56GbIB' are the reference's tables; 'NVLink5' is the table for the
# peer-to-peer kernels of this package on an NVSwitch box.
CONNECTION = _env_str('CONNECTION', 'NVLink5')

# Mixed precision in the sense of the reference's ``FP16`` switch (apex amp O2 with a static loss scale of 128,
# reference dl_trainer.py:278-281,821): fp32 master weights and fp32 gradients, half-precision forward / backward
# math (``torch.autocast``), the loss multiplied by ``LOSS_SCALE`` before backward and the gradients divided by it
# inside the update kernels.
FP16 = _env_flag('FP16', False)
LOSS_SCALE = float(_env_str('LOSS_SCALE', '128.0'))
ADAPTIVE_MERGE = _env_flag('ADAPTIVE_MERGE', True)
ORIGINAL_HOROVOD = _env_flag('ORIGINAL_HOROVOD', False)

# The reference declares FAKE_DATA but never reads it; here it selects synthetic datasets.
FAKE_DATA = _env_flag('FAKE_DATA', False)

# Where the momentum-SGD update happens on the fused NVLink data plane (plain SGD without gradient clipping only):
#   'fused'     inside the all-reduce kernel of each merged group (weights change during backward, ``step()`` only waits);
#   'deferred'  the group kernels only average (the result stays in their staging area, they never touch parameters or
#               momenta, so they are short and cheap to run beside backward) and ONE multi-tensor SGD kernel reads the
#               staged averages after backward -- the same kernel a single GPU runs, so the multi-GPU step pays for
#               communication only;
#   'separate'  the group kernels write the averaged gradient back to ``p.grad`` and a separate SGD kernel follows.
# The entry points try 'fused' and 'deferred' schedules and keep the faster one (``engine.tune_schedule``).
UPDATE_MODE = _env_str('UPDATE', 'fused').lower()
FUSED_UPDATE = UPDATE_MODE == 'fused'

# Swap BatchNorm+ReLU pairs and LSTMs for this package's fused CUDA modules when a model is built on a GPU.
FUSE_MODULES = _env_flag('FUSE', True)
# The PTB model's recurrent part: mgwfbp_b200.ops.lstm.FusedLSTM (this package's cell kernels; the layers run as a
# wavefront over chunks of time steps on two streams) unless this is switched off, in which case torch.nn.LSTM (the
# library's LSTM) is used.  Measured on B200 (batch 20, 35 steps, 1500 hidden, whole training step): 2.60 ms with the
# kernels here, 2.56 ms with the library's -- the named kernels are on the hot path at a cost of 1.6 %.
FUSE_LSTM = _env_flag('FUSE_LSTM', True)
# How many algorithms cuDNN's benchmark mode may time per convolution shape (-1: leave PyTorch's default of 10, 0: all).
CUDNN_BENCHMARK_LIMIT = int(_env_str('CUDNN_BENCHMARK_LIMIT', '-1'))
# Keep convolutional models and their inputs in channels-last (NHWC) memory format on the GPU.
CHANNELS_LAST = _env_flag('CHANNELS_LAST', True)

# Large nn.Linear layers fed by small batches: exchange activations + output gradients between ranks and run the
# tensor-core weight-gradient GEMM with the SGD epilogue instead of all-reducing the weight gradient.
GATHERED_WGRAD = _env_flag('GATHERED_WGRAD', True)
# On ONE GPU the same layers run that GEMM in their backward with the SGD update as its epilogue (no dW tensor, no
# separate update pass over these weights).  Off when gradients are clipped or accumulated.
FUSED_WGRAD_1GPU = _env_flag('FUSED_WGRAD_1GPU', True)

# Large 2-D weights whose gradient is one GEMM over the whole batch / sequence (the PTB model's LSTM weights and softmax
# layer) and for which gathering activations does not pay: form the gradient with the tensor-core GEMM whose epilogue
# stores every tile straight into the staging slot of the rank that owns it; owners add the slots up and broadcast the
# sums into every rank's (symmetric) gradient tensor.  The gradient never exists as a local tensor that has to be packed.
# Off by default: measured on 2 B200s with the PTB model it costs 3.26 ms/step against 3.08 through the merged all-reduce
# (the tensor-core GEMM is behind the library's on these K = 700 shapes, 347 against ~270 us for the five products, and the
# owners' pass plus the separate norm pass, 0.33 + 0.1 ms, cost about what one 204 MB two-shot all-reduce does).
SCATTER_WGRAD = _env_flag('SCATTER_WGRAD', False)

# After the fused all-reduce + update kernels ran, also store the averaged gradient back into ``p.grad``.  Off by
# default: with the update fused nobody reads the gradient again and the store is one more pass over the model
# (``optimizer.synchronize()`` + clipping paths do not fuse the update and always get the averaged gradient).
WRITE_BACK_GRADS = _env_flag('WRITE_BACK_GRADS', False)

# Every SHADOW_EVERY-th iteration the fused data plane is checked against a slow path: local gradients, parameters
# and momenta are snapshotted before each group is launched, averaged over the CPU control plane and the update is
# redone in plain PyTorch (utils/consistency.py, ShadowChecker).  0 = off.  Training steps are not graph-captured
# while this is on.
SHADOW_EVERY = int(_env_str('SHADOW', '0') or 0)

# Seconds of backward lost per second of all-reduce kernel running beside it (0 = overlapped communication is free,
# the assumption of the MG-WFBP recurrences; 1 = it costs as much as exposed communication and the schedule collapses
# to one message).  Only the fused NVLink data plane has such a cost: its kernels share SMs and memory bandwidth with
# backward.  The entry points measure it on the running box for the planned CTA count (``engine.fit_interference``)
# and then confirm the schedule by timing it (``engine.tune_schedule``); this value is what a bare
# ``DistributedOptimizer(...)`` uses when nothing was measured, or what ``MGWFBP_INTERFERENCE`` pins.
_interference_env = _env_str('INTERFERENCE', '')
INTERFERENCE_PINNED = _interference_env != ''
INTERFERENCE = float(_interference_env) if INTERFERENCE_PINNED else 0.25
# A merged group that becomes ready this close to the end of backward (milliseconds of profiled backward time left) can
# be treated like the schedule's last message: its kernel gets the CTA count of a message that has the GPU to itself
# instead of the few CTAs of an overlapped one, because most of it runs after backward anyway
# (``DistributedOptimizer(late_full=True)``; off unless asked for).
LATE_GROUP_MS = float(_env_str('LATE_GROUP_MS', '0.4'))
# Let the schedule trial also run its candidates with their late groups given the whole GPU (engine.build_distributed_optimizer).
# Off by default: the option is tested on CPU only (which groups count as late), no GPU time was left to measure it.
TRY_LATE_GROUPS = _env_flag('TRY_LATE_GROUPS', False)

# The stock comparison arm (reference dist_trainer.py:12-15 imports horovod.torch itself when this is set): gradients
# go through torch.distributed (NCCL on GPUs) in Horovod-style fusion buckets of 64 MB, the update is torch's own
# SGD.step, none of this package's communication or update kernels run.
HOROVOD_FUSION_ELEMENTS = 16 * 1024 * 1024

# 'auto' | 'oneshot' | 'twoshot' | 'nvls'
COMM_ALGO = _env_str('COMM_ALGO', 'auto')

MAX_EPOCHS = 200


def _build_prefix() -> str:
    prefix = ''
    if WARMUP:
        prefix += 'gwarmup'
    prefix += '-dc' + str(DELAY_COMM)
    prefix += '-' + EXCHANGE_MODE.lower()
    exp = '-tpds' + CONNECTION
    if FP16:
        exp += '-fp16'
    prefix += exp
    if ADAPTIVE_MERGE:
        prefix += '-ada'
    if ORIGINAL_HOROVOD:
        prefix += '-hvd'
    return prefix


PREFIX = _build_prefix()

hostname = socket.gethostname()
logger = logging.getLogger(hostname)
logger.setLevel(logging.DEBUG if DEBUG else logging.INFO)
formatter = logging.Formatter('%(asctime)s [%(filename)s:%(lineno)d] %(levelname)s %(message)s')
if not logger.handlers:
    strhdlr = logging.StreamHandler()
    strhdlr.setFormatter(formatter)
    logger.addHandler(strhdlr)
logger.propagate = False
