# -*- coding: utf-8 -*-
"""DeepSpeech-2 style acoustic model (the reference's ``lstman4``).

Two masked 2-D convolutions over the spectrogram, ``nb_layers`` sequence-wise batch-normalised
unidirectional LSTMs, a look-ahead convolution and a batch-normalised linear classifier, with
the module / parameter names of reference ``models/lstm_models.py:148-322`` (``conv.seq_module.*``,
``rnns.<i>.rnn.*``, ``lookahead.0.weight``, ``fc.0.module.*``) and the ``serialize`` /
``load_model`` package format (``:240-287``).  ``create_net`` mirrors ``models/lstman4.py:8-33``.
"""
from __future__ import annotations

import json
import math
import os
from collections import OrderedDict

import torch
import torch.nn as nn
import torch.nn.functional as F

supported_rnns = {'lstm': nn.LSTM, 'rnn': nn.RNN, 'gru': nn.GRU}
supported_rnns_inv = {v: k for k, v in supported_rnns.items()}

DEFAULT_LABELS = "_'ABCDEFGHIJKLMNOPQRSTUVWXYZ "


class SequenceWise(nn.Module):
    """Apply a module to ``T x N x H`` input by folding time into the batch."""

    def __init__(self, module):
        super().__init__()
        self.module = module

    def forward(self, x):
        t, n = x.size(0), x.size(1)
        return self.module(x.reshape(t * n, -1)).view(t, n, -1)


class MaskConv(nn.Module):
    """Zero the time steps beyond each sequence's length after every layer (input B x C x D x T)."""

    def __init__(self, seq_module):
        super().__init__()
        self.seq_module = seq_module

    def forward(self, x, lengths):
        for module in self.seq_module:
            x = module(x)
            t = torch.arange(x.size(3), device=x.device).view(1, 1, 1, -1)
            keep = t < lengths.to(x.device).view(-1, 1, 1, 1)
            x = x * keep
        return x, lengths


class InferenceBatchSoftmax(nn.Module):
    def forward(self, x):
        return x if self.training else F.softmax(x, dim=-1)


class BatchRNN(nn.Module):
    def __init__(self, input_size, hidden_size, rnn_type=nn.LSTM, bidirectional=False, batch_norm=True):
        super().__init__()
        self.input_size, self.hidden_size, self.bidirectional = input_size, hidden_size, bidirectional
        self.batch_norm = SequenceWise(nn.BatchNorm1d(input_size)) if batch_norm else None
        self.rnn = rnn_type(input_size=input_size, hidden_size=hidden_size, bidirectional=bidirectional, bias=True)
        self.num_directions = 2 if bidirectional else 1

    def flatten_parameters(self):
        self.rnn.flatten_parameters()

    def forward(self, x, output_lengths):
        if self.batch_norm is not None:
            x = self.batch_norm(x)
        packed = nn.utils.rnn.pack_padded_sequence(x, output_lengths.cpu(), enforce_sorted=False)
        packed, _ = self.rnn(packed)
        x, _ = nn.utils.rnn.pad_packed_sequence(packed, total_length=x.size(0))
        if self.bidirectional:
            x = x.view(x.size(0), x.size(1), 2, -1).sum(2)
        return x


class Lookahead(nn.Module):
    """Per-feature convolution over the next ``context`` time steps (input T x N x H)."""

    def __init__(self, n_features, context):
        super().__init__()
        if context <= 0:
            raise ValueError('context must be positive')
        self.n_features, self.context = n_features, context
        self.weight = nn.Parameter(torch.empty(n_features, context + 1))
        self.register_parameter('bias', None)
        bound = 1.0 / math.sqrt(self.weight.size(1))
        nn.init.uniform_(self.weight, -bound, bound)

    def forward(self, x):
        t = x.size(0)
        padded = F.pad(x, (0, 0, 0, 0, 0, self.context))
        windows = padded.unfold(0, self.context + 1, 1)[:t]           # T x N x H x (context+1)
        return (windows * self.weight).sum(dim=3)


class DeepSpeech(nn.Module):
    def __init__(self, rnn_type=nn.LSTM, labels='abc', rnn_hidden_size=768, nb_layers=5, audio_conf=None,
                 bidirectional=True, context=20):
        super().__init__()
        self.name = 'lstman4'
        self._version = '0.0.1'
        self._hidden_size, self._hidden_layers, self._rnn_type = rnn_hidden_size, nb_layers, rnn_type
        self._audio_conf = audio_conf or {}
        self._labels, self._bidirectional = labels, bidirectional
        sample_rate = self._audio_conf.get('sample_rate', 16000)
        window_size = self._audio_conf.get('window_size', 0.02)
        num_classes = len(labels)
        self.conv = MaskConv(nn.Sequential(
            nn.Conv2d(1, 32, kernel_size=(41, 11), stride=(2, 2), padding=(20, 5)), nn.BatchNorm2d(32),
            nn.Hardtanh(0, 20, inplace=True),
            nn.Conv2d(32, 32, kernel_size=(21, 11), stride=(2, 1), padding=(10, 5)), nn.BatchNorm2d(32),
            nn.Hardtanh(0, 20, inplace=True)))
        freq = int(math.floor((sample_rate * window_size) / 2) + 1)
        freq = int(math.floor(freq + 2 * 20 - 41) / 2 + 1)
        freq = int(math.floor(freq + 2 * 10 - 21) / 2 + 1)
        rnn_input = freq * 32
        rnns = [('0', BatchRNN(rnn_input, rnn_hidden_size, rnn_type, bidirectional, batch_norm=False))]
        for i in range(nb_layers - 1):
            rnns.append(('%d' % (i + 1), BatchRNN(rnn_hidden_size, rnn_hidden_size, rnn_type, bidirectional)))
        self.rnns = nn.Sequential(OrderedDict(rnns))
        self.lookahead = None if bidirectional else nn.Sequential(Lookahead(rnn_hidden_size, context=context),
                                                                  nn.Hardtanh(0, 20, inplace=True))
        self.fc = nn.Sequential(SequenceWise(nn.Sequential(nn.BatchNorm1d(rnn_hidden_size),
                                                           nn.Linear(rnn_hidden_size, num_classes, bias=False))))
        self.inference_softmax = InferenceBatchSoftmax()

    def get_seq_lens(self, input_length):
        seq = input_length
        for m in self.conv.modules():
            if type(m) is nn.Conv2d:
                seq = torch.div(seq + 2 * m.padding[1] - m.dilation[1] * (m.kernel_size[1] - 1) - 1, m.stride[1],
                                rounding_mode='floor') + 1
        return seq.int()

    def forward(self, x, lengths):
        out_len = self.get_seq_lens(lengths.cpu().int())
        x, _ = self.conv(x, out_len)
        b, c, d, t = x.size()
        x = x.view(b, c * d, t).permute(2, 0, 1).contiguous()        # T x N x H
        for rnn in self.rnns:
            x = rnn(x, out_len)
        if not self._bidirectional:
            x = self.lookahead(x)
        x = self.fc(x).transpose(0, 1)
        return self.inference_softmax(x), out_len

    # package format ---------------------------------------------------------------
    @staticmethod
    def is_parallel(model):
        return isinstance(model, (nn.parallel.DataParallel, nn.parallel.DistributedDataParallel))

    @staticmethod
    def serialize(model, optimizer=None, epoch=None, iteration=None, loss_results=None, cer_results=None,
                  wer_results=None, avg_loss=None, meta=None):
        model = model.module if DeepSpeech.is_parallel(model) else model
        package = {'version': model._version, 'hidden_size': model._hidden_size, 'hidden_layers': model._hidden_layers,
                   'rnn_type': supported_rnns_inv.get(model._rnn_type, model._rnn_type.__name__.lower()),
                   'audio_conf': model._audio_conf, 'labels': model._labels, 'state_dict': model.state_dict(),
                   'bidirectional': model._bidirectional}
        if optimizer is not None:
            package['optim_dict'] = optimizer.state_dict()
        if avg_loss is not None:
            package['avg_loss'] = avg_loss
        if epoch is not None:
            package['epoch'] = epoch + 1
        if iteration is not None:
            package['iteration'] = iteration
        if loss_results is not None:
            package.update(loss_results=loss_results, cer_results=cer_results, wer_results=wer_results)
        if meta is not None:
            package['meta'] = meta
        return package

    @classmethod
    def load_model_package(cls, package):
        model = cls(rnn_hidden_size=package['hidden_size'], nb_layers=package['hidden_layers'],
                    labels=package['labels'], audio_conf=package['audio_conf'],
                    rnn_type=supported_rnns[package['rnn_type']], bidirectional=package.get('bidirectional', True))
        model.load_state_dict(package['state_dict'])
        return model

    @classmethod
    def load_model(cls, path):
        model = cls.load_model_package(torch.load(path, map_location='cpu', weights_only=False))
        for r in model.rnns:
            r.flatten_parameters()
        return model

    @staticmethod
    def get_labels(model):
        return (model.module if DeepSpeech.is_parallel(model) else model)._labels

    @staticmethod
    def get_audio_conf(model):
        return (model.module if DeepSpeech.is_parallel(model) else model)._audio_conf

    @staticmethod
    def get_param_size(model):
        return sum(p.numel() for p in model.parameters())

    @staticmethod
    def get_meta(model):
        m = model.module if DeepSpeech.is_parallel(model) else model
        return {'version': m._version, 'hidden_size': m._hidden_size, 'hidden_layers': m._hidden_layers,
                'rnn_type': supported_rnns_inv[m._rnn_type]}


def create_net(nb_labers=5, labels=None, rnn_type='lstm', bidirectional=False, datapath=None, hidden_size=800,
               hidden_layers=5, sample_rate=16000, window_size=0.02, window_stride=0.01, window='hamming',
               noise_dir=None, noise_prob=0.4, noise_min=0.0, noise_max=0.5):
    """Build the AN4 acoustic model; labels come from ``<datapath>/labels.json`` when present,
    otherwise the 29-symbol English alphabet the reference ships (``labels.json``)."""
    if labels is None:
        path = os.path.join(datapath, 'labels.json') if datapath else None
        if path and os.path.isfile(path):
            with open(path) as f:
                labels = str(''.join(json.load(f)))
        else:
            labels = DEFAULT_LABELS
    audio_conf = dict(sample_rate=sample_rate, window_size=window_size, window_stride=window_stride, window=window,
                      noise_dir=noise_dir, noise_prob=noise_prob, noise_levels=(noise_min, noise_max))
    net = DeepSpeech(rnn_hidden_size=hidden_size, nb_layers=hidden_layers, labels=labels,
                     rnn_type=supported_rnns[rnn_type], audio_conf=audio_conf, bidirectional=bidirectional)
    return net, {'audio_conf': audio_conf, 'labels': labels}
