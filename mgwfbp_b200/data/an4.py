# -*- coding: utf-8 -*-
"""AN4 / LibriSpeech-style speech data: manifests, spectrograms, batching, greedy CTC decoding.

The reference's speech path imports a ``data_loader`` and a ``decoder`` module that are not in
its repository (``audio_data/__init__.py:1``, ``dl_trainer.py:493-494``); this module supplies the
pieces those imports were meant to provide: a manifest (``wav_path,transcript_path`` CSV rows,
the format of ``audio_data/an4_train_manifest.csv``) dataset producing log-magnitude STFT
spectrograms (20 ms Hamming window, 10 ms stride, 16 kHz -> 161 bins), a collate function that
returns ``(inputs[B,1,161,T], flat_targets, input_percentages, target_sizes)`` and a greedy
decoder with word / character error rates.
"""
from __future__ import annotations

import csv
import math
import wave
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch
from torch.utils.data import DataLoader, Dataset


def load_wav(path: str) -> Tuple[np.ndarray, int]:
    with wave.open(path, 'rb') as w:
        rate, n, width, ch = w.getframerate(), w.getnframes(), w.getsampwidth(), w.getnchannels()
        raw = w.readframes(n)
    dtype = {1: np.uint8, 2: np.int16, 4: np.int32}[width]
    data = np.frombuffer(raw, dtype=dtype).astype(np.float32)
    if ch > 1:
        data = data.reshape(-1, ch).mean(axis=1)
    return data / float(np.iinfo(dtype).max), rate


def spectrogram(signal: np.ndarray, sample_rate=16000, window_size=0.02, window_stride=0.01, normalize=True) -> torch.Tensor:
    n_fft = int(sample_rate * window_size)
    hop = int(sample_rate * window_stride)
    x = torch.from_numpy(np.ascontiguousarray(signal))
    spec = torch.stft(x, n_fft=n_fft, hop_length=hop, win_length=n_fft, window=torch.hamming_window(n_fft),
                      return_complex=True).abs()
    spec = torch.log1p(spec)
    if normalize:
        spec = (spec - spec.mean()) / (spec.std() + 1e-8)
    return spec


class SpectrogramDataset(Dataset):
    def __init__(self, audio_conf: dict, manifest_filepath: str, labels: str, normalize: bool = True):
        with open(manifest_filepath) as f:
            self.ids = [row for row in csv.reader(f) if len(row) >= 2]
        self.audio_conf, self.normalize = audio_conf, normalize
        self.labels_map = {c: i for i, c in enumerate(labels)}

    def __len__(self):
        return len(self.ids)

    def __getitem__(self, idx):
        wav, txt = self.ids[idx][0], self.ids[idx][1]
        signal, rate = load_wav(wav)
        spec = spectrogram(signal, self.audio_conf.get('sample_rate', rate), self.audio_conf.get('window_size', 0.02),
                           self.audio_conf.get('window_stride', 0.01), self.normalize)
        with open(txt) as f:
            transcript = f.read().replace('\n', '')
        return spec, [self.labels_map[c] for c in transcript if c in self.labels_map]


def collate_spectrograms(batch):
    batch = sorted(batch, key=lambda s: s[0].size(1), reverse=True)
    freq, longest = batch[0][0].size(0), batch[0][0].size(1)
    inputs = torch.zeros(len(batch), 1, freq, longest)
    pct = torch.zeros(len(batch))
    sizes = torch.zeros(len(batch), dtype=torch.int32)
    targets: List[int] = []
    for i, (spec, tgt) in enumerate(batch):
        t = spec.size(1)
        inputs[i, 0, :, :t] = spec
        pct[i] = t / float(longest)
        sizes[i] = len(tgt)
        targets.extend(tgt)
    return inputs, torch.tensor(targets, dtype=torch.int32), pct, sizes


class AudioDataLoader(DataLoader):
    def __init__(self, *args, **kwargs):
        kwargs.setdefault('collate_fn', collate_spectrograms)
        super().__init__(*args, **kwargs)


def _edit_distance(a: Sequence, b: Sequence) -> int:
    prev = list(range(len(b) + 1))
    for i, x in enumerate(a, 1):
        cur = [i]
        for j, y in enumerate(b, 1):
            cur.append(min(prev[j] + 1, cur[j - 1] + 1, prev[j - 1] + (x != y)))
        prev = cur
    return prev[-1]


class GreedyDecoder:
    """Best-path CTC decoding: arg-max per frame, collapse repeats, drop blanks."""

    def __init__(self, labels: str, blank_index: int = 0):
        self.labels, self.blank_index = labels, blank_index
        self.int_to_char = dict(enumerate(labels))

    def convert_to_strings(self, sequences, sizes=None):
        out = []
        for i, seq in enumerate(sequences):
            n = int(sizes[i]) if sizes is not None else len(seq)
            out.append([''.join(self.int_to_char[int(c)] for c in seq[:n])])
        return out

    def decode(self, probs: torch.Tensor, sizes=None):
        """``probs``: B x T x C.  Returns ``(strings, offsets)`` shaped like the reference expects."""
        best = probs.argmax(dim=2)
        strings, offsets = [], []
        for b in range(best.size(0)):
            n = int(sizes[b]) if sizes is not None else best.size(1)
            chars, offs, last = [], [], None
            for t in range(n):
                c = int(best[b, t])
                if c != self.blank_index and c != last:
                    chars.append(self.int_to_char[c])
                    offs.append(t)
                last = c
            strings.append([''.join(chars)])
            offsets.append([offs])
        return strings, offsets

    @staticmethod
    def wer(s1: str, s2: str) -> int:
        return _edit_distance(s1.split(), s2.split())

    @staticmethod
    def cer(s1: str, s2: str) -> int:
        return _edit_distance(s1.replace(' ', ''), s2.replace(' ', ''))


def wav_duration(path: str) -> float:
    """Length of a PCM wave file in seconds, from its header (the reference shells out to ``soxi -D``)."""
    with wave.open(path, 'rb') as w:
        return w.getnframes() / float(w.getframerate())


def order_and_prune_files(file_paths: Sequence[str], min_duration: Optional[float] = None,
                          max_duration: Optional[float] = None) -> List[str]:
    """Audio files sorted by duration, shortest first; with both bounds given, files outside
    ``[min_duration, max_duration]`` seconds are dropped (reference ``audio_data/utils.py:24-37``)."""
    timed = [(p.strip(), wav_duration(p.strip())) for p in file_paths]
    if min_duration and max_duration:
        timed = [(p, d) for p, d in timed if min_duration <= d <= max_duration]
    timed.sort(key=lambda pd: pd[1])
    return [p for p, _ in timed]


def create_manifest(data_path: str, tag: str, ordered: bool = True, out_dir: str = '.') -> str:
    """Write ``<tag>_manifest.csv`` listing ``wav_path,txt_path`` for every ``wav/*.wav`` under ``data_path``
    with its transcript in the sibling ``txt/`` folder (what the reference's ``audio_data/utils.py`` produces
    after its download step; downloading itself needs network access and is left to the user).
    ``ordered`` sorts by audio duration, shortest first."""
    import os
    wavs = []
    for root, _dirs, files in os.walk(data_path):
        for fn in files:
            if fn.lower().endswith('.wav'):
                wavs.append(os.path.join(root, fn))
    if ordered:
        def duration(p):
            with wave.open(p, 'rb') as w:
                return w.getnframes() / float(w.getframerate())
        wavs.sort(key=duration)
    else:
        wavs.sort()
    out = os.path.join(out_dir, '%s_manifest.csv' % tag)
    with open(out, 'w') as f:
        for wav in wavs:
            txt = wav.replace('/wav/', '/txt/').replace('.wav', '.txt')
            f.write('%s,%s\n' % (os.path.abspath(wav), os.path.abspath(txt)))
    return out
