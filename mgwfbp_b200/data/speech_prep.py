# -*- coding: utf-8 -*-
"""Offline preparation of the AN4 and LibriSpeech corpora for the DeepSpeech (``lstman4``) model.

The reference prepares both corpora with scripts that download the archives, convert the audio with
``sox`` and write duration-sorted manifests (``audio_data/an4.py:19-87``, ``audio_data/librispeech.py:37-113``,
``audio_data/utils.py:11-37``).  Training boxes have no network, so the preparers here start from an archive
or directory that is **already on disk**, and convert with the standard library where that is possible:

* AN4 ships headerless big-endian 16-bit PCM at 16 kHz: it is byte-swapped and wrapped in a RIFF header
  directly (no ``sox``).
* LibriSpeech ships FLAC.  A decoder is looked for in this order: the ``soundfile`` module, ``torchaudio``, a
  ``sox`` or ``flac`` binary on ``PATH``; a caller may also pass its own ``decode(path) -> (int16 samples, rate)``.
  Without any of them the preparer stops with a message that says so.

Resulting layout (identical to the reference's, so manifests are interchangeable)::

    <target>/<split>/[an4/]wav/<utterance>.wav
    <target>/<split>/[an4/]txt/<utterance>.txt        upper-cased transcript, markup removed
    <tag>_manifest.csv                                 "wav_path,txt_path" lines, shortest utterance first;
                                                       training splits pruned to [min_duration, max_duration]

    python -m mgwfbp_b200.data.speech_prep an4 --source an4_raw.bigendian.tar.gz --target-dir an4_dataset
    python -m mgwfbp_b200.data.speech_prep librispeech --source /data/LibriSpeech --target-dir LibriSpeech_dataset
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import tarfile
import tempfile
import wave
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np

from .an4 import order_and_prune_files

Decoder = Callable[[str], Tuple[np.ndarray, int]]

AN4_SAMPLE_RATE = 16000
# split name of the reference -> sub-directories of an extracted LibriSpeech tree / archive stems (librispeech.py:24-34)
LIBRISPEECH_SPLITS: Dict[str, Tuple[str, ...]] = {
    'train': ('train-clean-100', 'train-clean-360', 'train-other-500'),
    'val': ('dev-clean', 'dev-other'),
    'test_clean': ('test-clean',),
    'test_other': ('test-other',),
}


# ---------------------------------------------------------------------------------------------------
# shared pieces
# ---------------------------------------------------------------------------------------------------
def write_wav(path: str, samples: np.ndarray, rate: int) -> None:
    """16-bit mono PCM wave file."""
    data = np.asarray(samples)
    if data.dtype != np.int16:
        data = np.clip(np.round(data.astype(np.float64) * (32767.0 if np.issubdtype(data.dtype, np.floating) else 1.0)),
                       -32768, 32767).astype(np.int16)
    if data.ndim == 2:                                   # mix down to one channel
        data = data.astype(np.int32).mean(axis=1 if data.shape[1] <= 8 else 0).astype(np.int16)
    with wave.open(path, 'wb') as w:
        w.setnchannels(1)
        w.setsampwidth(2)
        w.setframerate(int(rate))
        w.writeframes(data.astype('<i2').tobytes())


def write_manifest(split_dir: str, out_path: str, min_duration: Optional[float] = None,
                   max_duration: Optional[float] = None) -> int:
    """``wav,txt`` lines for every wave file below ``split_dir``, shortest first, optionally pruned by duration
    (reference ``audio_data/utils.py:11-37``).  Returns the number of utterances kept."""
    wavs = [os.path.join(root, f) for root, _d, files in os.walk(split_dir) for f in files if f.lower().endswith('.wav')]
    kept = order_and_prune_files(sorted(wavs), min_duration, max_duration)
    with open(out_path, 'w') as f:
        for wav in kept:
            txt = wav.replace(os.sep + 'wav' + os.sep, os.sep + 'txt' + os.sep)[:-4] + '.txt'
            f.write('%s,%s\n' % (os.path.abspath(wav), os.path.abspath(txt)))
    return len(kept)


def _materialise(source: str, workdir: str) -> str:
    """``source`` as a directory: archives are unpacked below ``workdir``."""
    if os.path.isdir(source):
        return source
    if not os.path.isfile(source):
        raise FileNotFoundError('%s is neither a directory nor an archive (this tool does not download)' % source)
    with tarfile.open(source) as tar:
        try:
            tar.extractall(workdir, filter='data')
        except TypeError:                               # Python without extraction filters
            tar.extractall(workdir)
    return workdir


# ---------------------------------------------------------------------------------------------------
# AN4
# ---------------------------------------------------------------------------------------------------
def an4_transcript(line: str) -> str:
    """``<s> HELLO WORLD </s> (an4-utt-id)`` -> ``HELLO WORLD`` (what reference ``an4.py:63-65`` extracts)."""
    text = line.split('(')[0].strip()
    if text.startswith('<s>'):
        text = text[3:]
    return text.split('<')[0].strip().upper()


def raw_to_wav(raw_path: str, wav_path: str, rate: int = AN4_SAMPLE_RATE) -> None:
    """Headerless big-endian signed 16-bit mono PCM -> wave file (the reference calls
    ``sox -t raw -r 16000 -b 16 -e signed-integer -B -c 1``, ``an4.py:36-44``)."""
    samples = np.fromfile(raw_path, dtype='>i2').astype(np.int16)
    write_wav(wav_path, samples, rate)


def prepare_an4(source: str, target_dir: str, min_duration: float = 1, max_duration: float = 15,
                manifest_dir: str = '.') -> Dict[str, int]:
    """Lay out AN4 for training from ``source`` (``an4_raw.bigendian.tar.gz`` or the directory it unpacks to, the one
    that holds ``etc/`` and ``wav/``).  Returns ``{'train': n, 'val': n}``, the utterances listed in
    ``an4_train_manifest.csv`` (pruned to the duration bounds) and ``an4_val_manifest.csv`` (all of the test part)."""
    work = tempfile.mkdtemp(prefix='an4prep')
    try:
        root = _materialise(source, work)
        if not os.path.isdir(os.path.join(root, 'etc')) and os.path.isdir(os.path.join(root, 'an4', 'etc')):
            root = os.path.join(root, 'an4')
        if not os.path.isdir(os.path.join(root, 'etc')):
            raise FileNotFoundError('no etc/ directory with AN4 file lists below %s' % source)
        counts = {}
        for tag, manifest, bounds in (('train', 'an4_train_manifest.csv', (min_duration, max_duration)),
                                      ('test', 'an4_val_manifest.csv', (None, None))):
            split = os.path.join(target_dir, tag, 'an4')
            wav_out, txt_out = os.path.join(split, 'wav'), os.path.join(split, 'txt')
            os.makedirs(wav_out, exist_ok=True)
            os.makedirs(txt_out, exist_ok=True)
            with open(os.path.join(root, 'etc', 'an4_%s.fileids' % tag)) as f:
                ids = [l.strip() for l in f if l.strip()]
            with open(os.path.join(root, 'etc', 'an4_%s.transcription' % tag)) as f:
                texts = [l for l in f if l.strip()]
            if len(ids) != len(texts):
                raise ValueError('an4_%s: %d file ids but %d transcriptions' % (tag, len(ids), len(texts)))
            for rel, line in zip(ids, texts):
                base = os.path.basename(rel)
                src = os.path.join(root, 'wav', rel)
                dst = os.path.join(wav_out, base + '.wav')
                if os.path.isfile(src + '.raw'):
                    raw_to_wav(src + '.raw', dst)
                elif os.path.isfile(src + '.wav'):
                    shutil.copyfile(src + '.wav', dst)
                else:
                    raise FileNotFoundError('%s(.raw|.wav) listed in an4_%s.fileids is missing' % (src, tag))
                with open(os.path.join(txt_out, base + '.txt'), 'w') as t:
                    t.write(an4_transcript(line))
            counts['train' if tag == 'train' else 'val'] = write_manifest(
                os.path.join(target_dir, tag), os.path.join(manifest_dir, manifest), *bounds)
        return counts
    finally:
        shutil.rmtree(work, ignore_errors=True)


# ---------------------------------------------------------------------------------------------------
# LibriSpeech
# ---------------------------------------------------------------------------------------------------
def find_flac_decoder(sample_rate: int) -> Decoder:
    """The first FLAC decoder this machine offers (see the module docstring for the order)."""
    try:
        import soundfile

        def with_soundfile(path):
            data, rate = soundfile.read(path, dtype='int16')
            return data, rate
        return with_soundfile
    except ImportError:
        pass
    try:
        import torchaudio

        def with_torchaudio(path):
            data, rate = torchaudio.load(path)
            return (data.mean(0).clamp(-1, 1) * 32767.0).short().numpy(), rate
        return with_torchaudio
    except ImportError:
        pass
    for exe, make_cmd in (('sox', lambda src, dst: ['sox', src, '-r', str(sample_rate), '-b', '16', '-c', '1', dst]),
                          ('flac', lambda src, dst: ['flac', '-d', '-f', '-s', '-o', dst, src])):
        if shutil.which(exe):
            def with_binary(path, _make=make_cmd):
                fd, tmp = tempfile.mkstemp(suffix='.wav')
                os.close(fd)
                try:
                    subprocess.check_call(_make(path, tmp))
                    with wave.open(tmp, 'rb') as w:
                        raw = w.readframes(w.getnframes())
                        data = np.frombuffer(raw, dtype='<i2')
                        if w.getnchannels() > 1:
                            data = data.reshape(-1, w.getnchannels())
                        return data, w.getframerate()
                finally:
                    os.unlink(tmp)
            return with_binary
    raise RuntimeError('no FLAC decoder found: install the soundfile or torchaudio module, or put sox / flac on PATH, '
                       'or pass decode=... to prepare_librispeech')


def _resample(samples: np.ndarray, rate: int, want: int) -> np.ndarray:
    if rate == want:
        return samples
    n_out = int(round(len(samples) * float(want) / rate))
    x_old = np.arange(len(samples), dtype=np.float64)
    x_new = np.linspace(0.0, len(samples) - 1.0, n_out)
    return np.interp(x_new, x_old, samples.astype(np.float64)).round().astype(np.int16)


def read_transcripts(chapter_dir: str) -> Dict[str, str]:
    """``{utterance id: TEXT}`` from the ``*.trans.txt`` files of one chapter directory (``librispeech.py:51-59``)."""
    out: Dict[str, str] = {}
    for name in os.listdir(chapter_dir):
        if name.endswith('.trans.txt'):
            with open(os.path.join(chapter_dir, name)) as f:
                for line in f:
                    parts = line.split()
                    if parts:
                        out[parts[0]] = ' '.join(parts[1:]).strip().upper()
    return out


def prepare_librispeech(source: str, target_dir: str, parts: Optional[Sequence[str]] = None, sample_rate: int = 16000,
                        min_duration: float = 1, max_duration: float = 15, manifest_dir: str = '.',
                        decode: Optional[Decoder] = None) -> Dict[str, int]:
    """Lay out LibriSpeech for training.  ``source`` is a directory that holds either the extracted corpus
    (``.../LibriSpeech/train-clean-100/<speaker>/<chapter>/*.flac``) or the downloaded ``*.tar.gz`` archives;
    ``parts`` restricts the conversion to some of them (default: every part that is present).  One manifest per
    split (``libri_<split>_manifest.csv``); only the training split is pruned by duration.  Returns the number of
    utterances per split."""
    decode = decode or find_flac_decoder(sample_rate)
    counts: Dict[str, int] = {}
    work = tempfile.mkdtemp(prefix='libriprep')
    try:
        for split, members in LIBRISPEECH_SPLITS.items():
            split_dir = os.path.join(target_dir, split)
            wav_out, txt_out = os.path.join(split_dir, 'wav'), os.path.join(split_dir, 'txt')
            converted = 0
            for part in members:
                if parts is not None and part not in parts and part + '.tar.gz' not in parts:
                    continue
                part_dir = _locate_part(source, part, work)
                if part_dir is None:
                    continue
                os.makedirs(wav_out, exist_ok=True)
                os.makedirs(txt_out, exist_ok=True)
                for root, _dirs, files in os.walk(part_dir):
                    audio = sorted(f for f in files if f.endswith('.flac') or f.endswith('.wav'))
                    if not audio:
                        continue
                    texts = read_transcripts(root)
                    for name in audio:
                        utt = os.path.splitext(name)[0]
                        if utt not in texts:
                            raise KeyError('%s has no line in the transcript file of %s' % (utt, root))
                        samples, rate = decode(os.path.join(root, name))
                        write_wav(os.path.join(wav_out, utt + '.wav'), _resample(np.asarray(samples), rate, sample_rate), sample_rate)
                        with open(os.path.join(txt_out, utt + '.txt'), 'w') as t:
                            t.write(texts[utt])
                        converted += 1
            if converted:
                bounds = (min_duration, max_duration) if split == 'train' else (None, None)
                counts[split] = write_manifest(split_dir, os.path.join(manifest_dir, 'libri_%s_manifest.csv' % split), *bounds)
        return counts
    finally:
        shutil.rmtree(work, ignore_errors=True)


def _locate_part(source: str, part: str, work: str) -> Optional[str]:
    for cand in (os.path.join(source, 'LibriSpeech', part), os.path.join(source, part)):
        if os.path.isdir(cand):
            return cand
    archive = os.path.join(source, part + '.tar.gz')
    if os.path.isfile(archive):
        dest = os.path.join(work, part)
        os.makedirs(dest, exist_ok=True)
        _materialise(archive, dest)
        for cand in (os.path.join(dest, 'LibriSpeech', part), os.path.join(dest, part)):
            if os.path.isdir(cand):
                return cand
    return None


def main(argv: Optional[Iterable[str]] = None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest='corpus', required=True)
    for name, default_target in (('an4', 'an4_dataset'), ('librispeech', 'LibriSpeech_dataset')):
        p = sub.add_parser(name)
        p.add_argument('--source', required=True, help='archive or directory that is already on disk')
        p.add_argument('--target-dir', default=default_target)
        p.add_argument('--manifest-dir', default='.')
        p.add_argument('--min-duration', type=float, default=1, help='prune training utterances shorter than this (seconds)')
        p.add_argument('--max-duration', type=float, default=15, help='prune training utterances longer than this (seconds)')
        if name == 'librispeech':
            p.add_argument('--sample-rate', type=int, default=16000)
            p.add_argument('--files-to-use', default=None, help='comma-separated parts, e.g. train-clean-100,dev-clean')
    args = ap.parse_args(list(argv) if argv is not None else None)
    if args.corpus == 'an4':
        print(prepare_an4(args.source, args.target_dir, args.min_duration, args.max_duration, args.manifest_dir))
    else:
        parts = [p.strip() for p in args.files_to_use.split(',')] if args.files_to_use else None
        print(prepare_librispeech(args.source, args.target_dir, parts, args.sample_rate, args.min_duration, args.max_duration,
                                  args.manifest_dir))


if __name__ == '__main__':
    main()
