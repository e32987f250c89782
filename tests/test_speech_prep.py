"""Offline AN4 / LibriSpeech preparation on tiny synthetic corpora (no network, no sox), and the clock-sample parser."""
import io
import os
import tarfile
import wave

import numpy as np


def _tone(seconds, rate=16000, f=440.0):
    t = np.arange(int(seconds * rate)) / rate
    return (np.sin(2 * np.pi * f * t) * 12000).astype(np.int16)


def _make_an4_tree(root):
    os.makedirs(os.path.join(root, 'an4', 'etc'))
    utts = {'train': [('an4_clstk/fash/an251-fash-b', 'YES', 2.0), ('an4_clstk/fash/an253-fash-b', 'go home', 0.4),
                      ('an4_clstk/mabc/cen1-mabc-b', 'E R A S E', 1.2), ('an4_clstk/mabc/cen2-mabc-b', 'long one', 20.0)],
            'test': [('an4test_clstk/fcaw/an406-fcaw-b', 'RUBOUT G M E F THREE NINE', 0.5)]}
    for tag, items in utts.items():
        with open(os.path.join(root, 'an4', 'etc', 'an4_%s.fileids' % tag), 'w') as f, \
                open(os.path.join(root, 'an4', 'etc', 'an4_%s.transcription' % tag), 'w') as t:
            for rel, text, secs in items:
                f.write(rel + '\n')
                t.write('<s> %s </s> (%s)\n' % (text, os.path.basename(rel)))
                path = os.path.join(root, 'an4', 'wav', rel + '.raw')
                os.makedirs(os.path.dirname(path), exist_ok=True)
                _tone(secs).astype('>i2').tofile(path)              # headerless big-endian PCM, as the corpus ships it
    return utts


def test_an4_from_archive(tmp_path):
    from mgwfbp_b200.data.speech_prep import an4_transcript, prepare_an4
    src = tmp_path / 'src'
    _make_an4_tree(str(src))
    archive = tmp_path / 'an4_raw.bigendian.tar.gz'
    with tarfile.open(archive, 'w:gz') as tar:
        tar.add(str(src / 'an4'), arcname='an4')
    target, mdir = tmp_path / 'an4_dataset', tmp_path / 'manifests'
    mdir.mkdir()
    counts = prepare_an4(str(archive), str(target), manifest_dir=str(mdir))
    assert counts == {'train': 2, 'val': 1}                        # 0.4 s and 20 s training utterances pruned, test part whole
    lines = (mdir / 'an4_train_manifest.csv').read_text().strip().split('\n')
    wavs = [l.split(',')[0] for l in lines]
    assert [os.path.basename(w) for w in wavs] == ['cen1-mabc-b.wav', 'an251-fash-b.wav']     # shortest first
    with wave.open(wavs[1], 'rb') as w:
        assert (w.getframerate(), w.getnchannels(), w.getsampwidth(), w.getnframes()) == (16000, 1, 2, 32000)
        got = np.frombuffer(w.readframes(32000), dtype='<i2')
    np.testing.assert_array_equal(got, _tone(2.0))                 # byte order converted, samples untouched
    txt = lines[1].split(',')[1]
    assert open(txt).read() == 'YES' and '/txt/' in txt
    assert open(lines[0].split(',')[1]).read() == 'E R A S E'
    assert an4_transcript('<s> hello  world </s> (utt-1)') == 'HELLO  WORLD'
    val = (mdir / 'an4_val_manifest.csv').read_text().strip().split('\n')
    assert len(val) == 1 and val[0].split(',')[0].endswith('/test/an4/wav/an406-fcaw-b.wav')


def test_librispeech_layout_with_injected_decoder(tmp_path):
    from mgwfbp_b200.data.speech_prep import prepare_librispeech
    src = tmp_path / 'corpus' / 'LibriSpeech'
    samples = {}
    for part, spk, chap, n in (('train-clean-100', '19', '198', 3), ('dev-clean', '84', '121123', 2)):
        d = src / part / spk / chap
        d.mkdir(parents=True)
        with open(d / ('%s-%s.trans.txt' % (spk, chap)), 'w') as t:
            for i in range(n):
                utt = '%s-%s-%04d' % (spk, chap, i)
                t.write('%s some words number %d\n' % (utt, i))
                (d / (utt + '.flac')).write_bytes(b'fLaC-not-really')
                samples[utt] = _tone(1.5 + i, rate=8000)           # the fake decoder hands these out at 8 kHz

    def decode(path):
        return samples[os.path.splitext(os.path.basename(path))[0]], 8000
    mdir = tmp_path / 'm'
    mdir.mkdir()
    counts = prepare_librispeech(str(tmp_path / 'corpus'), str(tmp_path / 'out'), manifest_dir=str(mdir), decode=decode,
                                 min_duration=2, max_duration=15)
    assert counts == {'train': 2, 'val': 2}                        # the 1.5 s training utterance is pruned, validation is not
    first = (mdir / 'libri_train_manifest.csv').read_text().strip().split('\n')[0].split(',')
    with wave.open(first[0], 'rb') as w:
        assert w.getframerate() == 16000 and abs(w.getnframes() - 2.5 * 16000) <= 1            # resampled to the target rate
    assert open(first[1]).read() == 'SOME WORDS NUMBER 1'
    assert not (mdir / 'libri_test_clean_manifest.csv').exists()   # parts that are absent produce nothing


def test_clock_sample_parser():
    from mgwfbp_b200.utils.clocks import parse_samples
    lines = ['0, 1965, 1965, 180.2, 0x0000000000000000, Not Active, Not Active, Not Active, Not Active',
             '0, 1410, 1965, 1003.9, 0x0000000000000004, Not Active, Not Active, Not Active, Active',
             '0, 1395, 1965, 998.0, 0x0000000000000004, Not Active, Not Active, Not Active, Active', 'garbage']
    s = parse_samples(lines)
    assert s['samples'] == 3 and s['sm_max_mhz'] == 1965.0 and s['reasons'] == ['sw_power_cap']
    assert s['sm_mhz'] == 1402.5                                    # median of the samples taken under load
