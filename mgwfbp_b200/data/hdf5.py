# -*- coding: utf-8 -*-
"""ImageNet stored in one HDF5 file.

Layout of reference ``datasets.py:8-36`` / ``scripts/create_hdf5.py:46-124``: datasets
``train_img`` / ``val_img`` (uint8, N x H x W x 3, RGB) and ``train_labels`` / ``val_labels``;
opened read-only in SWMR mode.  ``h5py`` is imported lazily because it is optional.
"""
from __future__ import annotations

import csv
import os
from typing import Callable, Dict, Optional

import numpy as np
import torch


def _h5py():
    try:
        import h5py
        return h5py
    except ImportError as e:  # pragma: no cover - depends on the image
        raise ImportError('the HDF5 ImageNet dataset needs h5py; use data_dir="synthetic" otherwise') from e


class DatasetHDF5(torch.utils.data.Dataset):
    def __init__(self, hdf5fn: str, t: str, transform: Optional[Callable] = None,
                 target_transform: Optional[Callable] = None):
        super().__init__()
        if t not in ('train', 'val'):
            raise ValueError("t must be 'train' or 'val'")
        self.hf = _h5py().File(hdf5fn, 'r', libver='latest', swmr=True)
        self.t = t
        self.d = self.hf['%s_img' % t]
        self.n_images = self.d.shape[0]
        self.dlabel = self.hf['%s_labels' % t][...]
        self.transform, self.target_transform = transform, target_transform

    def __getitem__(self, index):
        img, target = self.d[index, ...], np.int64(self.dlabel[index])
        if self.transform is not None:
            img = self.transform(img)
        if self.target_transform is not None:
            target = self.target_transform(target)
        return img, target

    def __len__(self):
        return self.n_images


def read_label_mapping(csv_path: str) -> Dict[str, int]:
    """``wnid -> class index`` from a two-column CSV (``scripts/imagenet_label_mapping.csv``)."""
    mapping: Dict[str, int] = {}
    with open(csv_path) as f:
        for row in csv.reader(f):
            if len(row) >= 2 and row[1].strip().lstrip('-').isdigit():
                mapping[row[0].strip()] = int(row[1])
    return mapping


def create_hdf5(image_root: str, out_file: str, label_csv: str, size: int = 256, splits=('train', 'val')) -> str:
    """Convert ``<root>/<split>/<wnid>/*.JPEG`` folders into the single-file layout above.
    Images are resized to ``size x size`` (bicubic) and stored as RGB uint8."""
    from PIL import Image
    h5py = _h5py()
    mapping = read_label_mapping(label_csv)
    with h5py.File(out_file, 'w') as hf:
        for split in splits:
            files, labels = [], []
            base = os.path.join(image_root, split)
            for wnid in sorted(os.listdir(base)):
                folder = os.path.join(base, wnid)
                if not os.path.isdir(folder) or wnid not in mapping:
                    continue
                for fn in sorted(os.listdir(folder)):
                    files.append(os.path.join(folder, fn))
                    labels.append(mapping[wnid])
            imgs = hf.create_dataset('%s_img' % split, (len(files), size, size, 3), dtype=np.uint8)
            hf.create_dataset('%s_labels' % split, data=np.asarray(labels, dtype=np.int16))
            for i, fn in enumerate(files):
                with Image.open(fn) as im:
                    imgs[i] = np.asarray(im.convert('RGB').resize((size, size), Image.BICUBIC), dtype=np.uint8)
    return out_file


def _main(argv=None):
    """``python -m mgwfbp_b200.data.hdf5 <image_root> <out.hdf5> <label_csv> [--size 256]`` converts
    ImageNet folders to the single-file layout (the reference's ``scripts/create_hdf5.py``);
    ``--show N`` prints the first N labels and image shapes of an existing file instead
    (``scripts/test_read_hdf5.py`` without the plotting)."""
    import argparse
    ap = argparse.ArgumentParser(description=_main.__doc__)
    ap.add_argument('image_root')
    ap.add_argument('out_file')
    ap.add_argument('label_csv', nargs='?')
    ap.add_argument('--size', type=int, default=256)
    ap.add_argument('--show', type=int, default=0)
    a = ap.parse_args(argv)
    if a.show:
        ds = DatasetHDF5(a.out_file, 'train')
        for i in range(min(a.show, len(ds))):
            img, label = ds[i]
            print(i, int(label), getattr(img, 'shape', None))
        return
    print(create_hdf5(a.image_root, a.out_file, a.label_csv, a.size))


if __name__ == '__main__':
    _main()
