# -*- coding: utf-8 -*-
"""Gradient compressor registry.

Like the reference (``compression.py:5-19``) only the identity compressor exists; the
``--compressor`` / ``--density`` flags are plumbed through for call compatibility.
"""


class NoneCompressor:
    @staticmethod
    def compress(tensor, name=None):
        return tensor, tensor.dtype

    @staticmethod
    def decompress(tensor, ctc, name=None):
        return tensor


compressors = {'none': NoneCompressor, None: NoneCompressor}
