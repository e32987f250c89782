# -*- coding: utf-8 -*-
"""Drop-in module for ``import ptb_reader``."""
from mgwfbp_b200.data.ptb import (_read_words, _build_vocab, _file_to_word_ids, ptb_raw_data,  # noqa: F401
                                  TrainDataset, TestDataset)
