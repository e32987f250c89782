# -*- coding: utf-8 -*-
"""Two-layer LSTM language model for Penn Treebank.

``Embedding(V, 1500) -> Dropout(0.65) -> LSTM(1500, 1500, 2 layers, dropout 0.65) -> Dropout ->
Linear(1500, V)`` with the parameter names of reference ``models/lstm.py:5-47``
(``word_embeddings.weight``, ``lstm.weight_ih_l0`` ..., ``sm_fc.weight``).  The recurrent part is
either ``torch.nn.LSTM`` (cuDNN) or this package's :class:`~mgwfbp_b200.ops.lstm.FusedLSTM`,
which exposes the same parameter names and shapes.
"""
from __future__ import annotations

import torch
import torch.nn as nn


class lstm(nn.Module):
    def __init__(self, vocab_size, embedding_dim=1500, num_steps=35, batch_size=20, num_layers=2,
                 dp_keep_prob=0.35, fused=False):
        super().__init__()
        self.name = 'lstm'
        self.embedding_dim = embedding_dim
        self.num_steps = num_steps
        self.batch_size = batch_size
        self.vocab_size = vocab_size
        self.dp_keep_prob = dp_keep_prob
        self.num_layers = num_layers
        self.dropout = nn.Dropout(1 - dp_keep_prob)
        self.word_embeddings = nn.Embedding(vocab_size, embedding_dim)
        if fused:
            from ..ops.lstm import FusedLSTM
            self.lstm = FusedLSTM(embedding_dim, embedding_dim, num_layers=num_layers, dropout=1 - dp_keep_prob)
        else:
            self.lstm = nn.LSTM(input_size=embedding_dim, hidden_size=embedding_dim, num_layers=num_layers,
                                dropout=1 - dp_keep_prob)
        self.sm_fc = nn.Linear(embedding_dim, vocab_size)
        self.init_weights()

    def init_weights(self):
        r = 0.1
        nn.init.uniform_(self.word_embeddings.weight, -r, r)
        nn.init.zeros_(self.sm_fc.bias)
        nn.init.uniform_(self.sm_fc.weight, -r, r)

    def init_hidden(self):
        ref = next(self.parameters())
        shape = (self.num_layers, self.batch_size, self.embedding_dim)
        return (ref.new_zeros(shape), ref.new_zeros(shape))

    def forward(self, inputs, hidden):
        embeds = self.dropout(self.word_embeddings(inputs))
        out, hidden = self.lstm(embeds, hidden)
        out = self.dropout(out)
        logits = self.sm_fc(out.reshape(-1, self.embedding_dim))
        return logits.view(self.num_steps, self.batch_size, self.vocab_size), hidden


def repackage_hidden(h):
    """Detach hidden state from the graph of the previous truncated-BPTT window."""
    if torch.is_tensor(h):
        return h.detach()
    return tuple(repackage_hidden(v) for v in h)
