"""Language-model workloads: an RNN language model (LSTM / GRU / tanh / ReLU RNN with
optional tied input-output embeddings) and a Transformer-encoder language model.

Same architectures and constructor arguments as the reference's
``examples/LanguageModeling/model.py:6-62,108-152`` (cuDNN RNNs through ``torch.nn``;
sequence-first tensors), written for this package.
"""
import math

import torch
import torch.nn as nn
import torch.nn.functional as F

_RNNS = {"LSTM": (nn.LSTM, {}), "GRU": (nn.GRU, {}),
         "RNN_TANH": (nn.RNN, {"nonlinearity": "tanh"}), "RNN_RELU": (nn.RNN, {"nonlinearity": "relu"})}


class RNNModel(nn.Module):
    """Embedding -> dropout -> recurrent stack -> dropout -> vocabulary projection."""

    def __init__(self, rnn_type, ntoken, ninp, nhid, nlayers, dropout=0.5, tie_weights=False):
        super().__init__()
        if rnn_type not in _RNNS:
            raise ValueError(f"rnn_type must be one of {sorted(_RNNS)}")
        if tie_weights and nhid != ninp:
            raise ValueError("When using the tied flag, nhid must be equal to emsize")
        cls, extra = _RNNS[rnn_type]
        self.rnn_type, self.ntoken, self.nhid, self.nlayers = rnn_type, ntoken, nhid, nlayers
        self.drop = nn.Dropout(dropout)
        self.encoder = nn.Embedding(ntoken, ninp)
        self.rnn = cls(ninp, nhid, nlayers, dropout=dropout, **extra)
        self.decoder = nn.Linear(nhid, ntoken)
        if tie_weights:
            self.decoder.weight = self.encoder.weight
        nn.init.uniform_(self.encoder.weight, -0.1, 0.1)
        nn.init.uniform_(self.decoder.weight, -0.1, 0.1)

    def forward(self, tokens, hidden):
        x = self.drop(self.encoder(tokens))
        out, hidden = self.rnn(x, hidden)
        logits = self.decoder(self.drop(out)).view(-1, self.ntoken)
        return F.log_softmax(logits, dim=1), hidden

    def init_hidden(self, bsz):
        w = next(self.parameters())
        h = w.new_zeros(self.nlayers, bsz, self.nhid)
        return (h, h.clone()) if self.rnn_type == "LSTM" else h


def repackage_hidden(h):
    """Detach hidden states from their history (truncated BPTT)."""
    return h.detach() if isinstance(h, torch.Tensor) else tuple(repackage_hidden(v) for v in h)


class PositionalEncoding(nn.Module):
    """Fixed sinusoidal position signal added to sequence-first embeddings."""

    def __init__(self, d_model, dropout=0.1, max_len=5000):
        super().__init__()
        self.dropout = nn.Dropout(dropout)
        pos = torch.arange(max_len).unsqueeze(1)
        freq = torch.exp(torch.arange(0, d_model, 2) * (-math.log(10000.0) / d_model))
        pe = torch.zeros(max_len, 1, d_model)
        pe[:, 0, 0::2] = torch.sin(pos * freq)
        pe[:, 0, 1::2] = torch.cos(pos * freq)
        self.register_buffer("pe", pe)

    def forward(self, x):
        return self.dropout(x + self.pe[: x.size(0)])


class TransformerModel(nn.Module):
    """Causal Transformer-encoder language model."""

    def __init__(self, ntoken, ninp, nhead, nhid, nlayers, dropout=0.5):
        super().__init__()
        self.ninp = ninp
        self.pos_encoder = PositionalEncoding(ninp, dropout)
        layer = nn.TransformerEncoderLayer(ninp, nhead, nhid, dropout)
        self.transformer_encoder = nn.TransformerEncoder(layer, nlayers)
        self.encoder = nn.Embedding(ntoken, ninp)
        self.decoder = nn.Linear(ninp, ntoken)
        nn.init.uniform_(self.encoder.weight, -0.1, 0.1)
        nn.init.zeros_(self.decoder.bias)
        nn.init.uniform_(self.decoder.weight, -0.1, 0.1)

    def forward(self, src, has_mask=True):
        mask = nn.Transformer.generate_square_subsequent_mask(src.size(0)).to(src.device) if has_mask else None
        x = self.pos_encoder(self.encoder(src) * math.sqrt(self.ninp))
        return F.log_softmax(self.decoder(self.transformer_encoder(x, mask)), dim=-1)
