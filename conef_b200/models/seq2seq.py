"""Encoder-decoder Transformer for translation: ``nn.Transformer`` with scaled token
embeddings, sinusoidal positions and a generator, plus the mask helpers.

Same structure and call signature as the reference's
``examples/MachineTranslation/model.py:44-88`` and ``train_n_test.py:23-41``.
"""
import math

import torch
import torch.nn as nn

from .language import PositionalEncoding

PAD_IDX = 1


class TokenEmbedding(nn.Module):
    def __init__(self, vocab_size, emb_size):
        super().__init__()
        self.embedding = nn.Embedding(vocab_size, emb_size)
        self.emb_size = emb_size

    def forward(self, tokens):
        return self.embedding(tokens.long()) * math.sqrt(self.emb_size)


class Seq2SeqTransformer(nn.Module):
    def __init__(self, num_encoder_layers, num_decoder_layers, emb_size, nhead, src_vocab_size, tgt_vocab_size,
                 dim_feedforward=512, dropout=0.1):
        super().__init__()
        self.transformer = nn.Transformer(d_model=emb_size, nhead=nhead, num_encoder_layers=num_encoder_layers,
                                          num_decoder_layers=num_decoder_layers, dim_feedforward=dim_feedforward,
                                          dropout=dropout)
        self.generator = nn.Linear(emb_size, tgt_vocab_size)
        self.src_tok_emb = TokenEmbedding(src_vocab_size, emb_size)
        self.tgt_tok_emb = TokenEmbedding(tgt_vocab_size, emb_size)
        self.positional_encoding = PositionalEncoding(emb_size, dropout=dropout)

    def forward(self, src, trg, src_mask, tgt_mask, src_padding_mask, tgt_padding_mask, memory_key_padding_mask):
        src_emb = self.positional_encoding(self.src_tok_emb(src))
        tgt_emb = self.positional_encoding(self.tgt_tok_emb(trg))
        out = self.transformer(src_emb, tgt_emb, src_mask, tgt_mask, None, src_padding_mask, tgt_padding_mask,
                               memory_key_padding_mask)
        return self.generator(out)

    def encode(self, src, src_mask):
        return self.transformer.encoder(self.positional_encoding(self.src_tok_emb(src)), src_mask)

    def decode(self, tgt, memory, tgt_mask):
        return self.transformer.decoder(self.positional_encoding(self.tgt_tok_emb(tgt)), memory, tgt_mask)


def generate_square_subsequent_mask(sz, device):
    return torch.triu(torch.full((sz, sz), float("-inf"), device=device), diagonal=1)


def create_mask(src, tgt, pad_idx=PAD_IDX):
    """(src_mask, tgt_mask, src_padding_mask, tgt_padding_mask) for sequence-first batches."""
    src_len, tgt_len = src.shape[0], tgt.shape[0]
    tgt_mask = generate_square_subsequent_mask(tgt_len, src.device)
    src_mask = torch.zeros((src_len, src_len), device=src.device)
    # float masks (0 / -inf) so that every mask handed to the attention has one dtype
    src_pad = torch.zeros(src.shape[1], src_len, device=src.device).masked_fill((src == pad_idx).t(), float("-inf"))
    tgt_pad = torch.zeros(tgt.shape[1], tgt_len, device=src.device).masked_fill((tgt == pad_idx).t(), float("-inf"))
    return src_mask, tgt_mask, src_pad, tgt_pad
