"""Data utilities: synthetic datasets of the benchmark shapes, corpus batching, MLM masking, WordPiece."""
from .corpus import Corpus, Dictionary, batchify, get_batch
from .masking import mask_tokens
from .synthetic import (SyntheticBertShard, SyntheticImages, SyntheticTranslationPairs, collate_translation,
                        synthetic_token_stream)
from .tokenization import BasicTokenizer, BertTokenizer, WordpieceTokenizer

__all__ = ["Corpus", "Dictionary", "batchify", "get_batch", "mask_tokens", "SyntheticBertShard", "SyntheticImages",
           "SyntheticTranslationPairs", "collate_translation", "synthetic_token_stream", "BasicTokenizer",
           "BertTokenizer", "WordpieceTokenizer"]
