"""Data utilities: synthetic datasets of the benchmark shapes, corpus batching, MLM masking, WordPiece."""
from .corpus import Corpus, Dictionary, batchify, get_batch
from . import glue
from . import squad
from .masking import mask_tokens
from .pretraining import (PretrainingShard, ShardPrefetcher, create_training_instances, instances_to_arrays,
                          load_shard, read_documents, shard_files, write_shard)
from .synthetic import (SyntheticBertShard, SyntheticImages, SyntheticTranslationPairs, collate_translation,
                        synthetic_token_stream)
from .translation import ParallelText, build_vocab
from .tokenization import BasicTokenizer, BertTokenizer, WordpieceTokenizer

__all__ = ["Corpus", "Dictionary", "batchify", "get_batch", "mask_tokens", "SyntheticBertShard", "SyntheticImages",
           "SyntheticTranslationPairs", "collate_translation", "synthetic_token_stream", "BasicTokenizer",
           "BertTokenizer", "WordpieceTokenizer", "PretrainingShard", "ShardPrefetcher", "create_training_instances",
           "instances_to_arrays", "load_shard", "read_documents", "shard_files", "write_shard", "ParallelText", "build_vocab", "glue", "squad"]
