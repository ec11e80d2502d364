"""Model zoo of the example workloads (framework-layer PyTorch code)."""
from . import seq2seq
from .bert import (BertConfig, BertForMaskedLM, BertForPreTraining, BertForQuestionAnswering,
                   BertForSequenceClassification, BertModel, BertPretrainingCriterion)
from .language import PositionalEncoding, RNNModel, TransformerModel, repackage_hidden
from .seq2seq import Seq2SeqTransformer, create_mask
from .resnet_cifar import CifarResNet, ResNet20, ResNet32, ResNet56
from .wideresnet import WideResNet, WideResNet28_10, WideResNet40_10

__all__ = ["BertConfig", "BertModel", "BertForPreTraining", "BertForMaskedLM", "BertForSequenceClassification",
           "BertForQuestionAnswering", "BertPretrainingCriterion", "RNNModel", "TransformerModel",
           "PositionalEncoding", "repackage_hidden", "Seq2SeqTransformer", "create_mask", "seq2seq",
           "CifarResNet", "ResNet20", "ResNet32", "ResNet56", "WideResNet", "WideResNet28_10", "WideResNet40_10"]
