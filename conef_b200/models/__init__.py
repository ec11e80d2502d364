"""Model zoo of the example workloads (framework-layer PyTorch code)."""
from . import seq2seq
from .bert import (BertConfig, BertForMaskedLM, BertForMultipleChoice, BertForNextSentencePrediction,
                   BertForPreTraining, BertForQuestionAnswering, BertForSequenceClassification,
                   BertForTokenClassification, BertModel, BertPreTrainedModel, BertPretrainingCriterion,
                   load_tf_weights_in_bert, tf_variable_names)
from .language import PositionalEncoding, RNNModel, TransformerModel, repackage_hidden
from .seq2seq import Seq2SeqTransformer, create_mask
from .densenet import DenseNet, DenseNet121, DenseNet161, DenseNet169, DenseNet201, densenet_cifar
from .mobile import MobileNetV2, ShuffleNetV2
from .resnet import ResNet, ResNet18, ResNet34, ResNet50, ResNet101, ResNet152
from .resnext import ResNeXt, ResNeXt29_2x64d, ResNeXt29_4x64d, ResNeXt29_8x64d, ResNeXt29_32x4d
from .small_cnns import VGG, LeNet
from .resnet_cifar import CifarResNet, ResNet20, ResNet32, ResNet56
from .wideresnet import WideResNet, WideResNet28_10, WideResNet40_10

__all__ = ["BertConfig", "BertModel", "BertForPreTraining", "BertForMaskedLM", "BertForSequenceClassification",
           "BertForQuestionAnswering", "BertPretrainingCriterion", "RNNModel", "TransformerModel",
           "DenseNet", "DenseNet121", "DenseNet161", "DenseNet169", "DenseNet201", "densenet_cifar", "MobileNetV2",
           "ShuffleNetV2", "ResNet", "ResNet18", "ResNet34", "ResNet50", "ResNet101", "ResNet152", "ResNeXt",
           "ResNeXt29_2x64d", "ResNeXt29_4x64d", "ResNeXt29_8x64d", "ResNeXt29_32x4d", "VGG", "LeNet",
           "PositionalEncoding", "repackage_hidden", "Seq2SeqTransformer", "create_mask", "seq2seq",
           "CifarResNet", "ResNet20", "ResNet32", "ResNet56", "WideResNet", "WideResNet28_10", "WideResNet40_10"]
