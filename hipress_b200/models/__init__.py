"""Model families used by the benchmarks (none exist in the reference, which has no Python)."""
from .bert import BertForMaskedLM, bert_large, bert_tiny
from .layers import FusedAddLayerNorm, FusedBatchNormAct, FusedBiasReLU, FusedLinear, MaxPool3x3s2
from .resnet import ResNet, resnet50, resnet_tiny
from .vgg import VGG, vgg19, vgg_tiny

__all__ = ["BertForMaskedLM", "FusedAddLayerNorm", "FusedBatchNormAct", "FusedBiasReLU", "FusedLinear",
           "MaxPool3x3s2", "ResNet", "VGG", "bert_large", "bert_tiny", "resnet50", "resnet_tiny",
           "vgg19", "vgg_tiny"]
