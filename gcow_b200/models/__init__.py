from .resnet import resnet18, resnet34, resnet50, resnet101, resnet152, ResNet
from .bert import BertConfig, BertForPreTraining, bert_large, bert_base, bert_tiny

MODELS = {
    "resnet18": resnet18, "resnet34": resnet34, "resnet50": resnet50, "resnet101": resnet101,
    "resnet152": resnet152, "bert_large": bert_large, "bert_base": bert_base, "bert_tiny": bert_tiny,
}

from .zoo import build_model, swap_layers, torchvision_names  # noqa: E402

__all__ = ["MODELS", "ResNet", "BertConfig", "BertForPreTraining", "build_model", "swap_layers",
           "torchvision_names"] + list(MODELS)
