"""Any torchvision architecture on this library's kernels.

The reference's ImageNet study accepts every ``torchvision.models`` name (``models.__dict__[arch]()``,
default resnet18) and ``--pretrained`` (hw/models/train_imagenet.py:32-34,199-202). ``build_model`` serves a
name from this package's own zoo first (ResNet with fused BN+add+ReLU blocks, BERT) and otherwise builds the
torchvision model and re-classes its layers in place: ``nn.Conv2d -> ops.nn.Conv2d`` (tcgen05 GEMM /
implicit-GEMM / im2col kernels), ``nn.BatchNorm2d -> ops.nn.BatchNorm2d``, ``nn.Linear -> ops.nn.Linear``,
3x3/2 max-pool and global average pool to their kernels. Parameters, buffers and state-dict keys are
untouched, so torchvision checkpoints load as they are.
"""
from __future__ import annotations

import torch.nn as nn

from ..ops import nn as gnn


def swap_layers(model: nn.Module) -> dict:
    """Re-class the layers of ``model`` in place; returns how many of each kind were swapped."""
    counts = {"conv": 0, "bn": 0, "linear": 0, "maxpool": 0, "avgpool": 0}
    for parent in model.modules():
        for name, m in list(parent.named_children()):
            if type(m) is nn.MaxPool2d and m.kernel_size in (3, (3, 3)) and m.stride in (2, (2, 2)) \
                    and m.padding in (1, (1, 1)) and m.dilation in (1, (1, 1)) and not m.ceil_mode:
                setattr(parent, name, gnn.MaxPool3x3s2())
                counts["maxpool"] += 1
            elif type(m) is nn.AdaptiveAvgPool2d and m.output_size in (1, (1, 1)):
                setattr(parent, name, gnn.GlobalAvgPool())
                counts["avgpool"] += 1
    for m in model.modules():
        if type(m) is nn.Conv2d:
            m.__class__ = gnn.Conv2d          # same attributes; only forward differs
            counts["conv"] += 1
        elif type(m) is nn.BatchNorm2d:
            m.__class__ = gnn.BatchNorm2d
            counts["bn"] += 1
        elif type(m) is nn.Linear:
            m.__class__ = gnn.Linear
            counts["linear"] += 1
    return counts


def torchvision_names() -> list:
    import torchvision.models as tvm
    return sorted(n for n in tvm.__dict__ if n.islower() and not n.startswith("_") and callable(tvm.__dict__[n]))


def build_model(name: str, pretrained: bool = False, **kw) -> nn.Module:
    """Model ``name`` from this package's zoo or from torchvision (layers swapped to own kernels)."""
    from . import MODELS
    name = name.replace("-", "_")
    if name in MODELS and not pretrained:
        return MODELS[name](**kw)
    import torchvision.models as tvm
    if name not in tvm.__dict__ or not callable(tvm.__dict__[name]):
        raise KeyError(f"unknown architecture '{name}': not in gcow_b200.models.MODELS nor in torchvision.models")
    kw.pop("small_input", None)
    if pretrained:
        try:
            model = tvm.get_model(name, weights="DEFAULT", **{k: v for k, v in kw.items() if k != "num_classes"})
        except Exception as e:  # noqa: BLE001 - no network here: only weights already in the hub cache can load
            raise RuntimeError(f"--pretrained: the weights of '{name}' are not in the local torch hub cache and cannot "
                               f"be downloaded ({type(e).__name__}: {e}); load a checkpoint with --resume") from e
    else:
        model = tvm.__dict__[name](**kw)
    swap_layers(model)
    return model
