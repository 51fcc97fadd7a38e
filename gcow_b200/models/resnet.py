"""ResNet-50/101/152 (bottleneck) and ResNet-18/34 (basic block) for NHWC bf16 training.

Same architecture family as the reference's model zoo (hw/models/resenet.py:6-134:
1x1 -> 3x3(stride) -> 1x1x4 bottlenecks, 7x7/2 stem, 3x3/2 max-pool, four stages of
64/128/256/512 planes, global average pool, FC) with two of its defects not
reproduced: its basic block applies the second batch-norm twice and never the
first (hw/models/resenet.py:60-61), and its convolutions keep a bias in front of
batch-norm. Layers come from gcow_b200.ops.nn so that the sm_100a kernels are
used where they exist.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ..ops import nn as gnn


class Bottleneck(nn.Module):
    expansion = 4

    def __init__(self, inplanes: int, planes: int, stride: int = 1, downsample: nn.Module | None = None):
        super().__init__()
        self.conv1 = gnn.Conv2d(inplanes, planes, 1, bias=False)
        self.bn1 = gnn.BatchNorm2d(planes)
        self.conv2 = gnn.Conv2d(planes, planes, 3, stride=stride, padding=1, bias=False)
        self.bn2 = gnn.BatchNorm2d(planes)
        self.conv3 = gnn.Conv2d(planes, planes * 4, 1, bias=False)
        self.bn3 = gnn.BatchNorm2d(planes * 4)
        self.relu = nn.ReLU(inplace=True)
        self.downsample = downsample
        self.fork = False        # set by ResNet: the output feeds the next block's two branches

    def forward(self, x):
        # a forked input is a pair of tensors on the same memory, one per branch (see gnn.BatchNorm2d)
        xa, xb = x if isinstance(x, tuple) else (x, x)
        idt = xb if self.downsample is None else self.downsample(xb)
        out = self.bn1(self.conv1(xa), relu=True)
        out = self.bn2(self.conv2(out), relu=True)
        return self.bn3(self.conv3(out), residual=idt, relu=True, fork=self.fork)


class BasicBlock(nn.Module):
    expansion = 1

    def __init__(self, inplanes: int, planes: int, stride: int = 1, downsample: nn.Module | None = None):
        super().__init__()
        self.conv1 = gnn.Conv2d(inplanes, planes, 3, stride=stride, padding=1, bias=False)
        self.bn1 = gnn.BatchNorm2d(planes)
        self.conv2 = gnn.Conv2d(planes, planes, 3, padding=1, bias=False)
        self.bn2 = gnn.BatchNorm2d(planes)
        self.relu = nn.ReLU(inplace=True)
        self.downsample = downsample
        self.fork = False

    def forward(self, x):
        xa, xb = x if isinstance(x, tuple) else (x, x)
        idt = xb if self.downsample is None else self.downsample(xb)
        out = self.bn1(self.conv1(xa), relu=True)
        return self.bn2(self.conv2(out), residual=idt, relu=True, fork=self.fork)


class ResNet(nn.Module):
    def __init__(self, block, layers, num_classes: int = 1000, in_channels: int = 3, small_input: bool = False):
        super().__init__()
        self.inplanes = 64
        if small_input:   # CIFAR-style stem: 3x3/1 and no max-pool
            self.conv1 = gnn.Conv2d(in_channels, 64, 3, stride=1, padding=1, bias=False)
            self.maxpool = nn.Identity()
        else:
            self.conv1 = gnn.Conv2d(in_channels, 64, 7, stride=2, padding=3, bias=False)
            self.maxpool = gnn.MaxPool3x3s2()
        self.bn1 = gnn.BatchNorm2d(64)
        self.relu = nn.ReLU(inplace=True)
        self.layer1 = self._make_layer(block, 64, layers[0], 1)
        self.layer2 = self._make_layer(block, 128, layers[1], 2)
        self.layer3 = self._make_layer(block, 256, layers[2], 2)
        self.layer4 = self._make_layer(block, 512, layers[3], 2)
        self.avgpool = gnn.GlobalAvgPool()
        self.fc = gnn.Linear(512 * block.expansion, num_classes)
        for m in self.modules():
            if isinstance(m, nn.Conv2d):
                nn.init.kaiming_normal_(m.weight, mode="fan_out", nonlinearity="relu")
        blocks = [b for layer in (self.layer1, self.layer2, self.layer3, self.layer4) for b in layer]
        for b in blocks[:-1]:              # every block output but the last feeds two branches of the next block
            b.fork = True
        for m in self.modules():           # zero-init the last BN of every residual branch
            if isinstance(m, Bottleneck):
                nn.init.zeros_(m.bn3.weight)
            elif isinstance(m, BasicBlock):
                nn.init.zeros_(m.bn2.weight)

    def _make_layer(self, block, planes, blocks, stride):
        down = None
        if stride != 1 or self.inplanes != planes * block.expansion:
            down = nn.Sequential(gnn.Conv2d(self.inplanes, planes * block.expansion, 1, stride=stride, bias=False),
                                 gnn.BatchNorm2d(planes * block.expansion))
        layers = [block(self.inplanes, planes, stride, down)]
        self.inplanes = planes * block.expansion
        layers += [block(self.inplanes, planes) for _ in range(1, blocks)]
        return nn.Sequential(*layers)

    def forward(self, x):
        x = self.maxpool(self.bn1(self.conv1(x), relu=True))
        x = self.layer4(self.layer3(self.layer2(self.layer1(x))))
        x = torch.flatten(self.avgpool(x), 1)
        return self.fc(x)


def resnet18(num_classes=1000, **kw): return ResNet(BasicBlock, [2, 2, 2, 2], num_classes, **kw)
def resnet34(num_classes=1000, **kw): return ResNet(BasicBlock, [3, 4, 6, 3], num_classes, **kw)
def resnet50(num_classes=1000, **kw): return ResNet(Bottleneck, [3, 4, 6, 3], num_classes, **kw)
def resnet101(num_classes=1000, **kw): return ResNet(Bottleneck, [3, 4, 23, 3], num_classes, **kw)
def resnet152(num_classes=1000, **kw): return ResNet(Bottleneck, [3, 8, 36, 3], num_classes, **kw)
