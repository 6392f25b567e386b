"""ResNet-50 (He et al. 2015, bottleneck v1) with a separate ReLU module for every use,
the property the reference's own ResNetV1 has (Model/CNN/ResNetV1.py:12-49) and torchvision's
does not: the controller keys per-layer metadata by module path."""
from __future__ import annotations

import torch
from torch import nn


class Bottleneck(nn.Module):
    expansion = 4

    def __init__(self, inplanes: int, planes: int, stride: int = 1, project: bool = False):
        super().__init__()
        out = planes * self.expansion
        self.conv1 = nn.Conv2d(inplanes, planes, 1, bias=False)
        self.bn1 = nn.BatchNorm2d(planes)
        self.relu1 = nn.ReLU()
        self.conv2 = nn.Conv2d(planes, planes, 3, stride=stride, padding=1, bias=False)
        self.bn2 = nn.BatchNorm2d(planes)
        self.relu2 = nn.ReLU()
        self.conv3 = nn.Conv2d(planes, out, 1, bias=False)
        self.bn3 = nn.BatchNorm2d(out)
        self.relu3 = nn.ReLU()
        self.shortcut = None
        if project:
            self.shortcut = nn.Sequential(nn.Conv2d(inplanes, out, 1, stride=stride, bias=False),
                                          nn.BatchNorm2d(out))

    def forward(self, x):
        y = self.relu1(self.bn1(self.conv1(x)))
        y = self.relu2(self.bn2(self.conv2(y)))
        y = self.bn3(self.conv3(y))
        skip = x if self.shortcut is None else self.shortcut(x)
        return self.relu3(y + skip)


class ResNet(nn.Module):
    def __init__(self, depths=(3, 4, 6, 3), num_classes: int = 1000):
        super().__init__()
        self.conv1 = nn.Conv2d(3, 64, 7, stride=2, padding=3, bias=False)
        self.bn1 = nn.BatchNorm2d(64)
        self.relu1 = nn.ReLU()
        self.maxpool = nn.MaxPool2d(3, stride=2, padding=1)
        stages, inplanes = [], 64
        for i, (depth, planes) in enumerate(zip(depths, (64, 128, 256, 512))):
            blocks = []
            for b in range(depth):
                stride = 2 if (b == 0 and i > 0) else 1
                blocks.append(Bottleneck(inplanes, planes, stride, project=(b == 0)))
                inplanes = planes * Bottleneck.expansion
            stages.append(nn.Sequential(*blocks))
        self.layer1, self.layer2, self.layer3, self.layer4 = stages
        self.avgpool = nn.AdaptiveAvgPool2d(1)
        self.classifier = nn.Linear(inplanes, num_classes)
        for m in self.modules():
            if isinstance(m, nn.Conv2d):
                nn.init.kaiming_normal_(m.weight, mode="fan_out", nonlinearity="relu")

    def forward(self, x):
        x = self.maxpool(self.relu1(self.bn1(self.conv1(x))))
        x = self.layer4(self.layer3(self.layer2(self.layer1(x))))
        return self.classifier(torch.flatten(self.avgpool(x), 1))


def resnet50(num_classes: int = 1000) -> ResNet:
    return ResNet((3, 4, 6, 3), num_classes)
