"""Wide ResNet (bottleneck blocks, channels-last friendly) with torchvision
parameter names (``layer1.0.conv1.weight`` ...).  ``width_per_group`` widens
the 3x3 convolution of every bottleneck; the sizes 250M ... 4.6B use the
depths [6, 8, 46, 6]."""
from __future__ import annotations

import torch
from torch import nn

WIDERESNET_SIZES = {
    "250M": (128, [6, 8, 46, 6]),
    "1.3B": (320, [6, 8, 46, 6]),
    "2.4B": (448, [6, 8, 46, 6]),
    "3B": (512, [6, 8, 46, 6]),
    "4.6B": (640, [6, 8, 46, 6]),
}


def wideresnet_config(name):
    """``"wideresnet-250M"`` -> ``{"_name_or_path", "block_size": (width, depths)}``."""
    if not name.startswith("wideresnet-"):
        raise ValueError(f"expected 'wideresnet-<size>', got {name}")
    size = name.split("-", 1)[1]
    if size not in WIDERESNET_SIZES:
        raise ValueError(f"unknown size {size}; choose from {sorted(WIDERESNET_SIZES)}")
    return {"_name_or_path": name, "block_size": WIDERESNET_SIZES[size]}


class Bottleneck(nn.Module):
    expansion = 4

    def __init__(self, inplanes, planes, stride=1, downsample=None, base_width=64):
        super().__init__()
        width = int(planes * (base_width / 64.0))
        self.conv1 = nn.Conv2d(inplanes, width, 1, bias=False)
        self.bn1 = nn.BatchNorm2d(width)
        self.conv2 = nn.Conv2d(width, width, 3, stride=stride, padding=1, bias=False)
        self.bn2 = nn.BatchNorm2d(width)
        self.conv3 = nn.Conv2d(width, planes * self.expansion, 1, bias=False)
        self.bn3 = nn.BatchNorm2d(planes * self.expansion)
        self.relu = nn.ReLU(inplace=True)
        self.downsample = downsample

    def forward(self, x):
        identity = x
        out = self.relu(self.bn1(self.conv1(x)))
        out = self.relu(self.bn2(self.conv2(out)))
        out = self.bn3(self.conv3(out))
        if self.downsample is not None:
            identity = self.downsample(x)
        return self.relu(out + identity)


class WideResNet(nn.Module):
    def __init__(self, layers, width_per_group=64, num_classes=1000, in_channels=3):
        super().__init__()
        self.inplanes = 64
        self.base_width = width_per_group
        self.conv1 = nn.Conv2d(in_channels, 64, 7, stride=2, padding=3, bias=False)
        self.bn1 = nn.BatchNorm2d(64)
        self.relu = nn.ReLU(inplace=True)
        self.maxpool = nn.MaxPool2d(3, stride=2, padding=1)
        self.layer1 = self._make_layer(64, layers[0], 1)
        self.layer2 = self._make_layer(128, layers[1], 2)
        self.layer3 = self._make_layer(256, layers[2], 2)
        self.layer4 = self._make_layer(512, layers[3], 2)
        self.avgpool = nn.AdaptiveAvgPool2d((1, 1))
        self.fc = nn.Linear(512 * Bottleneck.expansion, num_classes)
        for m in self.modules():
            if isinstance(m, nn.Conv2d):
                nn.init.kaiming_normal_(m.weight, mode="fan_out", nonlinearity="relu")

    def _make_layer(self, planes, blocks, stride):
        downsample = None
        out = planes * Bottleneck.expansion
        if stride != 1 or self.inplanes != out:
            downsample = nn.Sequential(nn.Conv2d(self.inplanes, out, 1, stride=stride, bias=False),
                                       nn.BatchNorm2d(out))
        layers = [Bottleneck(self.inplanes, planes, stride, downsample, self.base_width)]
        self.inplanes = out
        layers += [Bottleneck(out, planes, base_width=self.base_width) for _ in range(1, blocks)]
        return nn.Sequential(*layers)

    def forward(self, x):
        x = self.maxpool(self.relu(self.bn1(self.conv1(x))))
        x = self.layer4(self.layer3(self.layer2(self.layer1(x))))
        return self.fc(torch.flatten(self.avgpool(x), 1))


class WideResNetWithLoss(nn.Module):
    """``forward(x, labels)`` -> ``{"output", "loss"}`` (cross entropy)."""

    def __init__(self, model):
        super().__init__()
        self.model = model

    def forward(self, x, labels=None):
        out = self.model(x)
        if labels is None:
            return {"output": out}
        loss = nn.functional.cross_entropy(out.float(), labels.reshape(-1))
        return {"output": out, "loss": loss}


def get_wideresnet(name_or_config, num_classes=1000):
    cfg = wideresnet_config(name_or_config) if isinstance(name_or_config, str) else name_or_config
    width, depths = cfg["block_size"]
    return WideResNetWithLoss(WideResNet(depths, width, num_classes))
