"""CLIP's modified ResNet as image tower (src/scaling/transformer/model/image_encoder/clip.py:22-168).

Differences from the torchvision ResNet, as in the CLIP release: a three-convolution stem followed by an average
pool, anti-aliased strided blocks (average pool before every convolution that would have had a stride), and no
classification head - the forward pass returns the final feature map as a token sequence ``[batch, h * w, channels]``.
Module and parameter names follow the CLIP checkpoints (``conv1 .. bn3``, ``layer1 .. layer4``, ``downsample.-1/0/1``)
so that published weights load unchanged.  Convolutions and batch norms run on cuDNN.
"""

from __future__ import annotations

from collections import OrderedDict
from typing import Any, Callable

import torch
from torch import nn

CLIP_MEAN = (0.48145466, 0.4578275, 0.40821073)
CLIP_STD = (0.26862954, 0.26130258, 0.27577711)


def clip_transform(n_px: tuple[int, int]) -> Callable[[Any], torch.Tensor]:
    """PIL image -> bicubic resize to ``n_px`` -> centre crop -> RGB -> tensor normalised with CLIP's statistics."""
    from torchvision.transforms import CenterCrop, Compose, InterpolationMode, Normalize, Resize, ToTensor

    return Compose([
        Resize(n_px, interpolation=InterpolationMode.BICUBIC),
        CenterCrop(n_px),
        lambda image: image.convert("RGB"),
        ToTensor(),
        Normalize(CLIP_MEAN, CLIP_STD),
    ])


class Bottleneck(nn.Module):
    """1x1 -> 3x3 -> (avg pool) -> 1x1 with a residual connection; output channels = 4 x ``planes``."""

    expansion = 4

    def __init__(self, inplanes: int, planes: int, stride: int = 1) -> None:
        super().__init__()
        out_planes = planes * self.expansion
        self.conv1 = nn.Conv2d(inplanes, planes, 1, bias=False)
        self.bn1 = nn.BatchNorm2d(planes)
        self.conv2 = nn.Conv2d(planes, planes, 3, padding=1, bias=False)
        self.bn2 = nn.BatchNorm2d(planes)
        self.avgpool = nn.AvgPool2d(stride) if stride > 1 else nn.Identity()
        self.conv3 = nn.Conv2d(planes, out_planes, 1, bias=False)
        self.bn3 = nn.BatchNorm2d(out_planes)
        self.relu = nn.ReLU(inplace=True)
        self.stride = stride
        self.downsample = None
        if stride > 1 or inplanes != out_planes:
            # the shortcut is pooled first; its convolution keeps stride 1
            self.downsample = nn.Sequential(OrderedDict([
                ("-1", nn.AvgPool2d(stride)),
                ("0", nn.Conv2d(inplanes, out_planes, 1, stride=1, bias=False)),
                ("1", nn.BatchNorm2d(out_planes)),
            ]))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shortcut = x if self.downsample is None else self.downsample(x)
        y = self.relu(self.bn1(self.conv1(x)))
        y = self.avgpool(self.relu(self.bn2(self.conv2(y))))
        y = self.bn3(self.conv3(y))
        return self.relu(y + shortcut)


class ClipModifiedResNet(nn.Module):
    def __init__(self, layers: list[int], num_init_channels: int = 64):
        super().__init__()
        c = num_init_channels
        self.conv1 = nn.Conv2d(3, c // 2, kernel_size=3, stride=2, padding=1, bias=False)
        self.bn1 = nn.BatchNorm2d(c // 2)
        self.conv2 = nn.Conv2d(c // 2, c // 2, kernel_size=3, padding=1, bias=False)
        self.bn2 = nn.BatchNorm2d(c // 2)
        self.conv3 = nn.Conv2d(c // 2, c, kernel_size=3, padding=1, bias=False)
        self.bn3 = nn.BatchNorm2d(c)
        self.avgpool = nn.AvgPool2d(2)
        self.relu = nn.ReLU(inplace=True)
        inplanes = c
        for i, (blocks, stride) in enumerate(zip(layers, (1, 2, 2, 2))):
            planes = c * 2 ** i
            stage = [Bottleneck(inplanes, planes, stride)]
            inplanes = planes * Bottleneck.expansion
            stage += [Bottleneck(inplanes, planes) for _ in range(1, blocks)]
            setattr(self, f"layer{i + 1}", nn.Sequential(*stage))
        self.output_channels = inplanes

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x = x.type(self.conv1.weight.dtype)
        for conv, bn in ((self.conv1, self.bn1), (self.conv2, self.bn2), (self.conv3, self.bn3)):
            x = self.relu(bn(conv(x)))
        x = self.avgpool(x)
        x = self.layer4(self.layer3(self.layer2(self.layer1(x))))
        return x.flatten(2).transpose(1, 2)  # [b, c, h, w] -> [b, h * w, c]
