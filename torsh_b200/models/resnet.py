"""ResNet / ResNeXt / Wide-ResNet (``crates/torsh-models/src/vision/resnet/models.rs:17-205``, ``config.rs:7-280``).

torchvision-v1 layout as in the reference: 7×7/2 conv (pad 3, no bias) → BN → ReLU → 3×3/2 max-pool (pad 1) → four
stages (``[3,4,6,3]`` bottlenecks for ResNet-50; 1×1 conv + BN down-sample when the stride or the channel count
changes) → adaptive average pool → ``Linear(2048, classes)``; options: SE blocks, dropout, ResNeXt ``groups`` /
``width_per_group``. Convolutions use Kaiming-normal (fan-out) init and run in channels-last.

On a GPU (plain ResNets: no groups, no SE) the forward pass runs channels-last bf16 end to end on the sm_100a kernels of
``torsh_b200.ops.conv``: every convolution is a tcgen05 GEMM, BatchNorm + ReLU (+ the residual add that closes a block)
is one fused pass, and parameters stay fp32 (bf16 autocast recipe).  ``model.use_kernels = False`` keeps PyTorch's
layers.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from .. import nn
from ..ops import conv as cv


@dataclass
class ResNetConfig:
    block: str = "bottleneck"
    layers: tuple = (3, 4, 6, 3)
    num_classes: int = 1000
    groups: int = 1
    width_per_group: int = 64
    use_se: bool = False
    se_reduction: int = 16
    dropout: float = 0.0
    zero_init_residual: bool = False

    @classmethod
    def resnet18(cls, **kw): return cls(block="basic", layers=(2, 2, 2, 2), **kw)
    @classmethod
    def resnet34(cls, **kw): return cls(block="basic", layers=(3, 4, 6, 3), **kw)
    @classmethod
    def resnet50(cls, **kw): return cls(layers=(3, 4, 6, 3), **kw)
    @classmethod
    def resnet101(cls, **kw): return cls(layers=(3, 4, 23, 3), **kw)
    @classmethod
    def resnet152(cls, **kw): return cls(layers=(3, 8, 36, 3), **kw)
    @classmethod
    def resnext50_32x4d(cls, **kw): return cls(groups=32, width_per_group=4, **kw)
    @classmethod
    def wide_resnet50_2(cls, **kw): return cls(width_per_group=128, **kw)


class SEBlock(nn.Module):
    def __init__(self, channels: int, reduction: int = 16):
        super().__init__()
        self.fc1 = nn.Conv2d(channels, channels // reduction, 1)
        self.fc2 = nn.Conv2d(channels // reduction, channels, 1)

    def forward(self, x):
        s = x.mean((2, 3), keepdim=True)
        return x * torch.sigmoid(self.fc2(torch.relu(self.fc1(s))))


class BasicBlock(nn.Module):
    expansion = 1

    def __init__(self, inplanes, planes, stride=1, downsample=None, groups=1, base_width=64, use_se=False, se_reduction=16):
        super().__init__()
        self.conv1 = nn.Conv2d(inplanes, planes, 3, stride, 1, bias=False)
        self.bn1 = nn.BatchNorm2d(planes)
        self.conv2 = nn.Conv2d(planes, planes, 3, 1, 1, bias=False)
        self.bn2 = nn.BatchNorm2d(planes)
        self.se = SEBlock(planes, se_reduction) if use_se else None
        self.downsample = downsample

    def forward(self, x):
        idt = x if self.downsample is None else self.downsample(x)
        out = torch.relu(self.bn1(self.conv1(x)))
        out = self.bn2(self.conv2(out))
        if self.se is not None:
            out = self.se(out)
        return torch.relu(out + idt)

    def forward_nhwc(self, x):
        idt = x if self.downsample is None else _down_nhwc(self.downsample, x)
        out = cv.batch_norm_nhwc(_conv_nhwc(self.conv1, x), self.bn1, relu=True)
        return cv.batch_norm_nhwc(_conv_nhwc(self.conv2, out), self.bn2, residual=idt, relu=True)


class BottleneckBlock(nn.Module):
    expansion = 4

    def __init__(self, inplanes, planes, stride=1, downsample=None, groups=1, base_width=64, use_se=False, se_reduction=16):
        super().__init__()
        width = int(planes * (base_width / 64.0)) * groups
        self.conv1 = nn.Conv2d(inplanes, width, 1, bias=False)
        self.bn1 = nn.BatchNorm2d(width)
        self.conv2 = nn.Conv2d(width, width, 3, stride, 1, groups=groups, bias=False)
        self.bn2 = nn.BatchNorm2d(width)
        self.conv3 = nn.Conv2d(width, planes * 4, 1, bias=False)
        self.bn3 = nn.BatchNorm2d(planes * 4)
        self.se = SEBlock(planes * 4, se_reduction) if use_se else None
        self.downsample = downsample

    def forward(self, x):
        idt = x if self.downsample is None else self.downsample(x)
        out = torch.relu(self.bn1(self.conv1(x)))
        out = torch.relu(self.bn2(self.conv2(out)))
        out = self.bn3(self.conv3(out))
        if self.se is not None:
            out = self.se(out)
        return torch.relu(out + idt)

    def forward_nhwc(self, x):
        idt = x if self.downsample is None else _down_nhwc(self.downsample, x)
        out = cv.batch_norm_nhwc(_conv_nhwc(self.conv1, x), self.bn1, relu=True)
        out = cv.batch_norm_nhwc(_conv_nhwc(self.conv2, out), self.bn2, relu=True)
        return cv.batch_norm_nhwc(_conv_nhwc(self.conv3, out), self.bn3, residual=idt, relu=True)


def _conv_nhwc(conv: torch.nn.Conv2d, x):
    return cv.conv2d_nhwc(x, conv.weight, conv.stride[0], conv.padding[0])


def _down_nhwc(seq, x):
    return cv.batch_norm_nhwc(_conv_nhwc(seq[0], x), seq[1])


class ResNet(nn.Module):
    def __init__(self, cfg: ResNetConfig | None = None):
        super().__init__()
        cfg = cfg or ResNetConfig()
        self.config = cfg
        block = BasicBlock if cfg.block == "basic" else BottleneckBlock
        self.inplanes = 64
        self.conv1 = nn.Conv2d(3, 64, 7, 2, 3, bias=False)
        self.bn1 = nn.BatchNorm2d(64)
        self.maxpool = nn.MaxPool2d(3, 2, 1)
        self.layer1 = self._make(block, 64, cfg.layers[0], 1, cfg)
        self.layer2 = self._make(block, 128, cfg.layers[1], 2, cfg)
        self.layer3 = self._make(block, 256, cfg.layers[2], 2, cfg)
        self.layer4 = self._make(block, 512, cfg.layers[3], 2, cfg)
        self.avgpool = nn.AdaptiveAvgPool2d((1, 1))
        self.dropout = nn.Dropout(cfg.dropout) if cfg.dropout > 0 else None
        self.fc = nn.Linear(512 * block.expansion, cfg.num_classes)
        for m in self.modules():
            if isinstance(m, torch.nn.Conv2d):
                torch.nn.init.kaiming_normal_(m.weight, mode="fan_out", nonlinearity="relu")
            elif isinstance(m, torch.nn.BatchNorm2d):
                torch.nn.init.ones_(m.weight)
                torch.nn.init.zeros_(m.bias)
        if cfg.zero_init_residual:
            for m in self.modules():
                if isinstance(m, BottleneckBlock):
                    torch.nn.init.zeros_(m.bn3.weight)
                elif isinstance(m, BasicBlock):
                    torch.nn.init.zeros_(m.bn2.weight)

    def _make(self, block, planes, n, stride, cfg):
        down = None
        if stride != 1 or self.inplanes != planes * block.expansion:
            down = nn.Sequential(nn.Conv2d(self.inplanes, planes * block.expansion, 1, stride, bias=False),
                                 nn.BatchNorm2d(planes * block.expansion))
        kw = dict(groups=cfg.groups, base_width=cfg.width_per_group, use_se=cfg.use_se, se_reduction=cfg.se_reduction)
        layers = [block(self.inplanes, planes, stride, down, **kw)]
        self.inplanes = planes * block.expansion
        layers += [block(self.inplanes, planes, **kw) for _ in range(1, n)]
        return nn.Sequential(*layers)

    def forward_features(self, x):
        x = self.maxpool(torch.relu(self.bn1(self.conv1(x))))
        return self.layer4(self.layer3(self.layer2(self.layer1(x))))

    use_kernels = True

    def _kernel_path(self, x) -> bool:
        return (self.use_kernels and x.is_cuda and self.config.groups == 1 and not self.config.use_se
                and self.config.width_per_group % 8 == 0)

    def forward_nhwc(self, x):
        """Channels-last bf16 pass; ``x`` is ``[N, 3, H, W]`` (any float dtype).  Returns fp32 logits."""
        from ..ops.linear import linear
        x = x.permute(0, 2, 3, 1).to(torch.bfloat16).contiguous()
        x = cv.batch_norm_nhwc(_conv_nhwc(self.conv1, x), self.bn1, relu=True)
        x = cv.max_pool_nhwc(x, 3, 2, 1)
        for stage in (self.layer1, self.layer2, self.layer3, self.layer4):
            for blk in stage:
                x = blk.forward_nhwc(x)
        x = cv.global_avg_pool_nhwc(x)
        if self.dropout is not None:
            x = self.dropout(x)
        return linear(x, self.fc.weight.to(torch.bfloat16), self.fc.bias.to(torch.bfloat16)).float()

    def forward(self, x):
        if self._kernel_path(x):
            return self.forward_nhwc(x)
        x = torch.flatten(self.avgpool(self.forward_features(x)), 1)
        if self.dropout is not None:
            x = self.dropout(x)
        return self.fc(x)

    @classmethod
    def resnet18(cls, num_classes=1000): return cls(ResNetConfig.resnet18(num_classes=num_classes))
    @classmethod
    def resnet34(cls, num_classes=1000): return cls(ResNetConfig.resnet34(num_classes=num_classes))
    @classmethod
    def resnet50(cls, num_classes=1000): return cls(ResNetConfig.resnet50(num_classes=num_classes))
    @classmethod
    def resnet101(cls, num_classes=1000): return cls(ResNetConfig.resnet101(num_classes=num_classes))
    @classmethod
    def resnet152(cls, num_classes=1000): return cls(ResNetConfig.resnet152(num_classes=num_classes))
