"""Plain-PyTorch ResNet-18 with GroupNorm used ONLY by the reference arm of
``opacus_b200/benchmarks/resnet_ddp.py`` (``--impl reference``); imports nothing from ``opacus_b200``.
"""
import torch.nn as nn
import torch.nn.functional as F


def _gn(ch: int, groups: int) -> nn.GroupNorm:
    return nn.GroupNorm(min(groups, ch), ch)


class BasicBlock(nn.Module):
    def __init__(self, cin: int, cout: int, stride: int, groups: int):
        super().__init__()
        self.conv1 = nn.Conv2d(cin, cout, 3, stride, 1, bias=False)
        self.gn1 = _gn(cout, groups)
        self.conv2 = nn.Conv2d(cout, cout, 3, 1, 1, bias=False)
        self.gn2 = _gn(cout, groups)
        self.short = None
        if stride != 1 or cin != cout:
            self.short = nn.Sequential(nn.Conv2d(cin, cout, 1, stride, bias=False), _gn(cout, groups))

    def forward(self, x):
        y = F.relu(self.gn1(self.conv1(x)))
        y = self.gn2(self.conv2(y))
        return F.relu(y + (x if self.short is None else self.short(x)))


class ResNet18GN(nn.Module):
    def __init__(self, num_classes: int = 10, groups: int = 32):
        super().__init__()
        self.conv1 = nn.Conv2d(3, 64, 3, 1, 1, bias=False)
        self.gn1 = _gn(64, groups)
        cfg = [(64, 1), (64, 1), (128, 2), (128, 1), (256, 2), (256, 1), (512, 2), (512, 1)]
        blocks, cin = [], 64
        for cout, stride in cfg:
            blocks.append(BasicBlock(cin, cout, stride, groups))
            cin = cout
        self.layers = nn.Sequential(*blocks)
        self.fc = nn.Linear(512, num_classes)

    def forward(self, x):
        x = F.relu(self.gn1(self.conv1(x)))
        x = self.layers(x)
        x = F.adaptive_avg_pool2d(x, 1).flatten(1)
        return self.fc(x)


def resnet18_gn(num_classes: int = 10, groups: int = 32) -> ResNet18GN:
    return ResNet18GN(num_classes, groups)
