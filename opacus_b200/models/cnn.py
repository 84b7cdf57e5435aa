"""The small MNIST-style CNN used for CPU runs: two conv layers with max
pooling of stride 1 (which makes the flattened size 512) and two linear layers
(same architecture as ``examples/mnist.py:38-55`` of the reference)."""
import torch.nn as nn
import torch.nn.functional as F


class SmallCNN(nn.Module):
    def __init__(self, num_classes: int = 10):
        super().__init__()
        self.conv1 = nn.Conv2d(1, 16, 8, 2, padding=3)
        self.conv2 = nn.Conv2d(16, 32, 4, 2)
        self.fc1 = nn.Linear(32 * 4 * 4, 32)
        self.fc2 = nn.Linear(32, num_classes)

    def forward(self, x):
        x = F.max_pool2d(F.relu(self.conv1(x)), 2, 1)   # 16 x 13 x 13
        x = F.max_pool2d(F.relu(self.conv2(x)), 2, 1)   # 32 x 4 x 4
        x = x.flatten(1)
        return self.fc2(F.relu(self.fc1(x)))
