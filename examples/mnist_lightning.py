"""DP training inside a LightningModule: the privacy engine is attached in ``configure_optimizers`` and the data
module is wrapped so that batches are Poisson sampled.  Needs ``lightning`` (or ``pytorch_lightning``).

Counterpart in the reference: ``examples/mnist_lightning.py``.
"""
import argparse
import os
import sys

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.data import DataLoader, TensorDataset

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))   # run from a source checkout

try:
    import lightning.pytorch as pl
except ImportError:                                   # pragma: no cover
    try:
        import pytorch_lightning as pl
    except ImportError:
        print("lightning is not installed; nothing to run")
        sys.exit(0)

from opacus_b200 import PrivacyEngine  # noqa: E402
from opacus_b200.lightning import DPLightningDataModule  # noqa: E402
from opacus_b200.models import SmallCNN  # noqa: E402


class LitClassifier(pl.LightningModule):
    def __init__(self, sigma=1.0, clip=1.0):
        super().__init__()
        self.model, self.sigma, self.clip = SmallCNN(), sigma, clip
        self.engine = PrivacyEngine()

    def forward(self, x):
        return self.model(x)

    def training_step(self, batch, _):
        x, y = batch
        return F.cross_entropy(self(x), y)

    def configure_optimizers(self):
        opt = torch.optim.SGD(self.model.parameters(), lr=0.1)
        loader = self.trainer._data_connector._train_dataloader_source.dataloader()
        self.model, opt, _ = self.engine.make_private(module=self.model, optimizer=opt, data_loader=loader,
                                                      noise_multiplier=self.sigma, max_grad_norm=self.clip,
                                                      poisson_sampling=isinstance(loader, DataLoader))
        return opt

    def on_train_epoch_end(self):
        self.log("epsilon", self.engine.get_epsilon(1e-5))


class Digits(pl.LightningDataModule):
    def train_dataloader(self):
        g = torch.Generator().manual_seed(0)
        return DataLoader(TensorDataset(torch.randn(2048, 1, 28, 28, generator=g), torch.randint(0, 10, (2048,), generator=g)),
                          batch_size=256)


if __name__ == "__main__":
    pl.Trainer(max_epochs=1, enable_checkpointing=False, logger=False).fit(LitClassifier(), DPLightningDataModule(Digits()))
