"""PyTorch-Lightning adapter: a data module whose training loader is Poisson
sampled (``opacus/lightning.py:23-61``).  Importing this module requires
``pytorch_lightning`` (or ``lightning.pytorch``)."""
from typing import Any, Optional

import torch

try:
    import pytorch_lightning as pl
except ImportError:  # pragma: no cover
    try:
        import lightning.pytorch as pl
    except ImportError as e:  # pragma: no cover
        raise ImportError("opacus_b200.lightning needs pytorch_lightning (or lightning) installed") from e

from .data_loader import DPDataLoader


class DPLightningDataModule(pl.LightningDataModule):
    def __init__(self, datamodule: "pl.LightningDataModule", generator: Optional[torch.Generator] = None):
        super().__init__()
        self.datamodule = datamodule
        self.generator = generator

    def prepare_data(self) -> None:
        self.datamodule.prepare_data()

    def setup(self, stage: Optional[str] = None) -> None:
        self.datamodule.setup(stage)

    def train_dataloader(self):
        return DPDataLoader.from_data_loader(self.datamodule.train_dataloader(), distributed=False,
                                             generator=self.generator)

    def val_dataloader(self):
        return self.datamodule.val_dataloader()

    def test_dataloader(self):
        return self.datamodule.test_dataloader()

    def predict_dataloader(self):
        return self.datamodule.predict_dataloader()

    def transfer_batch_to_device(self, batch: Any, device: torch.device, dataloader_idx: int) -> Any:
        return self.datamodule.transfer_batch_to_device(batch, device, dataloader_idx)

    def on_before_batch_transfer(self, batch: Any, dataloader_idx: int) -> Any:
        return self.datamodule.on_before_batch_transfer(batch, dataloader_idx)

    def on_after_batch_transfer(self, batch: Any, dataloader_idx: int) -> Any:
        return self.datamodule.on_after_batch_transfer(batch, dataloader_idx)
