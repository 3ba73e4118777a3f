"""Base record for layer inputs / outputs: device moves and contiguity for all tensor fields."""

import torch


class BaseLayerIO:
    def to_(self, device: torch.device) -> None:
        for name, value in vars(self).items():
            if isinstance(value, torch.Tensor):
                setattr(self, name, value.to(device))

    def contiguous_(self) -> None:
        for name, value in vars(self).items():
            if isinstance(value, torch.Tensor):
                setattr(self, name, value.contiguous())
