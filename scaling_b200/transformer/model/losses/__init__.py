from __future__ import annotations

from typing import Any, Union

from ...context.config import (
    BaseLossFunctionConfig,
    ContrastiveLossFunctionConfig,
    CrossEntropyLossFunctionConfig,
    LossFunctionType,
)
from .contrastive import ContrastiveLoss
from .cross_entropy import CrossEntropyLoss, vocab_parallel_cross_entropy


def create_loss_function(context: Any, loss_function_config: BaseLossFunctionConfig) -> Union[ContrastiveLoss, CrossEntropyLoss]:
    if loss_function_config.loss_type == LossFunctionType.CONTRASTIVE_LOSS:
        assert isinstance(loss_function_config, ContrastiveLossFunctionConfig), (
            "Provide ContrastiveLossFunctionConfig when selecting contrastive_loss"
        )
        return ContrastiveLoss(topology=context.topology, loss_config=loss_function_config)
    if loss_function_config.loss_type == LossFunctionType.CROSS_ENTROPY_LOSS:
        assert isinstance(loss_function_config, CrossEntropyLossFunctionConfig), (
            "Provide CrossEntropyLossFunctionConfig when selecting cross_entropy_loss"
        )
        arch = context.config.transformer_architecture
        return CrossEntropyLoss(loss_config=loss_function_config, umup_config=arch.umup, topology=context.topology,
                                vocab_size=arch.vocab_size)
    raise ValueError(f"Unknown loss function type: {loss_function_config.loss_type}")


__all__ = ["ContrastiveLoss", "CrossEntropyLoss", "create_loss_function", "vocab_parallel_cross_entropy"]
