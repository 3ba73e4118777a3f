"""Chat fine-tuning data (src/scaling/transformer/data/finetuning_chat_dataset.py:27-353).

A jsonl file; every line is one conversation as a list of ``{"type": "text" | "image", "content": ..., "has_loss":
bool}`` elements.  Text elements are tokenised (the first one with the regular tokenizer, later ones without a
leading space) and contribute to the loss where ``has_loss`` is set; image elements reserve 144 placeholder tokens.
"""

from __future__ import annotations

import hashlib
import json
import random
from pathlib import Path
from typing import Any, Optional

import torch

from ...core.data import BaseDataset
from ...core.data.blended_dataset import BaseBlendedDataset
from ...parallel.topology import Topology
from ..tokenizer import Tokenizer
from ._finetuning_common import (IMAGE_ENCODER_TOKEN_COUNTS, collate_items, image_transform, shift_locations,
                                 sync_text_image_batch)
from .dataset_item import TextImageDatasetItem
from .text_dataset_batch import TextDatasetBatch


class FinetuningChatDataset(BaseDataset[TextImageDatasetItem, TextDatasetBatch, TextDatasetBatch]):
    def __init__(self, data_path: Path, sequence_length: int, seed: int, softprompt_n_tokens: int,
                 tokenizer: Tokenizer, tokenizer_no_prefix_space: Tokenizer, shuffle: bool = True):
        self.data_path = Path(data_path)
        self.data_path_parent = self.data_path.parent
        self.sequence_length = sequence_length
        self.softprompt_n_tokens = softprompt_n_tokens
        self.tokenizer = tokenizer
        self.tokenizer_no_prefix_space = tokenizer_no_prefix_space
        with open(self.data_path, "r", encoding="UTF-8") as f:
            self.data_jsonl = [json.loads(line) for line in f if line.strip()]
        self.data: list[dict[str, Any]] = []
        self.load_data()
        self.seed: Optional[int] = None
        super().__init__(seed=seed, shuffle=shuffle)

    def load_data(self) -> None:
        """Tokenise every conversation once; items are cut to length in ``__getitem__``."""
        for conversation in self.data_jsonl:
            tokens: list[int] = []
            mask: list[int] = []
            image_paths: Optional[list[Path]] = None
            locations: Optional[list[tuple[int, int]]] = None
            first_text = True
            for element in conversation:
                kind, content = element["type"], element["content"]
                if kind == "text":
                    tok = self.tokenizer if first_text else self.tokenizer_no_prefix_space
                    ids = tok.encode(content)
                    tokens.extend(ids)
                    mask.extend([int(element.get("has_loss", False))] * len(ids))
                    first_text = False
                elif kind == "image":
                    image_paths = image_paths if image_paths is not None else []
                    locations = locations if locations is not None else []
                    image_paths.append(Path(content))
                    locations.append((len(tokens), len(tokens) + IMAGE_ENCODER_TOKEN_COUNTS))
                    tokens.extend([self.tokenizer.padding_token_id] * IMAGE_ENCODER_TOKEN_COUNTS)
                    mask.extend([0] * IMAGE_ENCODER_TOKEN_COUNTS)
                else:
                    raise NotImplementedError(f"Content type {kind} is not supported")
            self.data.append({"input_token_list": tokens[:-1], "target_token_list": tokens[1:],
                              "loss_mask_list": mask[1:], "prompt_images_path": image_paths,
                              "prompt_image_locations": locations})

    def ident(self) -> str:
        md5 = hashlib.md5()
        md5.update(str(self.data_path).encode("utf-8"))
        for tok in (self.tokenizer, self.tokenizer_no_prefix_space):
            md5.update(json.dumps(tok.tokenizer.get_vocab(), sort_keys=True, default=str).encode("utf-8"))
        return f"{md5.hexdigest()}-seq-{self.sequence_length}"

    def set_seed(self, seed: int, shuffle: bool = True) -> None:
        if self.seed is not None and self.seed == seed:
            return
        if shuffle:
            random.Random(seed).shuffle(self.data)
        self.seed = seed

    def __len__(self) -> int:
        return len(self.data)

    def __getitem__(self, index: int) -> TextImageDatasetItem:
        rec = self.data[index]
        S, pad, n_soft = self.sequence_length, self.tokenizer.padding_token_id, self.softprompt_n_tokens
        inputs = [0] * n_soft + rec["input_token_list"]
        targets = [0] * n_soft + rec["target_token_list"]
        mask = [0] * n_soft + rec["loss_mask_list"]
        locations = shift_locations(rec["prompt_image_locations"], n_soft)
        fill = max(S - len(inputs), 0)
        inputs = (inputs + [pad] * fill)[:S]
        targets = (targets + [pad] * fill)[:S]
        mask = (mask + [0] * fill)[:S]
        images = None
        if rec["prompt_images_path"] is not None:
            from PIL import Image

            images = [image_transform()(Image.open(str(self.data_path_parent / p))) for p in rec["prompt_images_path"]]
        return TextImageDatasetItem(
            input_token_ids=torch.tensor(inputs, dtype=torch.long), target_token_ids=torch.tensor(targets, dtype=torch.long),
            cumulative_seq_lengths=torch.tensor([0, S], dtype=torch.int32), position_ids=torch.arange(0, S),
            loss_weights=torch.tensor(mask, dtype=torch.float32), input_images=images, input_image_locations=locations,
        )

    def collate(self, batch: list[TextImageDatasetItem]) -> TextDatasetBatch:
        return collate_items(batch)

    @staticmethod
    def sync_batch_to_model_parallel(topology: Optional[Topology], batch: Optional[TextDatasetBatch]) -> TextDatasetBatch:
        return sync_text_image_batch(topology, batch)


class FinetuningChatBlendedDataset(BaseBlendedDataset[FinetuningChatDataset]):
    pass
