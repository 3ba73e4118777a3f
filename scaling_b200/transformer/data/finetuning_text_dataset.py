"""Prompt / completion fine-tuning data (src/scaling/transformer/data/finetuning_text_dataset.py:29-399).

Sources: a JSON file with a list of ``{"prompt": str | [str | "x.jpg", ...], "completion": str}`` records, or a
memory map whose documents are ``[len(prompt), *prompt tokens, *completion tokens]`` (see ``convert_jsonl``).
Every item is one sequence of ``sequence_length`` tokens: soft-prompt placeholders, prompt, completion, padding with
the end-of-text token.  The loss covers the completion and the first end-of-text token only.
"""

from __future__ import annotations

import hashlib
import json
import random
from pathlib import Path
from typing import Any, Optional, Union

import numpy as np
import torch

from ...core.data import BaseDataset, MemoryMapDataset, MemoryMapDatasetBuilder
from ...core.data.blended_dataset import BaseBlendedDataset
from ...parallel.topology import Topology
from ..tokenizer import Tokenizer
from ._finetuning_common import (IMAGE_ENCODER_TOKEN_COUNTS, collate_items, image_transform, shift_locations,
                                 sync_text_image_batch)
from .dataset_item import TextImageDatasetItem
from .text_dataset_batch import TextDatasetBatch


def _vocab_digest(md5: Any, tokenizer: Tokenizer) -> None:
    md5.update(json.dumps(tokenizer.tokenizer.get_vocab(), sort_keys=True, default=str).encode("utf-8"))


class FinetuningTextDataset(BaseDataset[TextImageDatasetItem, TextDatasetBatch, TextDatasetBatch]):
    def __init__(self, data_prefix: Path, sequence_length: int, seed: int, softprompt_n_tokens: int,
                 tokenizer: Tokenizer, tokenizer_no_prefix_space: Tokenizer, memory_map_dataset: bool = False,
                 shuffle: bool = True):
        self.data_prefix = Path(data_prefix)
        self.data_prefix_parent = self.data_prefix.parent
        self.sequence_length = sequence_length
        self.softprompt_n_tokens = softprompt_n_tokens
        self.tokenizer = tokenizer
        self.tokenizer_no_prefix_space = tokenizer_no_prefix_space
        self.memory_map_dataset = memory_map_dataset
        self.dataset: Optional[MemoryMapDataset] = None
        if memory_map_dataset:
            self.dataset = MemoryMapDataset(prefix_path=self.data_prefix)
            self.data: list[Any] = list(range(len(self.dataset)))
        else:
            with open(self.data_prefix, "r", encoding="UTF-8") as f:
                self.data = json.load(f)
        self.seed: Optional[int] = None
        super().__init__(seed=seed, shuffle=shuffle)

    def ident(self) -> str:
        md5 = hashlib.md5()
        md5.update(str(self.data_prefix).encode("utf-8"))
        if not self.memory_map_dataset:  # token ids in a memory map do not depend on the tokenizers
            _vocab_digest(md5, self.tokenizer)
            _vocab_digest(md5, self.tokenizer_no_prefix_space)
        return f"{md5.hexdigest()}-seq-{self.sequence_length}"

    def set_seed(self, seed: int, shuffle: bool = True) -> None:
        if self.seed is not None and self.seed == seed:
            return
        if shuffle:
            random.Random(seed).shuffle(self.data)
        self.seed = seed

    def __len__(self) -> int:
        return len(self.data)

    # ------------------------------------------------------------------ item assembly
    def get_memory_map_token_ids(self, index: int) -> tuple[list[int], list[int]]:
        assert self.dataset is not None
        doc = self.dataset[self.data[index]].tolist()
        n = doc[0]
        return doc[1:n + 1], doc[n + 1:]

    def _encode_prompt_parts(self, parts: list[str]):
        tokens: list[int] = []
        images: list[torch.Tensor] = []
        locations: list[tuple[int, int]] = []
        for i, part in enumerate(parts):
            assert isinstance(part, str)
            is_image = False
            if part.endswith(".jpg"):
                try:
                    is_image = (self.data_prefix_parent / part).is_file()
                except OSError:  # a long text that merely ends in ".jpg" is not a usable path
                    is_image = False
            if is_image:
                from PIL import Image

                images.append(image_transform()(Image.open(str(self.data_prefix_parent / part))))
                locations.append((len(tokens), len(tokens) + IMAGE_ENCODER_TOKEN_COUNTS))
                tokens.extend([self.tokenizer.padding_token_id] * IMAGE_ENCODER_TOKEN_COUNTS)
            else:
                tok = self.tokenizer if i == 0 else self.tokenizer_no_prefix_space
                tokens.extend(tok.encode(part))
        return tokens, images, locations

    def get_json_token_ids(self, index: int):
        rec = self.data[index]
        images = locations = None
        if isinstance(rec["prompt"], list):
            prompt, images, locations = self._encode_prompt_parts(rec["prompt"])
        else:
            assert isinstance(rec["prompt"], str)
            prompt = self.tokenizer.encode(rec["prompt"])
        return prompt, self.tokenizer.encode(rec["completion"]), images, locations

    def __getitem__(self, index: int) -> TextImageDatasetItem:
        pad = self.tokenizer.padding_token_id
        images = locations = None
        if self.memory_map_dataset:
            prompt, completion = self.get_memory_map_token_ids(index)
        else:
            prompt, completion, images, locations = self.get_json_token_ids(index)
        if self.softprompt_n_tokens > 0:
            prompt = [0] * self.softprompt_n_tokens + prompt
            locations = shift_locations(locations, self.softprompt_n_tokens)
        S = self.sequence_length
        padding = S - len(prompt) - len(completion) + 1
        tokens = (prompt + completion + [pad] * max(padding, 0))[:S + 1]
        weights = torch.ones(S, dtype=torch.float)
        weights[:max(len(prompt) - 1, 0)] = 0
        # padding is the end-of-text token: the first one is a real target, the rest is not
        if padding - 1 > 0:
            weights[-(padding - 1):] = 0
        return TextImageDatasetItem(
            input_token_ids=torch.tensor(tokens[:-1], dtype=torch.long),
            target_token_ids=torch.tensor(tokens[1:], dtype=torch.long),
            cumulative_seq_lengths=torch.tensor([0, S], dtype=torch.int32), position_ids=torch.arange(0, S),
            loss_weights=weights, input_images=images, input_image_locations=locations,
        )

    def collate(self, batch: list[TextImageDatasetItem]) -> TextDatasetBatch:
        return collate_items(batch)

    @staticmethod
    def sync_batch_to_model_parallel(topology: Optional[Topology], batch: Optional[TextDatasetBatch]) -> TextDatasetBatch:
        return sync_text_image_batch(topology, batch)

    @staticmethod
    def convert_jsonl(jsonl_file: Union[str, Path], tokenizer: Tokenizer, tokenizer_no_prefix_space: Tokenizer,
                      out_prefix_path: Union[str, Path]) -> None:
        """``{"prompt": ..., "completion": ...}`` lines -> memory map of ``[len(prompt), *prompt, *completion]``."""
        builder = MemoryMapDatasetBuilder(prefix_path=Path(out_prefix_path))
        with open(jsonl_file, "r", encoding="UTF-8") as f:
            for line in f:
                line = line.strip()
                if not line:
                    continue
                rec = json.loads(line)
                prompt = tokenizer.encode(rec["prompt"])
                completion = tokenizer_no_prefix_space.encode(rec["completion"])
                builder.add(np_array=np.array([len(prompt)] + prompt + completion))
        builder.finalize()


class FinetuningTextBlendedDataset(BaseBlendedDataset[FinetuningTextDataset]):
    pass
