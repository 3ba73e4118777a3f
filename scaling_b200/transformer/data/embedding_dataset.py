"""Contrastive embedding data: query, one positive, hard negatives (src/scaling/transformer/data/embedding_dataset.py:25-515).

Sources: a jsonl file with ``{"query": str | [instruction, text], "positives": [..], "negatives": [..]}`` lines, or a
memory map written by ``jsonl_to_embedding_mmap`` (token stream of query | positive | negatives per record plus a
``.lengths.json`` side file with the piece lengths and instruction lengths).  An item is the stack
``[query, positive, negative_0, ...]`` of right-padded sequences; loss weights select the tokens that are pooled into
the embedding (0 on padding and, where instructions are used, on the instruction part).
"""

from __future__ import annotations

import hashlib
import json
import random
from pathlib import Path
from typing import Any, Optional, Union

import numpy as np
import torch

from ...core.data import BaseDataset, BaseDatasetItem, MemoryMapDataset, MemoryMapDatasetBuilder, broadcast_data
from ...core.data.blended_dataset import BaseBlendedDataset
from ...parallel.topology import Topology
from ..tokenizer import Tokenizer
from .text_dataset_batch import TextDatasetBatch
from .utils import get_cumulative_seq_lengths


class EmbeddingDatasetItem(BaseDatasetItem):
    def __init__(self, input_token_ids: torch.Tensor, position_ids: torch.Tensor, loss_weights: torch.Tensor):
        self.input_token_ids = input_token_ids
        self.loss_weights = loss_weights
        self.position_ids = position_ids


class EmbeddingMemoryMapDataset(MemoryMapDataset):
    """Token memory map plus per-record lengths (query, positive, negatives, instruction parts)."""

    @property
    def file_path_lengths(self) -> Path:
        return Path(str(self.prefix_path) + ".lengths.json")

    def initialize(self) -> None:
        super().initialize()
        with open(self.file_path_lengths, "r", encoding="UTF-8") as f:
            rec = json.load(f)
        self.query_length: list[int] = rec["query_length"]
        self.positive_length: list[int] = rec["positive_length"]
        self.negative_start_indices: list[list[int]] = rec["negative_lengths"]
        self.query_instruction_length: list[int] = rec.get("query_instruction_length", [])
        self.positive_instruction_length: list[int] = rec.get("positive_instruction_length", [])
        self.negative_instruction_length: list[list[int]] = rec.get("negative_instruction_length", [])


class EmbeddingDatasetMemoryMapDatasetBuilder(MemoryMapDatasetBuilder):
    def __init__(self, prefix_path: Path):
        super().__init__(prefix_path=prefix_path)
        self._lengths: dict[str, list] = {"query_length": [], "positive_length": [], "negative_lengths": [],
                                          "query_instruction_length": [], "positive_instruction_length": [],
                                          "negative_instruction_length": []}

    def add(self, query_token_ids: np.ndarray, positive_token_ids: np.ndarray,  # type: ignore[override]
            negative_token_ids: list[np.ndarray], query_instruction_length: Optional[int] = None,
            positive_instruction_length: Optional[int] = None,
            negative_instruction_length: Optional[list[int]] = None) -> None:
        pieces = [np.asarray(query_token_ids), np.asarray(positive_token_ids)] + [np.asarray(n) for n in negative_token_ids]
        super().add(np_array=np.concatenate(pieces))
        self._lengths["query_length"].append(int(pieces[0].size))
        self._lengths["positive_length"].append(int(pieces[1].size))
        self._lengths["negative_lengths"].append([int(p.size) for p in pieces[2:]])
        if query_instruction_length is not None:
            assert positive_instruction_length is not None and negative_instruction_length is not None
            self._lengths["query_instruction_length"].append(int(query_instruction_length))
            self._lengths["positive_instruction_length"].append(int(positive_instruction_length))
            self._lengths["negative_instruction_length"].append([int(x) for x in negative_instruction_length])

    def finalize(self) -> None:
        super().finalize()
        with open(str(self.prefix_path) + ".lengths.json", "w", encoding="UTF-8") as f:
            json.dump(self._lengths, f)


class EmbeddingDataset(BaseDataset[EmbeddingDatasetItem, TextDatasetBatch, TextDatasetBatch]):
    def __init__(self, data_path: Path, sequence_length: int, seed: int, tokenizer: Tokenizer,
                 number_of_hard_negatives: int, memory_map_dataset: bool = False, use_instruction: bool = True,
                 query_side_only: bool = False, shuffle: bool = True):
        if number_of_hard_negatives > 1:
            raise NotImplementedError("number_of_hard_negatives > 1 is not supported; choose 0 or 1")
        if query_side_only:
            assert use_instruction, "query_side_only needs use_instructions to be set as well"
        self.data_path = Path(data_path)
        self.sequence_length = sequence_length
        self.tokenizer = tokenizer
        self.memory_map_dataset = memory_map_dataset
        self.number_of_hard_negatives = number_of_hard_negatives
        self.use_instruction = use_instruction
        self.query_side_only = query_side_only
        if memory_map_dataset:
            self.mem_map_dataset = EmbeddingMemoryMapDataset(prefix_path=self.data_path)
            self.data = list(range(len(self.mem_map_dataset)))
        else:
            with open(self.data_path, "r", encoding="UTF-8") as f:
                self.data_jsonl = [json.loads(line) for line in f.read().split("\n") if line != ""]
            self.load_dataset_from_jsonl()
            self.data = list(range(len(self.jsonl_dataset)))
        self.seed: Optional[int] = None
        super().__init__(seed=seed, shuffle=shuffle)

    # ------------------------------------------------------------------ loading
    @staticmethod
    def encode_sample(data_item: dict, tokenizer: Tokenizer) -> dict[str, Any]:
        """Token ids of query / first positive / negatives; with ``[instruction, text]`` pairs also the token count
        of each instruction."""
        if isinstance(data_item["query"], (tuple, list)):
            def pair(p):
                return tokenizer.encode(p[0] + " " + p[1]), len(tokenizer.encode(p[0]))

            q, ql = pair(data_item["query"])
            pos, pl = pair(data_item["positives"][0])
            negs = [pair(n) for n in data_item["negatives"]]
            return {"query_token_ids": q, "positive_token_ids": pos, "negative_token_ids": [n[0] for n in negs],
                    "query_instruction_length": ql, "positive_instruction_length": pl,
                    "negative_instruction_length": [n[1] for n in negs]}
        return {"query_token_ids": tokenizer.encode(data_item["query"]),
                "positive_token_ids": tokenizer.encode(data_item["positives"][0]),
                "negative_token_ids": [tokenizer.encode(n) for n in data_item["negatives"]],
                "query_instruction_length": None, "positive_instruction_length": None,
                "negative_instruction_length": None}

    def _is_valid_sample(self, s: dict[str, Any]) -> bool:
        if len(s["query_token_ids"]) == 0 or len(s["positive_token_ids"]) == 0:
            return False
        if any(len(n) == 0 for n in s["negative_token_ids"]):
            return False
        if not self.use_instruction:
            return True
        assert s["query_instruction_length"] is not None, "use_instruction needs [instruction, text] records"
        if s["query_instruction_length"] >= self.sequence_length:
            return False
        if self.query_side_only:
            return True
        if s["positive_instruction_length"] >= self.sequence_length:
            return False
        return not any(n >= self.sequence_length for n in s["negative_instruction_length"])

    def load_dataset_from_jsonl(self) -> None:
        self.jsonl_dataset = []
        for rec in self.data_jsonl:
            enc = EmbeddingDataset.encode_sample(rec, self.tokenizer)
            if self._is_valid_sample(enc):
                self.jsonl_dataset.append(enc)

    @staticmethod
    def jsonl_to_embedding_mmap(jsonl_file: Union[str, Path], tokenizer: Tokenizer,
                                out_prefix_path: Union[str, Path]) -> None:
        builder = EmbeddingDatasetMemoryMapDatasetBuilder(prefix_path=Path(out_prefix_path))
        with open(jsonl_file, "r", encoding="UTF-8") as f:
            for line in f:
                if line.strip() == "":
                    continue
                rec = json.loads(line)
                assert len(rec["positives"]) == 1 and len(rec["negatives"]) > 0
                enc = EmbeddingDataset.encode_sample(rec, tokenizer)
                builder.add(query_token_ids=np.array(enc["query_token_ids"]),
                            positive_token_ids=np.array(enc["positive_token_ids"]),
                            negative_token_ids=[np.array(n) for n in enc["negative_token_ids"]],
                            query_instruction_length=enc["query_instruction_length"],
                            positive_instruction_length=enc["positive_instruction_length"],
                            negative_instruction_length=enc["negative_instruction_length"])
        builder.finalize()
        with open(str(out_prefix_path) + ".done", "w") as f:
            f.write("True")

    # ------------------------------------------------------------------ dataset protocol
    def ident(self) -> str:
        md5 = hashlib.md5()
        md5.update(str(self.data_path).encode("utf-8"))
        md5.update(json.dumps(self.tokenizer.tokenizer.get_vocab(), sort_keys=True, default=str).encode("utf-8"))
        return f"{md5.hexdigest()}-seq-{self.sequence_length}"

    def set_seed(self, seed: int, shuffle: bool = True) -> None:
        if self.seed is not None and self.seed == seed:
            return
        if shuffle:
            random.Random(seed).shuffle(self.data)
        self.seed = seed

    def __len__(self) -> int:
        return len(self.data)

    def _record(self, index: int):
        src = self.data[index]
        if not self.memory_map_dataset:
            s = self.jsonl_dataset[src]
            return (s["query_token_ids"], s["positive_token_ids"], s["negative_token_ids"],
                    s["query_instruction_length"], s["positive_instruction_length"], s["negative_instruction_length"])
        mm = self.mem_map_dataset
        tokens = mm[src].tolist()
        ql, pl = mm.query_length[src], mm.positive_length[src]
        negs, off = [], ql + pl
        for n in mm.negative_start_indices[src]:
            negs.append(tokens[off:off + n])
            off += n
        qi = pi = ni = None
        if len(mm.query_instruction_length):
            qi, pi, ni = (mm.query_instruction_length[src], mm.positive_instruction_length[src],
                          mm.negative_instruction_length[src])
        return tokens[:ql], tokens[ql:ql + pl], negs, qi, pi, ni

    def __getitem__(self, index: int) -> EmbeddingDatasetItem:
        query, positive, negatives, qi, pi, ni = self._record(index)
        S = self.sequence_length
        if self.use_instruction:
            assert qi is not None, "use_instruction was set to true but the data has no instruction lengths"
            if not self.query_side_only:
                assert pi is not None and ni is not None
        # drop instruction prefixes that are not wanted on a side
        if not self.use_instruction:
            if qi is not None:
                query = query[qi:]
        if not self.use_instruction or self.query_side_only:
            if pi is not None:
                positive = positive[pi:]
            if ni is not None:
                negatives = [n[k:] for n, k in zip(negatives, ni)]
        assert len(negatives) >= self.number_of_hard_negatives, (
            "Selected number of hard negatives was smaller than the available negative samples for item"
        )

        def prepare(tokens: list[int], instruction: Optional[int], is_query: bool = False):
            tokens = tokens[:S]
            pad = S - len(tokens)
            ids = torch.tensor(tokens + [self.tokenizer.padding_token_id] * pad)
            w = torch.ones(S, dtype=torch.float)
            if instruction is not None and self.use_instruction and (is_query or not self.query_side_only):
                w[:instruction] = 0
            if pad > 0:
                w[-pad:] = 0
            return ids, w

        rows = [prepare(query, qi, True), prepare(positive, pi)]
        for i, n in enumerate(negatives[:self.number_of_hard_negatives]):
            rows.append(prepare(n, ni[i] if ni is not None else None))
        ids = torch.stack([r[0] for r in rows])
        return EmbeddingDatasetItem(input_token_ids=ids, position_ids=torch.arange(0, S).repeat(len(rows), 1),
                                    loss_weights=torch.stack([r[1] for r in rows]))

    def collate(self, batch: list[EmbeddingDatasetItem]) -> TextDatasetBatch:
        ids = torch.cat([b.input_token_ids for b in batch], dim=0)
        return TextDatasetBatch(
            input_token_ids=ids, position_ids=torch.cat([b.position_ids for b in batch], dim=0),
            cumulative_seq_lengths=get_cumulative_seq_lengths(ids, reset_attention_mask=False),
            loss_weights=torch.cat([b.loss_weights for b in batch], dim=0),
        )

    @staticmethod
    def sync_batch_to_model_parallel(topology: Optional[Topology] = None,
                                     batch: Optional[TextDatasetBatch] = None) -> TextDatasetBatch:
        if topology is None:
            assert batch is not None
            return batch
        if topology.model_parallel_rank == 0:
            assert batch is not None
            batch.contiguous_()
            assert batch.cumulative_seq_lengths_padded is not None
            longs = [batch.input_token_ids, batch.cumulative_seq_lengths_padded.to(torch.long), batch.position_ids]
            floats = [batch.loss_weights]
        else:
            assert batch is None
            longs, floats = [None, None, None], [None]
        lt = broadcast_data(tensors=longs, dtype=torch.long, topology=topology)
        ft = broadcast_data(tensors=floats, dtype=torch.float32, topology=topology)
        return TextDatasetBatch(input_token_ids=lt[0], cumulative_seq_lengths_padded=lt[1].to(torch.int32),
                                position_ids=lt[2], loss_weights=ft[0])


class EmbeddingBlendedDataset(BaseBlendedDataset[EmbeddingDataset]):
    pass
