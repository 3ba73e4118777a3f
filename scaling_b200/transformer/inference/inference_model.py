"""Single-process inference over a trained transformer (src/scaling/transformer/inference/inference_model.py:24-373).

``TransformerInferenceModule`` instantiates the layer specs of an architecture on a list of devices (a pipeline
inside one process), loads a layout-independent checkpoint and offers ``logits``, ``generate`` (greedy or sampled,
with or without the KV cache), hidden-state recording and sentence embeddings (``encode``).
"""

from __future__ import annotations

from pathlib import Path
from typing import Any, Callable, Optional, Sequence, Union

import numpy as np
import torch
import yaml

from ...core.data import BaseLayerIO
from ...core.nn.parallel_module import LayerSpec
from ...core.nn.parallel_module.inference_module import InferenceModule, RecorderSetting
from ...parallel.topology_config import PipePartitionMethod
from ..context.config import TransformerArchitectureConfig
from ..data.inference_settings import InferenceSettings
from ..data.text_dataset_batch import TextDatasetBatch
from ..model.layers.base import TransformerLayerIO
from ..model.model import get_transformer_layer_specs
from ..tokenizer import Tokenizer
from .sample import sample_argmax

_FP8_KEYS = ("fp8_config_attention", "fp8_config_attention_dense_out", "fp8_config_mlp", "fp8_config_mlp_dense_out",
             "fp8_config_lm_head")


class CompletionOutput:
    def __init__(self, completion_text: Optional[str], completion_tokens: list[int], completion_logits: torch.Tensor):
        self.completion_text = completion_text
        self.completion_tokens = completion_tokens
        self.completion_logits = completion_logits


class TransformerInferenceModule(InferenceModule):
    def __init__(self, layer_specs: list[LayerSpec], devices: Sequence[Union[int, str, torch.device]] = (0,),
                 pipe_partition_method: PipePartitionMethod = PipePartitionMethod.UNIFORM,
                 pipe_partition_overwrite: Optional[list[int]] = None, tokenizer: Optional[Tokenizer] = None):
        super().__init__(layer_specs=layer_specs, devices=devices, pipe_partition_method=pipe_partition_method,
                         pipe_partition_overwrite=pipe_partition_overwrite)
        self.tokenizer = tokenizer

    # ------------------------------------------------------------------ construction
    @staticmethod
    def _parse_config_file(config_file: Path, use_flash_attention: bool) -> TransformerArchitectureConfig:
        with open(config_file, "r") as f:
            config = yaml.safe_load(f)
        arch = config["transformer_architecture"]
        arch.setdefault("masked_softmax", {})["kernel"] = "flash_attention" if use_flash_attention else "torch"
        for key in _FP8_KEYS:  # checkpoints of fp8-trained models are loaded into fp8 storage
            if arch.get(key) is not None:
                arch[key]["load_in_fp8"] = True
        return TransformerArchitectureConfig.from_dict(arch)

    @classmethod
    def from_checkpoint(cls, checkpoint_dir: Union[Path, str],
                        devices: Sequence[Union[int, str, torch.device]] = (0,),
                        pipe_partition_method: PipePartitionMethod = PipePartitionMethod.UNIFORM,
                        pipe_partition_overwrite: Optional[list[int]] = None, config_file: Optional[Path] = None,
                        vocab_file: Optional[Path] = None,
                        use_flash_attention: bool = False) -> "TransformerInferenceModule":
        """``checkpoint_dir`` holds the per-layer weight files and, unless given explicitly, ``config.yml`` and
        ``vocab.json``."""
        checkpoint_dir = Path(checkpoint_dir)
        config_file = Path(config_file) if config_file is not None else checkpoint_dir / "config.yml"
        vocab_file = Path(vocab_file) if vocab_file is not None else checkpoint_dir / "vocab.json"
        assert config_file.is_file(), "Config file not found"
        assert vocab_file.is_file(), "Vocab file not found"
        arch = cls._parse_config_file(config_file, use_flash_attention)
        model = cls(layer_specs=get_transformer_layer_specs(architecture_config=arch), devices=devices,
                    pipe_partition_method=pipe_partition_method, pipe_partition_overwrite=pipe_partition_overwrite,
                    tokenizer=Tokenizer.from_file(str(vocab_file)))
        if arch.umup.enable:
            # the batch size only shapes backward multipliers, so 1 is as good as any value here
            model.umup_setup(effective_batch_size=1, depth=arch.num_layers, avg_sequence_length=arch.sequence_length)
        model.load_checkpoint(checkpoint_dir)
        return model

    # ------------------------------------------------------------------ forward helpers
    def forward(self, x: BaseLayerIO) -> TransformerLayerIO:  # type: ignore[override]
        out = super().forward(x)
        assert isinstance(out, TransformerLayerIO)
        return out

    def _tokens(self, input_text: Optional[str], input_tokens: Optional[list[int]]) -> list[int]:
        assert (input_text is None) ^ (input_tokens is None), "Either input_text or input_tokens needs to be provided"
        if input_text is not None:
            assert self.tokenizer is not None
            return self.tokenizer.encode(input_text)
        assert input_tokens is not None
        return list(input_tokens)

    def _pre_process_input(self, input_text: Optional[str] = None, input_tokens: Optional[list[int]] = None,
                           process_for_cached_inference: bool = True) -> TextDatasetBatch:
        ids = torch.tensor(self._tokens(input_text, input_tokens), dtype=torch.long).unsqueeze(0)
        settings = InferenceSettings(use_cache=process_for_cached_inference, reset_cache=True, cache_index=0,
                                     embedding_layers=[-1])
        return TextDatasetBatch(input_token_ids=ids, inference_settings=settings)

    @staticmethod
    def _post_process_output(output: TransformerLayerIO) -> torch.Tensor:
        return output.activations.squeeze()

    # ------------------------------------------------------------------ logits
    def logits(self, input_text: Optional[str] = None, input_tokens: Optional[list[int]] = None) -> torch.Tensor:
        """Final activations (normally the logits ``[seq, vocab]``) for a prompt."""
        return self._post_process_output(self.forward(self._pre_process_input(input_text, input_tokens))).squeeze()

    def logits_with_hidden_state_recorder(
        self, input_text: Optional[str] = None, input_tokens: Optional[list[int]] = None,
        recorder_settings_per_layer: Optional[dict[int, RecorderSetting]] = None,
    ) -> tuple[torch.Tensor, dict[int, dict[str, Any]]]:
        batch = self._pre_process_input(input_text, input_tokens)
        out, record = super().forward_with_hidden_state_recorder(
            batch, recorder_settings_per_layer=recorder_settings_per_layer)
        assert isinstance(out, TransformerLayerIO)
        return self._post_process_output(out), record

    # ------------------------------------------------------------------ generation
    def generate(self, max_tokens: int, input_text: Optional[str] = None, input_tokens: Optional[list[int]] = None,
                 sample_fn: Callable[[torch.Tensor], torch.Tensor] = sample_argmax,
                 stop_tokens: Optional[Sequence[int]] = None, use_cache: bool = True) -> CompletionOutput:
        """Complete a prompt token by token until ``max_tokens`` or a stop token (default: end of text).

        With the cache, the prompt is run once and every later step feeds one token with its position; without
        it the whole sequence is re-run every step.  ``completion_logits`` holds one row per generated token.
        """
        if stop_tokens is None:
            assert self.tokenizer is not None, "If no tokenizer is provided, a stop token needs to be set manually"
            stop_tokens = [self.tokenizer.eos_token_id]
        stops = set(int(t) for t in stop_tokens)
        batch = self._pre_process_input(input_text, input_tokens, process_for_cached_inference=use_cache)
        assert batch.input_token_ids is not None
        prompt_len = batch.input_token_ids.shape[-1]
        step_settings = InferenceSettings(use_cache=use_cache, reset_cache=not use_cache, cache_index=0,
                                          embedding_layers=[-1])
        tokens: list[int] = []
        per_step_logits: list[torch.Tensor] = []
        output: Optional[TransformerLayerIO] = None
        for k in range(max_tokens):
            output = self.forward(batch)
            nxt = sample_fn(output.activations)
            token = int(nxt.item())
            tokens.append(token)
            if use_cache:
                per_step_logits.append(output.activations[:, -1, :])
                batch = TextDatasetBatch(input_token_ids=nxt.reshape(1, 1).cpu(), inference_settings=step_settings,
                                         position_ids=torch.tensor([[prompt_len + k]]))
            else:
                assert batch.input_token_ids is not None
                ids = torch.cat((batch.input_token_ids.cpu(), nxt.reshape(1, 1).cpu()), dim=-1)
                batch = TextDatasetBatch(input_token_ids=ids, inference_settings=step_settings)
            if token in stops:
                break
        if use_cache:
            logits = torch.cat(per_step_logits) if per_step_logits else torch.empty(0)
        else:
            logits = self._post_process_output(output)[prompt_len - 1:] if output is not None else torch.empty(0)
        text = self.tokenizer.decode(tokens) if self.tokenizer is not None else None
        return CompletionOutput(completion_text=text, completion_tokens=tokens, completion_logits=logits)

    # ------------------------------------------------------------------ embeddings
    def _embedding_batch(self, rows: list[list[int]], instruction_length: int, pad_token_id: int) -> TextDatasetBatch:
        """Right-padded batch whose ``loss_weights`` select the tokens to pool: 0 on instruction and padding."""
        width = max(len(r) for r in rows)
        device = self._layer_devices[0]
        ids = torch.full((len(rows), width), pad_token_id, dtype=torch.int32)
        weights = torch.zeros((len(rows), width), dtype=torch.int32)
        for i, r in enumerate(rows):
            ids[i, :len(r)] = torch.tensor(r, dtype=torch.int32)
            weights[i, instruction_length:len(r)] = 1
        pos = torch.arange(width).unsqueeze(0).expand(len(rows), width).contiguous()
        return TextDatasetBatch(input_token_ids=ids.to(device), loss_weights=weights.to(device),
                                position_ids=pos.to(device))

    def encode(self, sentences: Union[list[str], str], batch_size: int = 256, max_length: int = 512,
               instruction: str = "", convert_to_tensor: bool = False,
               user_token: str = "<|start_header_id|>user<|end_header_id|>", embed_token: str = "\n<|embed|>\n",
               pad_token: str = "<|padding|>", **_: Any) -> Union[torch.Tensor, np.ndarray]:
        """Sentence embeddings from a model with an embedding head; prompt = user token + instruction + embed
        token + sentence, truncated to ``max_length`` tokens."""
        if isinstance(sentences, str):
            sentences = [sentences]
        assert self.tokenizer, "Tokenizer need to be set to encode embeddings"
        pad = self.tokenizer.encode(pad_token)
        assert len(pad) == 1, "pad_token was tokenized to more than one token."
        prefix = user_token + instruction + embed_token
        prefix_len = len(self.tokenizer.encode(prefix))
        chunks: list[Any] = []
        for start in range(0, len(sentences), batch_size):
            rows = [self.tokenizer.encode(prefix + s)[:max_length] for s in sentences[start:start + batch_size]]
            emb = self.forward(self._embedding_batch(rows, prefix_len, pad[0])).activations
            chunks.append(emb if convert_to_tensor else emb.float().cpu().numpy())
        if convert_to_tensor:
            return torch.cat(chunks, dim=0).cpu()
        return np.concatenate(chunks, axis=0)

    def encode_corpus(self, corpus: Union[list[str], str, list[dict[str, str]]], **kwargs: Any):
        if isinstance(corpus, list) and corpus and isinstance(corpus[0], dict):
            corpus = [(d["title"] + " " + d["text"]) if "title" in d else d["text"] for d in corpus]  # type: ignore[index]
        return self.encode(corpus, **kwargs)  # type: ignore[arg-type]

    def encode_queries(self, queries: Union[list[str], str], **kwargs: Any):
        return self.encode(queries, **kwargs)
