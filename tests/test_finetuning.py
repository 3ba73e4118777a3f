"""Parameter-efficient fine-tuning through the config (BitFit biases, adapters, soft prompt, LoRA merge): only the new
parameters train, they go to their own checkpoint files, and a base checkpoint without them loads non-strictly."""

import copy
from pathlib import Path

import pytest
import torch

from tests.test_transformer_training import losses, tiny_config
from tests.utils import dist_launcher

pytestmark = pytest.mark.dist

FINETUNE_ARCH = {
    "bitfit_bias_config": {"name": "ft"},
    "adapter_config": {"name": "ad", "attention_downsampling_factor": 0.25, "mlp_downsampling_factor": 0.25},
    "softprompt_config": {"name": "sp", "n_tokens": 4},
}
GROUPS = [{"group_name": "new", "parameters_include": ["bias_ft", "adapter_ad", "softprompt_sp"], "weight_decay": 0.0,
           "learning_rate_scheduler": {"learning_rate": 1e-2, "learning_rate_decay_style": "constant"}}]


def _finetune(rank, world_size, port, device, config):
    from scaling_b200.core.runner import LaunchConfig
    from scaling_b200.parallel import Topology
    from scaling_b200.transformer import TransformerConfig, TransformerContext, init_model, init_optimizer
    from scaling_b200.transformer.model import metrics_aggregation_fn
    from scaling_b200.transformer.model.losses import create_loss_function
    from scaling_b200.transformer.train import TransformerTrainer, _get_sync_batch, _read_datasets

    lc = LaunchConfig(master_port=port, master_addr="127.0.0.1", world_size=world_size, global_rank=rank,
                      local_slot=rank, payload=copy.deepcopy(config))
    cfg = TransformerConfig.from_dict(lc.overwrite_config_dict_with_launcher_args(dict(lc.payload)))
    topology = Topology(cfg.topology)
    context = TransformerContext(config=cfg, topology=topology)
    context.initialize(master_addr="127.0.0.1", master_port=str(port), seed=cfg.trainer.seed)
    model = init_model(context)
    optimizer = init_optimizer(context, model)
    dataset = _read_datasets(cfg)[0] if topology.is_io_rank else None
    trainer = TransformerTrainer(config=cfg.trainer, context=context, parallel_module=model, optimizer=optimizer,
                                 dataset=dataset, sync_batch_to_model_parallel=_get_sync_batch(cfg.data),
                                 loss_function=create_loss_function(context, cfg.training.loss_function_config),
                                 metrics_aggregation_fn=metrics_aggregation_fn)
    before = {n: p.detach().clone() for n, p in model.named_parameters()}
    metrics = trainer.run_training(return_metrics=True)
    changed = sorted(n for n, p in model.named_parameters() if not torch.equal(p.detach(), before[n]))
    frozen = sorted(n for n, p in model.named_parameters() if torch.equal(p.detach(), before[n]))
    return ([m["training/loss"] for m in metrics] if metrics else None, changed, frozen,
            cfg.trainer.separate_file_for_parameters)


def _is_new(name: str) -> bool:
    return any(tag in name for tag in ("bias_ft", "adapter_ad", "softprompt_sp"))


@pytest.mark.parametrize("world_size,mp", [(1, 1), (2, 2)])
def test_bitfit_adapter_softprompt_train_alone_and_get_their_own_files(tmp_path: Path, world_size, mp):
    base_dir = str(tmp_path / "base")
    losses(1, save_dir=base_dir, save_interval=2, iters=2)  # a plain pretrained checkpoint without the new parameters
    cfg = tiny_config(world_size, mp=mp, arch=FINETUNE_ARCH, groups=GROUPS, iters=3, load_dir=base_dir,
                      save_dir=str(tmp_path / "ft"), save_interval=3,
                      training={"allow_missing_params_in_optimizer": True})
    # with a named bias set the layers carry `bias_ft` in place of `bias`: the pretrained biases stay in the file
    cfg["trainer"].update(allowed_missing_keys_in_checkpoint=["bias_ft", "adapter_ad", "softprompt_sp"],
                          allowed_unexpected_keys_in_checkpoint=[r"\.bias$"],
                          load_optimizer_states=False, load_context=False)
    out = dist_launcher(_finetune, world_size, config=cfg)
    loss, changed, frozen, separate = out[0]
    assert sorted(separate) == ["adapter_ad", "bias_ft", "softprompt_sp"]
    assert changed and all(_is_new(n) for n in changed), changed
    assert frozen and not any(_is_new(n) for n in frozen), [n for n in frozen if _is_new(n)]
    assert all(l == l for l in loss)
    files = sorted(f.name for f in (tmp_path / "ft" / "global_step3").glob("model_state_layer_*.pt"))
    for tag in ("bias_ft", "adapter_ad", "softprompt_sp"):
        assert any(f.endswith(f"_{tag}.pt") for f in files), (tag, files)
    # the base files hold none of the new parameters, the separate files nothing else
    for f in (tmp_path / "ft" / "global_step3").glob("model_state_layer_*.pt"):
        keys = list(torch.load(f, map_location="cpu", weights_only=False).keys())
        separate_file = any(f.name.endswith(f"_{tag}.pt") for tag in ("bias_ft", "adapter_ad", "softprompt_sp"))
        assert all(_is_new(k) == separate_file for k in keys), (f.name, keys)


def test_base_checkpoint_without_the_new_parameters_needs_the_allowance(tmp_path: Path):
    base_dir = str(tmp_path / "base")
    losses(1, save_dir=base_dir, save_interval=2, iters=2)
    cfg = tiny_config(1, arch=FINETUNE_ARCH, groups=GROUPS, iters=1, load_dir=base_dir,
                      training={"allow_missing_params_in_optimizer": True})
    cfg["trainer"].update(load_optimizer_states=False, load_context=False,
                          allowed_unexpected_keys_in_checkpoint=[r"\.bias$"])
    with pytest.raises(AssertionError, match="(?i)missing|bias_ft|adapter_ad|softprompt"):
        dist_launcher(_finetune, 1, config=cfg)


# ---------------------------------------------------------------------------------------------- embeddings
def _embedding_setup(tmp_path: Path) -> tuple[str, str]:
    import json

    from scaling_b200.transformer.tokenizer import Tokenizer

    words = ["the", "cat", "sat", "on", "mat", "a", "dog", "ran", "far", "query", "doc", "good", "bad", "find", ":"]
    tok = Tokenizer.from_words(words)
    vocab = tmp_path / "vocab.json"
    vocab.write_text(tok.tokenizer.to_str())
    records = []
    for i in range(32):
        a, b, c = words[i % 9], words[(i + 3) % 9], words[(i + 5) % 9]
        records.append({"query": ["find :", f"{a} {b}"], "positives": [["doc :", f"the {a} {b} {c}"]],
                        "negatives": [["doc :", f"a {c} ran far"]]})
    data = tmp_path / "emb.jsonl"
    data.write_text("\n".join(json.dumps(r) for r in records) + "\n")
    return str(vocab), str(data)


@pytest.mark.parametrize("world_size", [1, 2])
def test_embedding_head_trains_with_the_contrastive_loss(tmp_path: Path, world_size):
    """Query / positive / hard-negative triples, pooled embedding head, in-batch negatives gathered over the
    data-parallel ranks; the language-model head is left out."""
    vocab, data = _embedding_setup(tmp_path)
    arch = {"vocab_size": 32, "vocab_file": vocab, "lm_head": False, "sequence_length": 12, "causal": True,
            "embedding_head_config": {"name": "emb", "proj_layers": [16], "pooling": "weighted_mean"}}
    training = {"loss_function_config": {"loss_type": "contrastive_loss", "number_of_hard_negatives": 1,
                                         "use_instructions": True}}
    cfg = tiny_config(world_size, arch=arch, iters=4, micro=4, training=training)
    cfg["data"] = {"embedding_dataset": True, "data_prefixes": [data]}
    out = dist_launcher(_finetune, world_size, config=cfg)
    loss, changed, _, _ = out[0]
    assert len(loss) == 4 and all(l == l and l > 0 for l in loss)
    assert any("embedding_head" in n or "emb" in n for n in changed)
    assert not any("lm_head" in n for n in changed)


# ---------------------------------------------------------------------------------------------- instruction / chat data
@pytest.mark.parametrize("kind,world_size,mp", [("finetuning_dataset", 1, 1), ("finetuning_chat_dataset", 2, 2)])
def test_prompt_completion_and_chat_data_train_with_masked_loss(tmp_path: Path, kind, world_size, mp):
    import json

    vocab, _ = _embedding_setup(tmp_path)
    words = ["the", "cat", "sat", "on", "mat", "a", "dog", "ran", "far"]
    if kind == "finetuning_dataset":
        records = [{"prompt": f"the {words[i % 9]} sat", "completion": f"on a {words[(i + 2) % 9]}"} for i in range(24)]
        data = tmp_path / "data.json"  # prompt / completion records are one json list
        data.write_text(json.dumps(records))
    else:
        records = [[{"type": "text", "content": f"the {words[i % 9]}", "has_loss": False},
                    {"type": "text", "content": f"ran {words[(i + 4) % 9]}", "has_loss": True}] for i in range(24)]
        data = tmp_path / "data.jsonl"  # one conversation per line
        data.write_text("\n".join(json.dumps(r) for r in records) + "\n")
    arch = {"vocab_size": 32, "vocab_file": vocab, "sequence_length": 12,
            "softprompt_config": {"name": "sp", "n_tokens": 2}}
    cfg = tiny_config(world_size, mp=mp, arch=arch, iters=3, micro=4)
    cfg["data"] = {kind: True, "data_prefixes": [str(data)]}
    loss, changed, _, _ = dist_launcher(_finetune, world_size, config=cfg)[0]
    assert len(loss) == 3 and all(l == l for l in loss)
    assert any("softprompt" in n for n in changed)


# ---------------------------------------------------------------------------------------------- images in the prompt
def test_image_prefix_finetuning_through_the_clip_tower(tmp_path: Path):
    """Prompt = image + text: the image is encoded by the CLIP tower into 144 positions of the input sequence; the
    text model trains on it with the tower frozen."""
    import json

    import numpy as np
    from PIL import Image

    vocab, _ = _embedding_setup(tmp_path)
    rng = np.random.default_rng(0)
    records = []
    for i in range(2):
        Image.fromarray(rng.integers(0, 255, size=(48, 64, 3), dtype=np.uint8)).save(tmp_path / f"img{i}.jpg")
        records.append({"prompt": [f"img{i}.jpg", "the cat"], "completion": "sat on a mat"})
    data = tmp_path / "data.json"
    data.write_text(json.dumps(records))
    arch = {"vocab_size": 32, "vocab_file": vocab, "sequence_length": 160, "image_encoder": True, "num_layers": 1}
    # the tower (136M parameters) stays frozen: its optimizer states alone would dominate a one-thread CPU test
    groups = [{"group_name": "text", "parameters_exclude": ["image_encoder"], "weight_decay": 0.0,
               "learning_rate_scheduler": {"learning_rate": 1e-3, "learning_rate_decay_style": "constant"}}]
    cfg = tiny_config(1, arch=arch, iters=1, micro=1, groups=groups,
                      training={"allow_missing_params_in_optimizer": True})
    cfg["data"] = {"finetuning_dataset": True, "data_prefixes": [str(data)]}
    loss, changed, frozen, _ = dist_launcher(_finetune, 1, config=cfg)[0]
    assert len(loss) == 1 and loss[0] == loss[0]
    assert changed and not any("image_encoder" in n for n in changed)
    assert any("image_encoder" in n for n in frozen)


def _image_batch_sync_worker(rank, world_size, port, device):
    import torch

    from scaling_b200.transformer.data._finetuning_common import sync_text_image_batch
    from scaling_b200.transformer.data.text_dataset import TextDatasetBatch
    from tests.test_core_distributed import _topology

    t = _topology(rank, world_size, port, mp=2)
    out = []
    for with_images in (True, False):
        batch = None
        if t.model_parallel_rank == 0:
            batch = TextDatasetBatch(
                input_token_ids=torch.arange(12).view(2, 6), target_token_ids=torch.arange(12).view(2, 6) + 1,
                cumulative_seq_lengths=torch.tensor([0, 6, 12], dtype=torch.int32),
                cumulative_seq_lengths_padded=torch.tensor([0, 6, 12, -1], dtype=torch.int32),
                position_ids=torch.arange(6).repeat(2, 1), loss_weights=torch.ones(2, 6),
                input_images=torch.full((1, 3, 4, 4), 0.5) if with_images else None,
                input_image_locations=torch.tensor([[1, 0, 4]]) if with_images else None)
        got = sync_text_image_batch(t, batch)
        out.append((got.input_token_ids.tolist(), got.loss_weights.sum().item(),
                    None if got.input_images is None else (tuple(got.input_images.shape), got.input_images.mean().item()),
                    None if got.input_image_locations is None else got.input_image_locations.tolist()))
    return out


def test_text_and_image_batches_reach_every_tensor_parallel_rank():
    r0, r1 = dist_launcher(_image_batch_sync_worker, 2)
    assert r0 == r1
    assert r1[0][2] == ((1, 3, 4, 4), 0.5) and r1[0][3] == [[1, 0, 4]]
    assert r1[1][2] is None and r1[1][3] is None  # a batch without images stays without


def test_adapters_soft_prompt_bias_set_and_lora_under_sequence_parallelism(tmp_path: Path):
    """With the residual stream split over the tokens: adapters gather and scatter like the MLP, the soft prompt is
    written into the whole sequence before it is split, the dense LoRA output joins after the reduction, gradients of
    replicated LoRA inputs are summed — the losses equal those of one process."""
    arch = dict(FINETUNE_ARCH, lora_config={"name": "lora", "rank": 4, "alpha": 8,
                                            "parallel_modules": ["query", "key", "value", "dense"]})
    groups = [dict(GROUPS[0], parameters_include=GROUPS[0]["parameters_include"] + ["lora"])]
    training = {"allow_missing_params_in_optimizer": True}
    init = str(tmp_path / "init")
    base = losses(1, save_initial=init, arch=arch, groups=groups, training=training)
    got = losses(2, mp=2, sp=True, load_dir=init, arch=arch, groups=groups, training=training)
    for a, b in zip(got, base):
        assert abs(a - b) < 2e-5 * max(1.0, abs(b)), (got, base)


def test_embedding_head_layouts_agree(tmp_path: Path):
    """The replicated pooling head behind tensor, sequence and pipeline parallel trunks: same losses as one process
    (under sequence parallelism every rank sends the same complete gradient into the token gather: it is scaled so
    that the sum over the ranks is the gradient itself)."""
    from tests.test_transformer_training import run_training

    vocab, data = _embedding_setup(tmp_path)
    arch = {"vocab_size": 32, "vocab_file": vocab, "lm_head": False, "sequence_length": 12, "causal": True,
            "embedding_head_config": {"name": "emb", "proj_layers": [16], "pooling": "weighted_mean"}}
    training = {"loss_function_config": {"loss_type": "contrastive_loss", "number_of_hard_negatives": 1,
                                         "use_instructions": True}}

    def cfg(ws, **kw):
        c = tiny_config(ws, arch=arch, iters=4, micro=4, training=training, **kw)
        c["data"] = {"embedding_dataset": True, "data_prefixes": [data]}
        return c

    init = str(tmp_path / "init")
    base = dist_launcher(run_training, 1, config=cfg(1), save_initial=init)[0]
    for kw in (dict(mp=2, sp=True), dict(pp=2, ga=1)):
        got = dist_launcher(run_training, 2, config=cfg(2, load_dir=init, **kw))[0]
        for a, b in zip(got, base):
            assert abs(a - b) < 2e-5 * max(1.0, abs(b)), (kw, got, base)
