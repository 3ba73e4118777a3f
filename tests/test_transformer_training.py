"""Transformer application on CPU ranks (gloo): layouts agree and resume is exact."""

import copy
from pathlib import Path

import pytest

from tests.utils import dist_launcher


def tiny_config(world_size, mp=1, pp=1, zero=False, ga=1, micro=4, iters=6, save_dir=None, load_dir=None,
                save_interval=None, ckpt="disabled", arch=None, sp=False, kernel="flash_attention", groups=None,
                training=None):
    dp = world_size // (mp * pp)
    architecture = {
        "vocab_size": 128, "hidden_size": 64, "num_layers": 2, "num_attention_heads": 4, "sequence_length": 32,
        "precision": "float32", "masked_softmax": {"kernel": kernel}, "weight_tying": False,
        "dropout_embedding": 0.0,
    }
    architecture.update(arch or {})
    return {
        "topology": {"world_size": world_size, "model_parallel_size": mp, "pipe_parallel_size": pp,
                     "data_parallel_size": dp, "micro_batch_size": micro // dp, "gradient_accumulation_steps": ga,
                     "device": "cpu", "backend": "gloo", "activation_checkpointing_type": ckpt,
                     "sequence_parallel": sp},
        "optimizer": {"zero": zero, "gradient_clipping": 1.0},
        "training_groups": groups or [{"group_name": "all", "weight_decay": 0.01,
                                       "learning_rate_scheduler": {"learning_rate": 1e-3,
                                                                   "learning_rate_decay_style": "constant"}}],
        "training": training or {},
        "trainer": {"train_iterations": iters, "seed": 11, "save_dir": save_dir, "load_dir": load_dir,
                    "save_interval": save_interval, "assert_checkpoint_loaded": load_dir is not None,
                    "delete_past_optimizer_states": False},
        "transformer_architecture": architecture,
        "data": {"synthetic_samples": 256},
    }


def run_training(rank, world_size, port, device, config, save_initial=None):
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
    if save_initial is not None:
        trainer.save_checkpoint(Path(save_initial))
    metrics = trainer.run_training(return_metrics=True)
    return [m["training/loss"] for m in metrics] if metrics else None


def losses(world_size, save_initial=None, **kw):
    return dist_launcher(run_training, world_size, config=tiny_config(world_size, **kw), save_initial=save_initial)[0]


@pytest.mark.dist
def test_transformer_layouts_agree(tmp_path: Path):
    init = str(tmp_path / "init")
    base = losses(1, save_initial=init)
    assert base[-1] < base[0]
    for kw in (dict(world_size=2, mp=2), dict(world_size=2, pp=2, ga=2, micro=2), dict(world_size=2, zero=True),
               dict(world_size=2, mp=2, sp=True), dict(world_size=1, ckpt="every_layer"),
               dict(world_size=1, kernel="torch")):
        ws = kw.pop("world_size")
        got = losses(ws, load_dir=init, **kw)
        for a, b in zip(got, base):
            assert abs(a - b) < 2e-3, (kw, got, base)


DROPOUT = {"dropout_embedding": 0.1, "dropout_attention_probs": 0.1, "dropout_after_attention": 0.1,
           "dropout_after_mlp": 0.1}


@pytest.mark.dist
@pytest.mark.parametrize("layout", [dict(world_size=1), dict(world_size=2, mp=2),
                                    dict(world_size=2, pp=2, ga=2, micro=2, arch={"weight_tying": True}),
                                    dict(world_size=1, arch=DROPOUT), dict(world_size=1, arch=DROPOUT, kernel="torch"),
                                    dict(world_size=2, mp=2, arch=DROPOUT)])
def test_transformer_resume_is_bit_identical(tmp_path: Path, layout):
    layout = dict(layout)
    ws = layout.pop("world_size")
    full = losses(ws, iters=6, save_dir=str(tmp_path), save_interval=4, **layout)
    resumed = losses(ws, iters=6, load_dir=str(tmp_path), **layout)
    assert resumed == full[4:], (resumed, full[4:])


LLAMA_ARCH = {"norm_type": "rms", "mlp_type": "swiglu", "mlp_factor": 2.5, "attention_bias": False, "mlp_bias": False,
              "attention_qkv_in_one": False, "attention_num_kv_heads": 2, "num_attention_heads": 4,
              "relative_position_embedding_type": "rotary_complex"}


@pytest.mark.dist
def test_llama_style_architecture_layouts_agree(tmp_path: Path):
    """RMSNorm + SwiGLU + grouped-query attention + interleaved rotary, with activation checkpointing: tensor,
    sequence and pipeline parallel layouts reproduce the single-process losses."""
    init = str(tmp_path / "init")
    base = losses(1, save_initial=init, arch=LLAMA_ARCH)
    for kw in (dict(world_size=2, mp=2, ckpt="every_layer"), dict(world_size=2, mp=2, sp=True),
               dict(world_size=2, pp=2, ga=2, micro=2, ckpt="every_layer"), dict(world_size=2, zero=True)):
        ws = kw.pop("world_size")
        got = losses(ws, load_dir=init, arch=LLAMA_ARCH, **kw)
        for a, b in zip(got, base):
            assert abs(a - b) < 2e-4 * max(1.0, abs(b)), (kw, got, base)


@pytest.mark.dist
def test_lora_finetuning_trains_only_the_adapters(tmp_path: Path):
    """LoRA on q/k/v/dense with a frozen base under tensor parallelism: the losses agree with one process."""
    arch = dict(LLAMA_ARCH, lora_config={"name": "lora", "rank": 4, "alpha": 8,
                                         "parallel_modules": ["query", "key", "value", "dense"]})
    groups = [{"group_name": "lora", "parameters_include": ["lora"], "weight_decay": 0.0,
               "learning_rate_scheduler": {"learning_rate": 1e-2, "learning_rate_decay_style": "constant"}}]
    training = {"allow_missing_params_in_optimizer": True}
    init = str(tmp_path / "init")
    base = losses(1, save_initial=init, arch=arch, groups=groups, training=training, iters=8)
    got = losses(2, mp=2, load_dir=init, arch=arch, groups=groups, training=training, iters=8)
    for a, b in zip(got, base):
        assert abs(a - b) < 2e-4 * max(1.0, abs(b)), (got, base)


UMUP_ARCH = {"umup": {"enable": True}, "norm_type": "rms", "mlp_bias": False, "attention_bias": False,
             "weight_tying": False, "relative_position_embedding_type": "rotary"}


@pytest.mark.dist
def test_unit_scaled_parametrization_layouts_agree(tmp_path: Path):
    """u-μP (unit-scaled weights, forward / backward multipliers, residual scaling): tensor- and pipeline-parallel
    layouts and the torch attention path reproduce the single-process losses; the losses start near log(vocab)."""
    import math

    init = str(tmp_path / "init")
    base = losses(1, save_initial=init, arch=UMUP_ARCH)
    assert abs(base[0] - math.log(128)) < 1.0, base
    for kw in (dict(world_size=2, mp=2), dict(world_size=2, pp=2, ga=2, micro=2), dict(world_size=1, kernel="torch")):
        ws = kw.pop("world_size")
        got = losses(ws, load_dir=init, arch=UMUP_ARCH, **kw)
        for a, b in zip(got, base):
            assert abs(a - b) < 5e-4 * max(1.0, abs(b)), (kw, got, base)


@pytest.mark.dist
def test_tied_embedding_and_head_across_pipeline_stages(tmp_path: Path):
    """The embedding on the first stage and the head on the last share one weight: gradients of the two copies are
    summed and the copies stay equal; layouts agree and the checkpoint holds the weight once per owner layer."""
    arch = {"weight_tying": True}
    init = str(tmp_path / "init")
    base = losses(1, save_initial=init, arch=arch)
    for kw in (dict(world_size=2, pp=2, ga=2, micro=2), dict(world_size=2, mp=2), dict(world_size=2, zero=True)):
        ws = kw.pop("world_size")
        got = losses(ws, load_dir=init, arch=arch, **kw)
        for a, b in zip(got, base):
            # the shared weight counts once in the gradient norm, whichever stages hold copies of it
            assert abs(a - b) < 2e-5 * max(1.0, abs(b)), (kw, got, base)
    untied = losses(1, arch={"weight_tying": False})
    assert untied != base


@pytest.mark.dist
def test_activation_checkpointing_replays_dropout_exactly(tmp_path: Path):
    """Recomputation restores the random state of the first pass: with dropout everywhere, per-layer and per-stage
    checkpointing give the losses of the run that keeps its activations, bit for bit, also under tensor parallelism
    (where the dropout masks of the tensor-parallel ranks have to agree)."""
    arch = {"dropout_embedding": 0.1, "dropout_after_attention": 0.1, "dropout_after_mlp": 0.1,
            "dropout_attention_probs": 0.1, "masked_softmax": {"kernel": "torch"}}
    init = str(tmp_path / "init")
    plain = losses(1, save_initial=init, arch=arch)
    assert plain != losses(1, load_dir=init, arch=dict(arch, dropout_after_mlp=0.0, dropout_after_attention=0.0,
                                                       dropout_embedding=0.0, dropout_attention_probs=0.0))
    for ckpt in ("every_layer", "every_pipe_stage"):
        assert losses(1, load_dir=init, arch=arch, ckpt=ckpt) == plain, ckpt
    tp_plain = losses(2, mp=2, load_dir=init, arch=arch)
    assert losses(2, mp=2, load_dir=init, arch=arch, ckpt="every_layer") == tp_plain


@pytest.mark.dist
def test_multi_query_attention_with_fewer_kv_heads_than_tensor_parallel_ranks(tmp_path: Path):
    """One KV head, two tensor-parallel ranks: the KV projections are replicated, each rank back-propagates only
    through its own query heads; weight and input gradients of the replicated projections are summed over the group."""
    arch = dict(LLAMA_ARCH, attention_num_kv_heads=1)
    init = str(tmp_path / "init")
    base = losses(1, save_initial=init, arch=arch)
    for kw in (dict(mp=2), dict(mp=2, sp=True)):
        got = losses(2, load_dir=init, arch=arch, **kw)
        for a, b in zip(got, base):
            assert abs(a - b) < 2e-5 * max(1.0, abs(b)), (kw, got, base)
    # the KV projections are replicated with two ranks and ordinary column-parallel weights with one: a checkpoint of
    # the former resumes into the latter with its optimizer states (the keys differ in the parallel flags only)
    ckpt = str(tmp_path / "tp")
    head = losses(2, mp=2, load_dir=init, arch=arch, iters=3, save_dir=ckpt, save_interval=3)
    tail = losses(1, load_dir=ckpt, arch=arch)
    for a, b in zip(head + tail, base):
        assert abs(a - b) < 2e-5 * max(1.0, abs(b)), (head, tail, base)


@pytest.mark.dist
def test_local_attention_windows_train_and_layouts_agree(tmp_path: Path):
    """Heads restricted to a window of recent tokens (all of them, or the first two of four next to two global
    heads): the window changes the result, and pipeline / tensor / data parallel layouts reproduce it."""
    init = str(tmp_path / "init")
    plain = losses(1, save_initial=init)
    mixed_arch = {"num_local_attention_heads": 2, "local_attention_window_size": 8}
    mixed = losses(1, load_dir=init, arch=mixed_arch)
    assert mixed[-1] < mixed[0] and max(abs(a - b) for a, b in zip(mixed, plain)) > 1e-4
    got = losses(2, load_dir=init, arch=mixed_arch, pp=2, ga=2, micro=2)
    assert all(abs(a - b) < 2e-3 for a, b in zip(got, mixed)), (got, mixed)
    all_arch = {"num_local_attention_heads": 4, "local_attention_window_size": 8}
    local = losses(1, load_dir=init, arch=all_arch)
    assert max(abs(a - b) for a, b in zip(local, mixed)) > 1e-5
    for kw in (dict(mp=2), dict(zero=True)):
        got = losses(2, load_dir=init, arch=all_arch, **kw)
        assert all(abs(a - b) < 2e-3 for a, b in zip(got, local)), (kw, got, local)
