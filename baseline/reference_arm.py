"""Reference arm of the benchmark: the UNMODIFIED Aleph-Alpha/scaling package installed under
``baseline/_ref``, driven through its own public API (``TransformerConfig`` -> ``Topology`` -> ``TransformerContext``
-> ``init_model`` / ``init_optimizer`` -> ``ParallelModule.train_step`` fed by its ``DataLoader``), same model, batch,
precision and optimizer settings as our arm.  Nothing from ``scaling_b200`` is imported here.  The only additions
are a synthetic ``BaseDataset`` subclass (the reference ships no synthetic data source) and the timing harness.
If the reference cannot be imported or run, one json line ``{"impl": "reference", "unavailable": "<reason>"}`` is
printed and the process exits 0.
"""

from __future__ import annotations

import json
import os
import sys
from pathlib import Path

REF = Path(__file__).resolve().parent / "_ref"


def _unavailable(reason: str) -> None:
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": reason.replace("\n", " ")[:300]}), flush=True)


def reference_architecture(lay: dict) -> tuple[dict, str | None]:
    """Architecture dict for the reference and, where the reference cannot run the named one, a note on what was
    changed.  The reference divides the KV heads by the tensor-parallel size with integer division and then
    divides by the result (scaling/core/nn/attention/attention.py), so fewer KV heads than tensor-parallel ranks
    raise ZeroDivisionError: in that case its arm runs with as many KV heads as tensor-parallel ranks."""
    arch = dict(lay["arch"])
    note = None
    kv = arch.get("attention_num_kv_heads")
    if kv is not None and kv < lay["mp"]:
        arch["attention_num_kv_heads"] = lay["mp"]
        note = f"reference run with attention_num_kv_heads={lay['mp']} (it cannot run {kv} KV heads on TP={lay['mp']})"
    return arch, note


def run_reference(args, lay, ClockSampler, dist_env, result_line) -> None:
    if not (REF / "scaling").is_dir():
        _unavailable("baseline/_ref is missing (pip install --target baseline/_ref of the reference was not run)")
        return
    sys.path.insert(0, str(REF))
    try:
        import torch
        import torch.distributed as dist
        import scaling
        from scaling.core import DataLoader, Topology
        from scaling.core.data import BaseDataset
        from scaling.transformer import TransformerConfig, TransformerContext, init_model, init_optimizer
        from scaling.transformer.data.text_dataset import TextDataset
        from scaling.transformer.data.text_dataset_batch import TextDatasetBatch, TextDatasetBatchBeforeSync
        from scaling.transformer.data.text_dataset_item import TextDatasetItem
        from scaling.transformer.model.losses import create_loss_function
        from scaling.transformer.model.model import metrics_aggregation_fn
    except Exception as e:  # noqa: BLE001
        _unavailable(f"import of the reference failed: {type(e).__name__}: {e}")
        return
    if REF.resolve() not in Path(scaling.__file__).resolve().parents:
        _unavailable(f"`scaling` resolved to {scaling.__file__}, not to the installed reference")
        return
    if not torch.cuda.is_available():
        _unavailable("the reference hard-codes CUDA/NCCL and no GPU is visible")
        return

    rank, world, local = dist_env(args)
    arch, note = reference_architecture(lay)
    seq, vocab = arch["sequence_length"], arch["vocab_size"]
    micro, ga, dp = lay["micro"], lay["ga"], lay["dp"]

    class SyntheticDataset(BaseDataset):
        def __init__(self, n, seed):
            g = torch.Generator().manual_seed(1234)
            self.table = torch.randint(1, vocab, (n, seq + 1), generator=g, dtype=torch.int64)
            super().__init__(seed=seed, shuffle=True)

        def ident(self):
            return "synthetic"

        def __len__(self):
            return self.table.shape[0]

        def __getitem__(self, i):
            return TextDatasetItem(token_ids=self.table[i])

        def set_seed(self, seed, shuffle=True):
            self.seed = seed

        def collate(self, batch):
            return TextDatasetBatchBeforeSync(token_ids=torch.stack([b.token_ids for b in batch]))

        @staticmethod
        def sync_batch_to_model_parallel(topology, batch):
            return TextDataset.sync_batch_to_model_parallel(topology, batch)

    try:
        group = {"group_name": "all", "weight_decay": 0.1,
                 "learning_rate_scheduler": {"learning_rate": 3e-4, "learning_rate_decay_style": "constant"}}
        if lay["lora"]:
            group = dict(group, group_name="lora", parameters_include=["lora"], weight_decay=0.0)
        cfg = TransformerConfig.from_dict({
            "topology": {"world_size": world, "global_rank": rank, "local_slot": local,
                         "model_parallel_size": lay["mp"], "pipe_parallel_size": lay["pp"],
                         "data_parallel_size": dp, "micro_batch_size": micro, "gradient_accumulation_steps": ga,
                         "activation_checkpointing_type": lay["ckpt"],
                         "sequence_parallel": bool(getattr(args, "sequence_parallel", False) and lay["mp"] > 1)},
            "optimizer": {"zero": True, "gradient_clipping": 1.0, "beta1": 0.9, "beta2": 0.95},
            "training_groups": [group],
            "training": {"allow_missing_params_in_optimizer": True} if lay["lora"] else {},
            "transformer_architecture": dict(arch, precision="bfloat16", weight_tying=False,
                                             masked_softmax={"kernel": "flash_attention"}, causal=True),
            "trainer": {"seed": 42},
        })
        topology = Topology(cfg.topology)
        context = TransformerContext(config=cfg, topology=topology)
        context.initialize(master_addr=os.environ["MASTER_ADDR"], master_port=os.environ["MASTER_PORT"], seed=42)
        model = init_model(context)
        optimizer = init_optimizer(context, model)
        loss_fn = create_loss_function(context, cfg.training.loss_function_config)
        total = 2 * (args.steps + args.warmup) + 2
        dataset = SyntheticDataset(micro * dp * ga * total, 42)
        loader = DataLoader(seed=42, consumed_samples=0, dataset=dataset, topology=topology, pin_memory=True) \
            if topology.is_io_rank else None
        sync = SyntheticDataset.sync_batch_to_model_parallel
        dev = topology.device

        # The reference's batch sync always assembles the batch on the host and copies it to the device
        # (scaling/core/data/broadcast_data.py), so there is no device-resident input path through its API:
        # both numbers below are measured with the stock DataLoader.
        def barrier():
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()

        def timed(n_warm, n_steps, dl):
            for _ in range(n_warm):
                model.train_step(dl, optimizer, sync, loss_fn, metrics_aggregation_fn)
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(n_steps):
                model.train_step(dl, optimizer, sync, loss_fn, metrics_aggregation_fn)
            e1.record()
            barrier()
            ms = torch.tensor([e0.elapsed_time(e1) / n_steps], device=dev)
            if world > 1:
                dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            return float(ms.item())

        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        dev_ms = timed(args.warmup, args.steps, loader)
        e2e_ms = timed(args.warmup, args.steps, loader)
        clocks = sampler.stop() if rank == 0 else {}
    except Exception as e:  # noqa: BLE001
        import traceback

        traceback.print_exc(file=sys.stderr)
        _unavailable(f"the reference failed to run: {type(e).__name__}: {e}")
        return
    if rank == 0:
        tokens = micro * seq * dp * ga
        line = result_line(args, world, tokens, dev_ms, e2e_ms, clocks, 0, micro * ga * (seq + 1) * 8, 4 * ga,
                           "reference", lay)
        line["gpu_launches"] = None
        if note:
            line["details"] = {"reference_deviation": note}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
