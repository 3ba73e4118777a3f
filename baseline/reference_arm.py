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


def run_reference(args, MODEL, MICRO_BATCH, ClockSampler, dist_env, result_line) -> None:
    if not (REF / "scaling").is_dir():
        _unavailable("baseline/_ref is missing (pip install --target baseline/_ref of the reference was not run)")
        return
    sys.path.insert(0, str(REF))
    try:
        import torch
        import torch.distributed as dist
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
    if not torch.cuda.is_available():
        _unavailable("the reference hard-codes CUDA/NCCL and no GPU is visible")
        return

    rank, world, local = dist_env(args)
    seq = MODEL["sequence_length"]

    class SyntheticDataset(BaseDataset):
        def __init__(self, n, seed):
            g = torch.Generator().manual_seed(1234)
            self.table = torch.randint(1, MODEL["vocab_size"], (n, seq + 1), generator=g, dtype=torch.int64)
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
        cfg = TransformerConfig.from_dict({
            "topology": {"world_size": world, "global_rank": rank, "local_slot": local, "model_parallel_size": 1,
                         "pipe_parallel_size": 1, "data_parallel_size": world, "micro_batch_size": MICRO_BATCH,
                         "gradient_accumulation_steps": 1},
            "optimizer": {"zero": True, "gradient_clipping": 1.0, "beta1": 0.9, "beta2": 0.95},
            "training_groups": [{"group_name": "all", "weight_decay": 0.1,
                                 "learning_rate_scheduler": {"learning_rate": 3e-4,
                                                             "learning_rate_decay_style": "constant"}}],
            "transformer_architecture": dict(MODEL, precision="bfloat16", norm_type="layernorm", mlp_type="default",
                                             relative_position_embedding_type="rotary", weight_tying=False,
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
        dataset = SyntheticDataset(MICRO_BATCH * world * total, 42)
        loader = DataLoader(seed=42, consumed_samples=0, dataset=dataset, topology=topology, pin_memory=True)
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
        tokens = MICRO_BATCH * seq * world
        line = result_line(args, world, tokens, dev_ms, e2e_ms, clocks, 0, MICRO_BATCH * (seq + 1) * 8, 4, "reference")
        line["gpu_launches"] = None
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
