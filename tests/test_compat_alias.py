"""Code written against ``scaling.core`` / ``scaling.transformer`` runs on this library through ``compat/scaling``."""

import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent

# An application in the style of the original MLP example: its own layers on BaseLayer, LayerSpec list, ParallelModule,
# Optimizer - every name imported from the `scaling` package.
APP = r'''
import torch
import torch.nn.functional as F
from scaling.core import (BaseLayer, BaseLayerIO, ColumnParallelLinear, LayerSpec, Optimizer, OptimizerConfig,
                          OptimizerParamGroup, OptimizerParamGroupConfig, ParallelModule, RowParallelLinear)
from scaling.core import BaseDataset, BaseDatasetBatch, BaseDatasetItem, DataLoader
from scaling.core.logging import logger
from scaling.core.optimizer import LearningRateSchedulerConfig
from scaling.core.topology import Topology, TopologyConfig
from scaling.core.topology.topology_config import TopologyConfig as TC2
from scaling.core.nn.linear.column_parallel_linear import ColumnParallelLinear as CPL2
from scaling.transformer.context import TransformerConfig
import scaling_b200.parallel
assert TC2 is TopologyConfig is scaling_b200.parallel.TopologyConfig and CPL2 is ColumnParallelLinear


class IO(BaseLayerIO):
    def __init__(self, activations):
        self.activations = activations


class Batch(BaseDatasetBatch):
    def __init__(self, inputs=None, targets=None):
        self.inputs, self.targets = inputs, targets

    def only_inputs(self):
        return Batch(inputs=self.inputs)

    def only_targets(self):
        return Batch(targets=self.targets)


class Item(BaseDatasetItem):
    def __init__(self, x, y):
        self.x, self.y = x, y


class Data(BaseDataset):
    def __init__(self):
        g = torch.Generator().manual_seed(0)
        self.x = torch.rand(256, 32, generator=g)
        self.y = (self.x[:, 0] > 0.5).long()
        super().__init__(seed=0, shuffle=True)

    def ident(self):
        return "toy"

    def __len__(self):
        return 256

    def __getitem__(self, i):
        return Item(self.x[i], self.y[i])

    def set_seed(self, seed, shuffle=True):
        self.seed = seed

    def collate(self, batch):
        return Batch(torch.stack([b.x for b in batch]), torch.stack([b.y for b in batch]))

    @staticmethod
    def sync_batch_to_model_parallel(topology, batch):
        return batch


class Layer(BaseLayer[IO, IO, IO]):
    def __init__(self, cls, n_in, n_out, topology, act):
        super().__init__()
        self.linear = cls(in_features=n_in, out_features=n_out, topology=topology, dtype=torch.float32,
                          **({"parallel_output": True} if cls is ColumnParallelLinear else {"parallel_input": True}))
        self.act = act

    def forward(self, x):
        h = x.activations if isinstance(x, IO) else x.inputs
        return IO(self.act(self.linear(h)))

    @staticmethod
    def input_to_tuple(x):
        return (x.activations if isinstance(x, IO) else x.inputs,)

    @staticmethod
    def tuple_to_input(d):
        return IO(d[0])

    @staticmethod
    def output_to_tuple(x):
        return (x.activations,)

    @staticmethod
    def tuple_to_last_stage_activation(d):
        return IO(d[0])


topology = Topology(TopologyConfig.from_dict({"world_size": 1, "model_parallel_size": 1, "pipe_parallel_size": 1,
                                              "global_rank": 0, "local_slot": 0, "micro_batch_size": 32,
                                              "gradient_accumulation_steps": 1, "device": "cpu", "backend": "gloo"}))
topology.initialize_distributed(master_addr="127.0.0.1", master_port="PORT", seed=1)
specs = [LayerSpec(Layer, ColumnParallelLinear, 32, 64, topology, F.relu),
         LayerSpec(Layer, RowParallelLinear, 64, 2, topology, lambda t: t)]
model = ParallelModule(layer_specs=specs, topology=topology)
group = OptimizerParamGroup(
    named_parameters_with_meta=model.named_parameters_with_meta(),
    config=OptimizerParamGroupConfig(name="all", weight_decay=0.0, learning_rate_scheduler=LearningRateSchedulerConfig(
        learning_rate=0.01, learning_rate_decay_style="constant")))
optimizer = Optimizer(config=OptimizerConfig(), parameter_groups=[group], topology=topology)
loader = DataLoader(seed=0, consumed_samples=0, dataset=Data(), topology=topology)
loss_fn = lambda out, batch: F.cross_entropy(out.activations, batch.targets)
losses = [model.train_step(loader, optimizer, Data.sync_batch_to_model_parallel, loss_fn).loss for _ in range(80)]
assert min(losses[-5:]) < 0.8 * losses[0], losses
print("ALIAS-OK", round(losses[0], 3), round(losses[-1], 3))
'''


def test_an_application_written_against_scaling_core_trains():
    from tests.utils import find_free_port

    env = dict(os.environ, PYTHONPATH=os.pathsep.join([str(ROOT / "compat"), str(ROOT)]))
    res = subprocess.run([sys.executable, "-c", APP.replace("PORT", str(find_free_port()))], capture_output=True,
                         text=True, env=env, cwd="/tmp", timeout=600)
    assert res.returncode == 0 and "ALIAS-OK" in res.stdout, res.stdout[-2000:] + res.stderr[-4000:]


def test_the_alias_is_opt_in():
    """Without compat/ on the path nothing named `scaling` is importable from this repository: an installed copy of
    the original package keeps its name to itself (the benchmark's reference arm relies on that)."""
    env = {k: v for k, v in os.environ.items() if k != "PYTHONPATH"}
    code = "import importlib.util, sys; sys.path.insert(0, %r); print(importlib.util.find_spec('scaling'))" % str(ROOT)
    res = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, cwd="/tmp", timeout=120)
    assert res.returncode == 0 and res.stdout.strip() == "None", res.stdout + res.stderr
