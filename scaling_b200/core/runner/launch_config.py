"""What a rank learns from its launcher: rendezvous address, ranks and the base64 payload.

Environment contract of the node launcher: MASTER_ADDR, MASTER_PORT, WORLD_SIZE, RANK, LOCAL_SLOT
(src/scaling/core/runner/launch_config.py:40-83).  torchrun's LOCAL_RANK is accepted as a synonym
for LOCAL_SLOT so that scripts also start under ``python -m torch.distributed.run``.
"""

from __future__ import annotations

import base64
import json
import os
from argparse import REMAINDER, ArgumentParser
from pathlib import Path
from typing import Any, Optional

from pydantic import Field

from ..config import BaseConfig


def encode_base64(d: dict) -> str:
    return base64.urlsafe_b64encode(json.dumps(d).encode("utf-8")).decode("utf-8")


def decode_base64(s: str) -> dict[Any, Any]:
    return json.loads(base64.urlsafe_b64decode(s))


class LaunchConfig(BaseConfig):
    master_port: int = Field(description="rendezvous port")
    master_addr: str = Field(description="address of the master node")
    world_size: int = Field(description="number of ranks in the job")
    global_rank: int = Field(description="rank of this process")
    local_slot: int = Field(description="device index of this process on its node")
    payload: Optional[dict[Any, Any]] = Field(None, description="decoded job payload (the config dict)")

    @classmethod
    def from_launcher_args(cls, argv: Optional[list[str]] = None) -> "LaunchConfig":
        env = os.environ
        parser = ArgumentParser(description="rank entry point")
        parser.add_argument("--payload", type=str, default=None, help="base64 encoded payload")
        parser.add_argument("remaining_args", nargs=REMAINDER)
        args = parser.parse_args(argv)
        return cls(
            master_addr=env["MASTER_ADDR"],
            master_port=int(env["MASTER_PORT"]),
            world_size=int(env["WORLD_SIZE"]),
            global_rank=int(env["RANK"]),
            local_slot=int(env.get("LOCAL_SLOT", env.get("LOCAL_RANK", "0"))),
            payload=None if args.payload is None else decode_base64(args.payload),
        )

    def overwrite_config_dict_with_launcher_args(self, config_dict: dict[str, Any]) -> dict[str, Any]:
        topo = config_dict.setdefault("topology", {})
        topo["world_size"] = self.world_size
        topo["global_rank"] = self.global_rank
        topo["local_slot"] = self.local_slot
        log_dir = (config_dict.get("logger") or {}).get("log_dir")
        prof = config_dict.setdefault("profiler", {})
        if prof.get("profiler_output") is None and log_dir is not None:
            prof["profiler_output"] = str(Path(log_dir) / "profile.json")
        return config_dict
