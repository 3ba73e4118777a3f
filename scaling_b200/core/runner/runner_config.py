"""Runner settings (fields of src/scaling/core/runner/runner_config.py:10-73)."""

from __future__ import annotations

from enum import Enum
from pathlib import Path
from typing import List, Optional, Tuple

from pydantic import Field

from ..config import BaseConfig


class RunnerType(Enum):
    PDSH = "pdsh"
    PDSH_DOCKER = "pdsh_docker"


class RunnerDockerConfig(BaseConfig):
    docker_container: Optional[str] = Field(None, description="image to start on every node")
    docker_sudo: bool = Field(False, description="prefix the docker command with sudo")
    docker_mounts: Optional[List[Tuple[str, str]]] = Field(None, description="(host dir, container dir) pairs")


class RunnerConfig(BaseConfig, populate_by_name=True):
    runner_type: RunnerType = Field(RunnerType.PDSH, description="how node launchers are started")
    hostsfile: Optional[Path] = Field(
        None, description="MPI-style hosts file, one 'name slots=N' per line", alias="hostfile"
    )
    hosts: Optional[List[str]] = Field(None, description="hosts given inline ('name slots=4' or 'name slots=0,2')")
    master_port: int = Field(29500, description="rendezvous port of torch.distributed")
    master_addr: Optional[str] = Field(None, description="address of node 0; looked up with 'hostname -I' if omitted")
    script: Optional[Path] = Field(None, description="user script every rank runs")
    default_gpu_count: int = Field(8, description="slots per host when the host entry names none")
    docker_config: RunnerDockerConfig = Field(RunnerDockerConfig(), description="docker options for pdsh_docker")
    use_determined: bool = Field(False, description="track metrics and checkpoints with Determined")
