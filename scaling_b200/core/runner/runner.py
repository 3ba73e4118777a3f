"""Job runner: turns a host list into per-node launcher commands (pdsh, optionally in docker).

Behaviour of the reference runner (src/scaling/core/runner/runner.py:19-266): hosts come from
``hosts`` or a hosts file (``name``, ``name slots=4`` or ``name slots=0,2,3``); without hosts the
local GPUs are used; the master address is looked up over ssh unless given; NCCL/PYTHON/UCX/MV2
environment variables are exported to the remote shells; the payload travels as url-safe base64 json.
A single local node is started directly without pdsh.
"""

from __future__ import annotations

import os
import subprocess
import sys
from collections import OrderedDict
from shlex import quote
from typing import Any

import torch

from .launch_config import encode_base64
from .runner_config import RunnerConfig, RunnerType

EXPORT_PREFIXES = ("NCCL", "PYTHON", "MV2", "UCX", "CUDA", "SB200", "TORCH")
ENVIRONMENT_FILE = os.path.join(os.path.expanduser("~"), ".deepspeed_env")
PDSH_FAN_OUT = 1024
LOCAL_NAMES = ("localhost", "127.0.0.1")
LAUNCH_MODULE = "scaling_b200.core.runner.launch"


def parse_host(config: RunnerConfig, host_str: str) -> tuple[str, list[int]]:
    parts = host_str.split()
    if len(parts) == 1:
        return parts[0], list(range(config.default_gpu_count))
    if len(parts) != 2:
        raise ValueError(f"cannot parse host '{host_str}'")
    name, spec = parts
    key, _, value = spec.partition("=")
    assert key == "slots" and value != "", f"host entry must look like 'nodename slots=8', got '{host_str}'"
    if "," in value:
        return name, [int(s) for s in value.split(",") if s]
    return name, list(range(int(value)))


def hosts_str_to_resource_pool(config: RunnerConfig, hosts: list[str]) -> "OrderedDict[str, list[int]]":
    pool: "OrderedDict[str, list[int]]" = OrderedDict()
    for h in hosts:
        name, slots = parse_host(config, h)
        if name in pool:
            raise ValueError(f"host '{name}' defined more than once")
        pool[name] = slots
    if not pool:
        n = torch.cuda.device_count()
        assert n > 0, "no hosts given and no local GPUs found"
        pool["localhost"] = list(range(n))
    return pool


def get_resource_pool(config: RunnerConfig) -> dict[str, Any]:
    if config.hostsfile is not None and config.hosts is not None:
        raise ValueError("Both hostsfile and hosts cannot be defined at the same time.")
    hosts: list[str] = []
    if config.hostsfile is not None:
        if not config.hostsfile.is_file():
            raise ValueError(f"Hostsfile not found: {config.hostsfile}")
        hosts = [ln.strip() for ln in config.hostsfile.read_text().splitlines() if ln.strip()]
    elif config.hosts is not None:
        hosts = list(config.hosts)
    pool = hosts_str_to_resource_pool(config, hosts)
    return {
        "nodes": [{"name": n, "slots": s} for n, s in pool.items()],
        "world_size": sum(len(s) for s in pool.values()),
    }


class PDSHRunner:
    def __init__(self, master_addr: str, config: RunnerConfig, resource_pool: dict[str, Any], payload: dict[Any, Any],
                 exports: dict[str, str], environment: dict[str, str]):
        self.master_addr = master_addr
        self.config = config
        self.resource_pool = resource_pool
        self.payload = payload
        self.exports = exports
        self.environment = environment
        self.environment["PDSH_RCMD_TYPE"] = "ssh"

    @property
    def name(self) -> str:
        return "pdsh"

    @property
    def is_local(self) -> bool:
        nodes = self.resource_pool["nodes"]
        return len(nodes) == 1 and nodes[0]["name"] in LOCAL_NAMES

    def _docker_prefix(self) -> list[str]:
        dc = self.config.docker_config
        cmd = (["sudo"] if dc.docker_sudo else []) + ["docker", "run", "--rm", "--privileged"]
        for k, v in self.exports.items():
            if not k.lower().startswith("python"):
                cmd += ["--env", f"{k}={quote(v)}"]
        for host_dir, cont_dir in dc.docker_mounts or []:
            cmd += ["-v", f"{host_dir}:{cont_dir}"]
        cmd += ["--network=host", "--gpus", "all", "--ipc=host", "--name=scaling_b200", "--ulimit", "memlock=-1",
                "--ulimit", "stack=67108864", str(dc.docker_container)]
        return cmd

    def get_cmd(self) -> list[str]:
        docker = self.config.runner_type == RunnerType.PDSH_DOCKER
        cmd: list[str] = []
        if not self.is_local:
            workers = ",".join(n["name"] for n in self.resource_pool["nodes"])
            cmd += ["pdsh", "-f", str(PDSH_FAN_OUT), "-w", workers]
        if docker:
            cmd += self._docker_prefix()
        elif not self.is_local:
            cmd.append("".join(f"export {k}={quote(v)}; " for k, v in self.exports.items()))
            cmd.append(f"cd {os.path.abspath('')};")
        cmd += ["python" if docker else sys.executable, "-u", "-m", LAUNCH_MODULE,
                f"--resource_pool={encode_base64(self.resource_pool)}"]
        if not self.is_local:
            cmd.append("--node_rank=%n")  # pdsh substitutes the node index
        cmd += [f"--master_addr={self.master_addr}", f"--master_port={self.config.master_port}",
                str(self.config.script.absolute()), "--payload", encode_base64(self.payload)]
        return cmd


def _collect_exports(env: dict[str, str]) -> dict[str, str]:
    exports = {k.strip(): v.strip() for k, v in env.items() if k.startswith(EXPORT_PREFIXES)}
    if os.path.isfile(ENVIRONMENT_FILE):
        with open(ENVIRONMENT_FILE) as f:
            for line in f:
                if "=" in line:
                    k, v = line.strip().split("=", 1)
                    exports[k] = v
    return exports


def runner_main(config: RunnerConfig, payload: dict[str, Any]) -> int:
    assert config.script is not None, "must provide a script to run"
    pool = get_resource_pool(config)
    assert pool["world_size"] > 0, "could not identify resources"
    if config.master_addr is not None:
        master_addr = config.master_addr
    else:
        first = pool["nodes"][0]["name"]
        if first in LOCAL_NAMES:
            master_addr = "127.0.0.1"
        else:
            master_addr = subprocess.check_output(["ssh", first, "hostname", "-I"]).decode().split()[0]
    env = os.environ.copy()
    here = os.path.abspath("")
    env["PYTHONPATH"] = here + (":" + env["PYTHONPATH"] if env.get("PYTHONPATH") else "")
    runner = PDSHRunner(master_addr, config, pool, payload, _collect_exports(env), env)
    proc = subprocess.Popen(runner.get_cmd(), env=env)
    proc.wait()
    if proc.returncode > 0:
        sys.exit(proc.returncode)
    return proc.returncode
