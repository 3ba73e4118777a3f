from .launch_config import LaunchConfig, decode_base64, encode_base64
from .runner import get_resource_pool, parse_host, runner_main
from .runner_config import RunnerConfig, RunnerDockerConfig, RunnerType

__all__ = ["LaunchConfig", "RunnerConfig", "RunnerDockerConfig", "RunnerType", "decode_base64", "encode_base64",
           "get_resource_pool", "parse_host", "runner_main"]
