"""Simulation and drawing of pipeline schedules.

``illustrate`` executes the per-stage instruction lists in lock step: every communication
instruction completes only together with its counterpart on the neighbouring stage and the
tied-gradient reduction is a barrier over all stages; the result lists what each stage does per
step and how often it idles (same model as src/scaling/core/nn/pipeline_schedule/base.py:40-147).
``SimulationEngine`` replays a schedule with measured durations from a ``profile.json`` written by
the profiler and renders a timeline (``base.py:276-697`` in the reference).  Images need Pillow.
"""

from __future__ import annotations

import json
from collections import defaultdict
from pathlib import Path
from typing import Any, Optional, Type

from ....parallel.topology import Topology
from ....parallel.topology_config import TopologyConfig
from .instructions import PEER_OF, InstructionBase

_COLORS = {
    "ForwardPass": (66, 133, 244), "BackwardPass": (219, 68, 55), "Loss": (244, 180, 0),
    "LoadMicroBatch": (15, 157, 88), "SendActivation": (171, 71, 188), "RecvActivation": (0, 172, 193),
    "SendGrad": (255, 112, 67), "RecvGrad": (158, 157, 36), "ReduceTiedGrads": (93, 64, 55),
    "OptimizerStep": (96, 125, 139),
}


def _stage_programs(schedule_cls: Type, grad_acc: int, stages: int) -> list[list[InstructionBase]]:
    programs = []
    for stage in range(stages):
        topo = Topology(TopologyConfig(
            global_rank=stage, pipe_parallel_size=stages, gradient_accumulation_steps=grad_acc,
            model_parallel_size=1, data_parallel_size=1, micro_batch_size=1,
        ))
        programs.append(schedule_cls(topology=topo).instructions())
    return programs


def _ready(programs: list[list[InstructionBase]], pc: list[int], stage: int) -> bool:
    """Can ``stage`` complete its current instruction, given what the other stages are waiting on?"""
    ins = programs[stage][pc[stage]]
    n = len(programs)
    if ins.name == "ReduceTiedGrads":
        return all(pc[s] < len(programs[s]) and programs[s][pc[s]].name == "ReduceTiedGrads" for s in range(n))
    if ins.name in PEER_OF:
        peer_name, offset = PEER_OF[ins.name]
        peer = (stage + offset) % n
        return pc[peer] < len(programs[peer]) and programs[peer][pc[peer]].name == peer_name
    return True


def illustrate(schedule_cls: Type, gradient_accumulation_steps: int, pipe_parallel_size: int) -> dict[str, Any]:
    programs = _stage_programs(schedule_cls, gradient_accumulation_steps, pipe_parallel_size)
    n = pipe_parallel_size
    pc = [0] * n
    steps: list[dict[int, Optional[dict[str, Any]]]] = []
    while any(pc[s] < len(programs[s]) for s in range(n)):
        go = [pc[s] < len(programs[s]) and _ready(programs, pc, s) for s in range(n)]
        if not any(go):
            raise RuntimeError(f"schedule deadlocks at program counters {pc}")
        row: dict[int, Optional[dict[str, Any]]] = {}
        for s in range(n):
            if go[s]:
                ins = programs[s][pc[s]]
                row[s] = {"name": ins.name, "micro_batch_id": ins.micro_batch_id, "buffer_id": ins.buffer_id}
            else:
                row[s] = None
        for s in range(n):
            if go[s]:
                pc[s] += 1
        steps.append(row)
    idle = {s: sum(1 for row in steps if row[s] is None) for s in range(n)}
    total = sum(idle.values())
    return {
        "steps": steps,
        "count_idling": idle,
        "pct_idling": {s: c / len(steps) for s, c in idle.items()},
        "count_idling_total": total,
        "pct_idling_total": total / (len(steps) * n),
    }


def visualize_lockstep(schedule_cls: Type, gradient_accumulation_steps: int, pipe_parallel_size: int):
    from PIL import Image, ImageDraw

    info = illustrate(schedule_cls, gradient_accumulation_steps, pipe_parallel_size)
    cell_w, cell_h, pad = 110, 28, 4
    steps = info["steps"]
    img = Image.new("RGB", (pad + cell_w * pipe_parallel_size, pad + cell_h * (len(steps) + 1)), (255, 255, 255))
    draw = ImageDraw.Draw(img)
    for s in range(pipe_parallel_size):
        draw.text((pad + s * cell_w + 4, pad), f"stage {s}", fill=(0, 0, 0))
    for i, row in enumerate(steps):
        for s, cmd in row.items():
            if cmd is None:
                continue
            x0, y0 = pad + s * cell_w, pad + (i + 1) * cell_h
            draw.rectangle([x0, y0, x0 + cell_w - 2, y0 + cell_h - 2], fill=_COLORS.get(cmd["name"], (200, 200, 200)))
            label = cmd["name"] + ("" if cmd["micro_batch_id"] is None else f" {cmd['micro_batch_id']}")
            draw.text((x0 + 3, y0 + 7), label, fill=(255, 255, 255))
    return img


class SimulationInstruction:
    def __init__(self, instruction: InstructionBase, stage: int, duration: float):
        self.instruction = instruction
        self.stage = stage
        self.duration = duration
        self.start: Optional[float] = None
        self.end: Optional[float] = None

    def __repr__(self) -> str:
        return f"{self.instruction.name}[stage {self.stage}, mb {self.instruction.micro_batch_id}] {self.start}->{self.end}"


class SimulationEngine:
    """Event simulation: compute instructions take their measured time, communication completes when
    both partners have arrived (plus the transfer time), the tied-gradient reduction is a barrier."""

    def __init__(self, schedule_cls: Type, gradient_accumulation_steps: Any = None, pipe_parallel_size: int = 1,
                 durations: Optional[dict[str, float]] = None, default_duration: float = 1.0,
                 profile_data: Optional[dict] = None):
        if isinstance(gradient_accumulation_steps, dict):  # SimulationEngine(schedule, profile_data)
            profile_data, gradient_accumulation_steps = gradient_accumulation_steps, None
        if profile_data is not None:
            gradient_accumulation_steps, pipe_parallel_size, durations = self._read_profile(profile_data)
        self.stages = pipe_parallel_size
        self.durations = durations or {}
        self.default_duration = default_duration
        programs = _stage_programs(schedule_cls, gradient_accumulation_steps, pipe_parallel_size)
        self.programs = [
            [SimulationInstruction(i, s, self.get_duration(i.name, s)) for i in prog] for s, prog in enumerate(programs)
        ]

    @classmethod
    def from_profile(cls, schedule_cls: Type, profile_file: str | Path) -> "SimulationEngine":
        return cls(schedule_cls, profile_data=json.loads(Path(profile_file).read_text()))

    @staticmethod
    def _read_profile(data: dict) -> tuple[int, int, dict[str, float]]:
        """(gradient accumulation steps, pipeline stages, mean duration per timer and per timer@stage) of a gathered
        profile: sizes at the top level or under "topology", observations as dicts or as rows of "fields"."""
        topo = data if "pipe_parallel_size" in data else data["topology"]
        fields = data.get("fields") or ["timer_name", "step", "micro_batch_id", "buffer_id", "pipe_parallel_rank",
                                        "data_parallel_rank", "model_parallel_rank", "duration"]
        sums: dict[str, list[float]] = defaultdict(list)
        for row in data["observations"]:
            rec = dict(zip(fields, row)) if isinstance(row, (list, tuple)) else row
            sums[f"{rec['timer_name']}@{rec['pipe_parallel_rank']}"].append(float(rec["duration"]))
            sums[rec["timer_name"]].append(float(rec["duration"]))
        durations = {k: sum(v) / len(v) for k, v in sums.items()}
        return topo["gradient_accumulation_steps"], topo["pipe_parallel_size"], durations

    def get_duration(self, name: str, stage: int) -> float:
        for key in (f"{name}@{stage}", name, f"Instruction{name}"):
            if key in self.durations:
                return self.durations[key]
        return self.default_duration

    def reset_simulation(self) -> None:
        for prog in self.programs:
            for ins in prog:
                ins.start = ins.end = None

    def simulate(self) -> None:
        self.reset_simulation()
        n = self.stages
        pc = [0] * n
        clock = [0.0] * n
        names = [[i.instruction for i in prog] for prog in self.programs]
        while any(pc[s] < len(self.programs[s]) for s in range(n)):
            progressed = False
            for s in range(n):
                if pc[s] >= len(self.programs[s]):
                    continue
                cur = self.programs[s][pc[s]]
                name = cur.instruction.name
                if name == "ReduceTiedGrads":
                    if not _ready(names, pc, s):
                        continue
                    t0 = max(clock)
                    for r in range(n):
                        ins = self.programs[r][pc[r]]
                        ins.start, ins.end = t0, t0 + ins.duration
                        clock[r] = ins.end
                        pc[r] += 1
                    progressed = True
                    break
                if name in PEER_OF:
                    if not _ready(names, pc, s):
                        continue
                    peer = (s + PEER_OF[name][1]) % n
                    other = self.programs[peer][pc[peer]]
                    t0 = max(clock[s], clock[peer])
                    t1 = t0 + max(cur.duration, other.duration)
                    cur.start, cur.end, other.start, other.end = t0, t1, t0, t1
                    clock[s] = clock[peer] = t1
                    pc[s] += 1
                    pc[peer] += 1
                    progressed = True
                    continue
                cur.start, cur.end = clock[s], clock[s] + cur.duration
                clock[s] = cur.end
                pc[s] += 1
                progressed = True
            if not progressed:
                raise RuntimeError(f"schedule deadlocks at program counters {pc}")

    def summarize(self) -> dict[str, Any]:
        total = max((i.end or 0.0) for prog in self.programs for i in prog)
        busy = {s: sum(i.duration for i in prog) for s, prog in enumerate(self.programs)}
        return {
            "total_time": total,
            "busy_time": busy,
            "pct_idling": {s: 1.0 - busy[s] / total if total > 0 else 0.0 for s in busy},
            "pct_idling_total": 1.0 - sum(busy.values()) / (total * self.stages) if total > 0 else 0.0,
        }

    def visualize(self, milliseconds_per_pixel: float = 10, pipe_pixels: int = 200):
        from PIL import Image, ImageDraw

        summary = self.summarize()
        seconds_per_pixel = milliseconds_per_pixel / 1000.0
        height = int(summary["total_time"] / seconds_per_pixel) + 40
        img = Image.new("RGB", (pipe_pixels * self.stages + 8, max(height, 60)), (255, 255, 255))
        draw = ImageDraw.Draw(img)
        for s, prog in enumerate(self.programs):
            draw.text((4 + s * pipe_pixels, 4), f"stage {s}", fill=(0, 0, 0))
            for ins in prog:
                y0 = 24 + int((ins.start or 0.0) / seconds_per_pixel)
                y1 = 24 + max(int((ins.end or 0.0) / seconds_per_pixel), y0 + 1)
                draw.rectangle([4 + s * pipe_pixels, y0, (s + 1) * pipe_pixels - 2, y1],
                               fill=_COLORS.get(ins.instruction.name, (200, 200, 200)))
        return img

    def next_instruction_for_rank(self, pipe_parallel_rank: int) -> Optional[SimulationInstruction]:
        for ins in self.programs[pipe_parallel_rank]:
            if ins.end is None:
                return ins
        return None
