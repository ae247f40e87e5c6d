"""Mode -> builder / interpreter maps (reference ``megakernels/dispatch.py:17-42``).

``latency`` is the batch-1 instruction set (the persistent megakernel),
``throughput`` the batched one (operator-level executor).  The reference's PyTorch
interpreter (``make_pyvm_interpreter``) is a correctness oracle, not a product
path; its restatement lives with the tests' oracle and is deliberately not
reachable from this package.
"""
from __future__ import annotations

from pathlib import Path

from .demos.latency.mk import LatencyMK_Interpreter
from .demos.latency.scheduler import LatencyScheduleBuilder
from .demos.throughput.mk import ThroughputMK_Interpreter
from .demos.throughput.scheduler import ThroughputScheduleBuilder
from .mk import MK_Interpreter
from .scheduler import ScheduleBuilder

BUILDER_MAP = {"latency": LatencyScheduleBuilder, "throughput": ThroughputScheduleBuilder}
MK_INTERPRETER_MAP = {"latency": LatencyMK_Interpreter, "throughput": ThroughputMK_Interpreter}


def make_schedule_builder(mode: str) -> ScheduleBuilder:
    return BUILDER_MAP[mode]()


def make_mk_interpreter(mode: str, mk_dir: Path | str | None = None) -> MK_Interpreter:
    return MK_INTERPRETER_MAP[mode](mk_dir)
