"""Mode name -> schedule builder / megakernel interpreter.

Reference: megakernels/dispatch.py:17-42.  Only the ``latency`` setting is in
this package: the reference's ``throughput`` setting has no kernel in its own
tree, and its Python VM is test infrastructure that lives outside the product.
"""

from __future__ import annotations

from pathlib import Path

from megakernels_b200.demos.latency.mk import LatencyMK_Interpreter
from megakernels_b200.demos.latency.scheduler import (
    LatencyScheduleBuilder,
    LatencyScheduleOptions,
)
from megakernels_b200.mk import MK_Interpreter
from megakernels_b200.scheduler import ScheduleBuilder

BUILDER_MAP = {"latency": LatencyScheduleBuilder}
MK_INTERPRETER_MAP = {"latency": LatencyMK_Interpreter}


def make_schedule_builder(mode: str, options: LatencyScheduleOptions | None = None) -> ScheduleBuilder:
    if mode not in BUILDER_MAP:
        raise KeyError(f"unknown setting {mode!r}; available: {sorted(BUILDER_MAP)}")
    return BUILDER_MAP[mode](options)


def make_mk_interpreter(mode: str, mk_dir: Path | None = None) -> MK_Interpreter:
    if mode not in MK_INTERPRETER_MAP:
        raise KeyError(f"unknown setting {mode!r}; available: {sorted(MK_INTERPRETER_MAP)}")
    return MK_INTERPRETER_MAP[mode](mk_dir)


def make_pyvm_interpreter(mode: str):
    raise NotImplementedError(
        "the Python VM is a CPU checker, not a product path; it lives in oracle/python_vm.py "
        "and is only used by the tests"
    )
