"""Small host helpers (reference: megakernels/utils.py:11-13, 107-109)."""

from __future__ import annotations

import os

import torch

_SM_COUNT_OVERRIDE: int | None = None


def assert_div(a: int, b: int) -> int:
    """Exact integer division (reference: megakernels/utils.py:11-13)."""
    if a % b != 0:
        raise AssertionError(f"{a} is not divisible by {b}")
    return a // b


def set_sm_count_override(n: int | None) -> None:
    """Pin the SM count used by the scheduler.

    The scheduler only needs a number; pinning it lets schedules for a 148-SM
    B200 be built and inspected on a machine without a GPU.
    """
    global _SM_COUNT_OVERRIDE
    _SM_COUNT_OVERRIDE = n


def get_sm_count(device=None) -> int:
    """Number of SMs = number of instruction queues.

    Reference: megakernels/utils.py:107-109 (reads the CUDA device
    properties).  Resolution order here: explicit override, the environment
    variable ``MKB200_SM_COUNT``, then the CUDA device properties.
    """
    if _SM_COUNT_OVERRIDE is not None:
        return _SM_COUNT_OVERRIDE
    env = os.environ.get("MKB200_SM_COUNT")
    if env:
        return int(env)
    if not torch.cuda.is_available():
        raise RuntimeError(
            "get_sm_count: no CUDA device; call set_sm_count_override(n) or set "
            "MKB200_SM_COUNT to build schedules without a GPU"
        )
    if device is None or (isinstance(device, str) and device == "cuda"):
        device = torch.cuda.current_device()
    return torch.cuda.get_device_properties(device).multi_processor_count


def trepr(t: torch.Tensor) -> str:
    """Short tensor summary (reference: megakernels/utils.py:100-104)."""
    return f"shape={tuple(t.shape)}, sum={t.sum()}, vals={t}"
