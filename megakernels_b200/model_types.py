"""Plain data carriers shared by the model container and the generators.

Reference: megakernels/model_types.py:19-60 (BatchState, ExtraModelConfig).
Only the fields the latency decode path touches are kept.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch
from torch import Tensor

KV_Cache = tuple[Tensor, Tensor]
DeviceType = torch.device | str


@dataclass
class BatchState:
    input_ids: Tensor
    position_ids: Tensor | None = None
    seq_len: int | None = None
    output_ids: Tensor | None = None
    hidden_states: Tensor | None = None
    position_embeddings: tuple[Tensor, Tensor] | None = None

    def __post_init__(self):
        if self.seq_len is None:
            self.seq_len = self.input_ids.shape[-1]


@dataclass
class ExtraModelConfig:
    """Flags that are not part of the Hugging Face config.

    ``tp_size``/``tp_rank``/``tp_group`` describe Megatron-style tensor
    parallelism: q/k/v/up/gate are split along their output rows, o/down along
    their input columns, and each rank owns ``num_kv_heads / tp_size`` KV heads
    (reference: megakernels/llama.py:665-691, 202-207).
    """

    tp_size: int = 1
    tp_rank: int = 0
    tp_group: Any | None = None
    rope_scaling: dict | None = None
    interleave_rope: bool = False
    max_len_override: int | None = None
    max_batch_size: int = 1
