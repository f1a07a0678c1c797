"""Shared helpers of the parity tests (CPU side)."""

from __future__ import annotations

import torch

from megakernels_b200.demos.latency.scheduler import (
    LatencyScheduleBuilder,
    LatencyScheduleOptions,
)
from megakernels_b200.llama import LlamaConfig, LlamaForCausalLM
from megakernels_b200.model_types import ExtraModelConfig

SEED_WEIGHTS, SEED_KV, SEED_TOKENS = 0, 2, 3


def load_fixture(path):
    return torch.load(path, map_location="cpu", weights_only=False)


def config_from_fixture(fx) -> LlamaConfig:
    return LlamaConfig(**fx["config"])


def build_model(cfg, max_len, device="cpu", tp_size=1, tp_rank=0, seed=SEED_WEIGHTS):
    extra = ExtraModelConfig(
        interleave_rope=True, max_len_override=max_len, tp_size=tp_size, tp_rank=tp_rank
    )
    return LlamaForCausalLM.from_random(cfg, extra, device=device, seed=seed)


def fill_kv(model, prefill: int, poison: bool = False, seed: int = SEED_KV):
    """Seeded N(0,1) KV prefix; optionally N(0,100) beyond it (diff_test.py:112-118)."""
    gen = torch.Generator().manual_seed(seed)
    k, v = model.stacked_kv_cache
    kk = torch.zeros(k.shape, dtype=torch.float32)
    vv = torch.zeros(v.shape, dtype=torch.float32)
    kk[:, :, :prefill] = torch.randn(kk[:, :, :prefill].shape, generator=gen)
    vv[:, :, :prefill] = torch.randn(vv[:, :, :prefill].shape, generator=gen)
    if poison:
        kk[:, :, prefill:] = torch.randn(kk[:, :, prefill:].shape, generator=gen) * 100
        vv[:, :, prefill:] = torch.randn(vv[:, :, prefill:].shape, generator=gen) * 100
    k.copy_(kk.to(k.dtype))
    v.copy_(vv.to(v.dtype))


def seeded_tokens(vocab: int, n: int, seed: int = SEED_TOKENS):
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=gen).tolist()


def build_schedule(model, options: LatencyScheduleOptions | None = None, **kw):
    return LatencyScheduleBuilder(options).build(model, **kw)
