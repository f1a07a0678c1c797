"""``python -m megakernels_b200.scripts.generate mode=mk ...``

Same ``key=value`` command line and timing method as the reference script
(megakernels/scripts/generate.py:28-207): CUDA events around a whole
generation of ``ntok - 1`` tokens, ``num_warmup`` + ``num_iters`` repeats.
Differences: ``model=`` names an architecture preset (``llama-1b``,
``llama-8b``, ``llama-70b``) initialised from ``seed=`` or a local checkpoint
directory, and the prompt is a list of token ids (``prompt_ids=1,2,3`` or
``prompt_len=32`` random ids) because no tokenizer ships with this package.
Only ``mode=mk`` exists here.
"""

from __future__ import annotations

import sys
import time
from dataclasses import dataclass, fields
from pathlib import Path

import torch

from megakernels_b200.dispatch import make_mk_interpreter, make_schedule_builder
from megakernels_b200.demos.latency.scheduler import (
    LatencyScheduleOptions,
    pick_num_attention_partitions,
)
from megakernels_b200.generators import MK_Generator
from megakernels_b200.llama import LlamaConfig, LlamaForCausalLM
from megakernels_b200.model_types import ExtraModelConfig
from megakernels_b200.scheduler import assign_to_sms, tensorize_instructions

PRESETS = {
    "llama-1b": LlamaConfig.llama_3_2_1b,
    "llama-8b": LlamaConfig.llama_3_1_8b,
    "llama-70b": LlamaConfig.llama_3_1_70b,
    "meta-llama/Llama-3.2-1B-Instruct": LlamaConfig.llama_3_2_1b,
    "meta-llama/Llama-3.1-8B-Instruct": LlamaConfig.llama_3_1_8b,
}


@dataclass
class ScriptConfig:
    model: str = "llama-1b"
    device: str = "cuda:0"
    prompt_ids: str = ""
    prompt_len: int = 32
    seed: int = 0
    layers: int = 0
    ntok: int = 100
    mode: str = "mk"
    interleave_rope: bool = True
    mk_dir: str = ""
    tokens: bool = True
    num_warmup: int = 5
    num_iters: int = 10
    barrier_fill_val: int = 0
    batch_size: int = 1
    max_len_override: int = 16384
    noops: bool = False
    skip_mk: bool = False
    skip_rest: bool = False
    sched: str = "rr"
    setting: str = "latency"
    memory_fraction: float = 0.0
    attn_partitions: int = 0
    coalesce_o_proj: bool = False
    merge_in_last_partial: bool = False

    def finalize(self):
        if self.mode != "mk":
            raise SystemExit(
                f"mode={self.mode}: only mode=mk exists in this package (the torch and Python-VM "
                "paths of the reference are CPU checkers under oracle/)"
            )
        assert self.interleave_rope, "interleave_rope must be True for mk mode"
        assert self.batch_size == 1, "the latency megakernel decodes one sequence"

    def once(self):
        self.num_warmup, self.num_iters = 0, 1

    def l1(self):
        self.model = "llama-1b"

    def l8(self):
        self.model = "llama-8b"


def parse_cli(argv: list[str]) -> ScriptConfig:
    """``key=value`` pairs and zero-argument presets, as pydra does for the reference."""
    cfg = ScriptConfig()
    types = {f.name: f.type for f in fields(cfg)}
    for arg in argv:
        if "=" not in arg:
            if not hasattr(cfg, arg) or arg in types:
                raise SystemExit(f"unknown preset {arg!r}")
            getattr(cfg, arg)()
            continue
        key, val = arg.split("=", 1)
        if key not in types:
            raise SystemExit(f"unknown option {key!r}")
        cur = getattr(cfg, key)
        if isinstance(cur, bool):
            setattr(cfg, key, val.lower() in ("1", "true", "t", "yes"))
        elif isinstance(cur, int):
            setattr(cfg, key, int(val))
        elif isinstance(cur, float):
            setattr(cfg, key, float(val))
        else:
            setattr(cfg, key, val)
    cfg.finalize()
    return cfg


@torch.inference_mode()
def main(config: ScriptConfig):
    torch.cuda.set_device(config.device)
    extra = ExtraModelConfig(
        interleave_rope=config.interleave_rope,
        max_len_override=config.max_len_override,
        max_batch_size=config.batch_size,
    )
    if config.model in PRESETS:
        overrides = {"num_hidden_layers": config.layers} if config.layers else {}
        model = LlamaForCausalLM.from_random(
            PRESETS[config.model](**overrides),
            extra,
            device=config.device,
            seed=config.seed,
            draw_on="device",
        )
    else:
        model = LlamaForCausalLM.from_pretrained(Path(config.model), extra, device=config.device)

    if config.prompt_ids:
        prompt = torch.tensor([int(t) for t in config.prompt_ids.split(",")], dtype=torch.long)
    else:
        g = torch.Generator().manual_seed(1)
        prompt = torch.randint(0, model.config.vocab_size, (config.prompt_len,), generator=g)
    prompt = prompt.to(model.device)
    prompt_len = prompt.numel()
    print(f"Input ids shape: {tuple(prompt.shape)}")

    n_part = config.attn_partitions or pick_num_attention_partitions(
        prompt_len, config.ntok, model.device, model.num_kv_heads()
    )
    options = LatencyScheduleOptions(
        num_attention_partitions=n_part, coalesce_o_proj=config.coalesce_o_proj,
        merge_in_last_partial=config.merge_in_last_partial,
    )
    schedule = make_schedule_builder(config.setting, options).build(model)
    queues = assign_to_sms(
        config.sched, schedule=schedule, memory_fraction=config.memory_fraction or None
    )
    tensorize_instructions(schedule.globs, queues)

    interpreter = make_mk_interpreter(config.setting, Path(config.mk_dir) if config.mk_dir else None)
    gen = MK_Generator(
        model,
        interpreter,
        schedule,
        barrier_fill_val=config.barrier_fill_val,
        skip_mk=config.skip_mk,
        skip_rest=config.skip_rest,
    )
    first = gen.prefill(prompt)
    gen.check()
    if config.noops:
        gen.replace_with_noops()

    output_tokens = torch.zeros(config.batch_size, config.ntok, device=model.device, dtype=torch.long)
    output_tokens[:, 0] = first

    times, cpu_times = [], []
    for _ in range(config.num_warmup + config.num_iters):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        t0 = time.time()
        gen.generate(output_tokens, prompt_len, config.ntok - 1)
        t1 = time.time()
        end.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(end) / 1000)
        cpu_times.append(t1 - t0)
    gen.check()

    timed = times[config.num_warmup :]
    elapsed = sum(timed) / len(timed)
    cpu = sum(cpu_times[config.num_warmup :]) / len(timed)
    print(f"Average time: {elapsed * 1000:.2f}ms (CPU: {cpu * 1000:.2f}ms)")
    if config.tokens:
        print("Output ids: ", output_tokens.cpu())
    fwd_per_second = (config.ntok - 1) / elapsed
    print(f"Fwd per second: {fwd_per_second:.2f}")
    print(f"Tokens per second: {config.batch_size * fwd_per_second:.2f}")
    return output_tokens


if __name__ == "__main__":
    main(parse_cli(sys.argv[1:]))
