"""``python -m megakernels_b200.scripts.profile_op op=upgate ...``: one instruction type alone.

Builds a small model of the chosen architecture, schedules one token, blanks every
instruction except those of one opcode (the others become NoOps), presets all barrier
counters so that no wait blocks, and launches the megakernel a few times.  Run it under a
profiler (one kernel, a few launches) to see what a single instruction type does to the
memory system, or on its own for the launch time and the bytes it streams.  The outputs of
such a launch are meaningless; only the traffic is.

    op        qkv | partial | reduction | oproj | upgate | downproj | lm_head | all
    model     llama-1b | llama-8b (default) | llama-70b (one rank's widths need tp=)
    layers    depth of the model (default 4)
    prefill   cached positions (default 1024)
    launches  timed launches after 3 warm-up launches (default 5)

The reference has no counterpart (its scripts time whole generations,
megakernels/scripts/generate.py:167-207).
"""

from __future__ import annotations

import sys

import torch

from megakernels_b200.demos.latency.scheduler import LatencyScheduleOptions, pick_num_attention_partitions
from megakernels_b200.dispatch import make_mk_interpreter, make_schedule_builder
from megakernels_b200.generators import MK_Generator
from megakernels_b200.llama import LlamaConfig, LlamaForCausalLM
from megakernels_b200.model_types import ExtraModelConfig
from megakernels_b200.scheduler import assign_to_sms, tensorize_instructions

OPCODES = {"qkv": 1, "partial": 2, "reduction": 3, "oproj": 4, "upgate": 5, "downproj": 6, "lm_head": 7}
PRESETS = {
    "llama-1b": LlamaConfig.llama_3_2_1b,
    "llama-8b": LlamaConfig.llama_3_1_8b,
    "llama-70b": LlamaConfig.llama_3_1_70b,
}


def bytes_streamed(cfg: LlamaConfig, op: str, layers: int, seq_len: int) -> int:
    """Algorithmic bytes of the kept instructions: bf16 weights once, K and V of the cached positions."""
    H, I, D = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim
    Hq, Hkv, V = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.vocab_size
    per_layer = {
        "qkv": (Hq + 2 * Hkv) * D * H * 2,
        "partial": 2 * Hkv * D * 2 * seq_len,
        "reduction": 0,
        "oproj": H * Hq * D * 2,
        "upgate": 2 * I * H * 2,
        "downproj": H * I * 2,
    }
    if op == "lm_head":
        return V * H * 2
    if op == "all":
        return layers * sum(per_layer.values()) + V * H * 2
    return layers * per_layer[op]


def main(argv: list[str]):
    opts = dict(op="upgate", model="llama-8b", layers="4", prefill="1024", launches="5", vocab="0")
    for arg in argv:
        key, _, val = arg.partition("=")
        if key not in opts:
            raise SystemExit(f"unknown option {key!r}; options: {sorted(opts)}")
        opts[key] = val
    op, layers, prefill = opts["op"], int(opts["layers"]), int(opts["prefill"])
    if op != "all" and op not in OPCODES:
        raise SystemExit(f"op must be one of {sorted(OPCODES)} or 'all'")
    overrides = {"num_hidden_layers": layers}
    if int(opts["vocab"]):
        overrides["vocab_size"] = int(opts["vocab"])
    cfg = PRESETS[opts["model"]](**overrides)
    device = torch.device("cuda", torch.cuda.current_device())
    extra = ExtraModelConfig(interleave_rope=True, max_len_override=prefill + 16)
    model = LlamaForCausalLM.from_random(cfg, extra, device=device, seed=0, draw_on="device")
    for c in model.stacked_kv_cache:
        c[:, :, :prefill].normal_()
    parts = pick_num_attention_partitions(prefill, 16, device, model.num_kv_heads(), min_chunk_size=128)
    options = LatencyScheduleOptions(num_attention_partitions=parts, coalesce_o_proj=True)
    schedule = make_schedule_builder("latency", options).build(model)
    tensorize_instructions(schedule.globs, assign_to_sms("rr", schedule=schedule))
    globs = schedule.globs
    globs.pos_id = prefill
    if op != "all":
        keep = globs.instructions[:, :, 0] == OPCODES[op]
        globs.instructions[~keep] = 0
    kept = int((globs.instructions[:, :, 0] != 0).sum())
    # every counter far above any threshold: no instruction waits for a producer that was blanked
    gen = MK_Generator(model, make_mk_interpreter("latency"), schedule,
                       barrier_fill_val=0 if op == "all" else 1 << 20, fused_argmax=False)
    tok = torch.tensor([[1]], device=device)
    for _ in range(3):
        gen.run(tok, prefill)
    gen.check()
    n = int(opts["launches"])
    events = []
    torch.cuda.profiler.start()
    for _ in range(n):
        globs.hidden_states[:] = model.model.embed_tokens.embed_tokens.weight[1]
        gen.fill()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        gen.last_call = gen.interpreter.interpret(globs)
        e1.record()
        events.append((e0, e1))
    torch.cuda.profiler.stop()
    gen.check()
    ms = sorted(a.elapsed_time(b) for a, b in events)[n // 2]
    nbytes = bytes_streamed(cfg, op, layers, prefill)
    print(f"op={op} model={opts['model']} layers={layers} prefill={prefill} partitions={parts} "
          f"instructions={kept} launch_ms={ms:.4f} algorithmic_MB={nbytes / 1e6:.1f} "
          f"GB_per_s={nbytes / ms / 1e6:.0f}")


if __name__ == "__main__":
    main(sys.argv[1:])
