"""Generate the golden fixtures by running the reference implementation itself.

Run once on a machine that has a checkout of the reference (point
``MK_REFERENCE_DIR`` at it):

    python tests/golden/make_golden.py

It imports the reference's Python package unmodified (two in-process shims: a
stub ``accelerate`` module, which the reference only uses for checkpoint
loading, and a fixed SM count of 148 in place of a CUDA device query), builds
seeded random-init models through the reference's own classes, and records

* ``sched_1b.json``  - SHA-256 of the reference's serialized instruction tensor
  for the Llama-3.2-1B shape under every assignment mode (rr, zz, wave, dag);
* ``pyvm_1b_w2.pt``  - reference Python-VM and torch-path outputs of three
  teacher-forced decode steps on a 2-layer model with 1B widths;
* ``torch_8b_w1.pt`` - reference torch-path outputs on a 1-layer model with 8B
  widths (the reference's Python VM cannot run this shape);
* RoPE table rows for both rope-scaling settings.

The tests never import the reference: they rebuild the same weights from the
same seeds with this repository's code and compare against these files.
"""

from __future__ import annotations

import contextlib
import hashlib
import json
import os
import sys
import types
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent
if "MK_REFERENCE_DIR" not in os.environ:
    raise SystemExit("set MK_REFERENCE_DIR to a checkout of the reference (HazyResearch/Megakernels)")
REF = Path(os.environ["MK_REFERENCE_DIR"])
sys.path.insert(0, str(REPO))
sys.path.insert(0, str(REF))

import transformers  # noqa: E402,F401  (must be imported before the accelerate stub)

_acc = types.ModuleType("accelerate")


@contextlib.contextmanager
def _init_empty_weights(include_buffers=False):
    yield


_acc.init_empty_weights = _init_empty_weights
sys.modules["accelerate"] = _acc

import megakernels.utils as ref_utils  # noqa: E402

ref_utils.get_sm_count = lambda device=None: 148
import megakernels.instructions as ref_instructions  # noqa: E402
import megakernels.demos.latency.scheduler as ref_lat_sched  # noqa: E402

ref_instructions.get_sm_count = ref_utils.get_sm_count
ref_lat_sched.get_sm_count = ref_utils.get_sm_count

from megakernels.demos.latency.python_vm import INSTRUCTION_TO_SOLVER  # noqa: E402
from megakernels.dispatch import make_schedule_builder  # noqa: E402
from megakernels.llama import LlamaForCausalLM as RefLlama  # noqa: E402
from megakernels.model_types import BatchState, ExtraModelConfig as RefExtra  # noqa: E402
from megakernels.python_vm import interpret_with_pyvm  # noqa: E402
from megakernels.scheduler import assign_to_sms, tensorize_instructions  # noqa: E402
from transformers import LlamaConfig as HFLlamaConfig  # noqa: E402

from megakernels_b200.llama import LlamaConfig, LlamaForCausalLM  # noqa: E402
from megakernels_b200.model_types import ExtraModelConfig  # noqa: E402

SEED_WEIGHTS, SEED_KV, SEED_TOKENS = 0, 2, 3
ROPE_ROWS = [0, 1, 7, 20, 21, 22, 63]


def hf_config(cfg: LlamaConfig) -> HFLlamaConfig:
    return HFLlamaConfig(
        hidden_size=cfg.hidden_size,
        intermediate_size=cfg.intermediate_size,
        num_hidden_layers=cfg.num_hidden_layers,
        num_attention_heads=cfg.num_attention_heads,
        num_key_value_heads=cfg.num_key_value_heads,
        head_dim=cfg.head_dim,
        vocab_size=cfg.vocab_size,
        max_position_embeddings=cfg.max_position_embeddings,
        rms_norm_eps=cfg.rms_norm_eps,
        rope_theta=cfg.rope_theta,
        tie_word_embeddings=cfg.tie_word_embeddings,
        rope_scaling=dict(cfg.rope_scaling) if cfg.rope_scaling else None,
    )


@torch.no_grad()
def build_reference_model(cfg: LlamaConfig, max_len: int, seeded: bool = True) -> RefLlama:
    """Reference model with seeded N(0, 0.02) matrices and unit norm weights."""
    torch.set_default_dtype(torch.bfloat16)
    model = RefLlama(hf_config(cfg), RefExtra(interleave_rope=True, max_len_override=max_len))
    gen = torch.Generator().manual_seed(SEED_WEIGHTS)
    for name, p in model.named_parameters():
        if "norm" in name:
            p.fill_(1.0)
        elif name == "lm_head.lm_head.weight" and cfg.tie_word_embeddings:
            continue
        elif seeded:
            p.copy_(torch.randn(p.shape, generator=gen, dtype=torch.float32) * 0.02)
        else:
            p.zero_()
    if cfg.tie_word_embeddings:
        model.lm_head.lm_head.weight = model.model.embed_tokens.embed_tokens.weight
    model.requires_grad_(False)
    model.model.interleave_rope()
    model.stack_params()
    model.setup_caches()
    torch.set_default_dtype(torch.float32)
    return model


def check_same_weights(ref: RefLlama, mine: LlamaForCausalLM):
    sp, mp = ref.stacked_params, mine.stacked_params
    for name in ("qkv_proj", "o_proj", "up_proj", "gate_proj", "down_proj"):
        assert torch.equal(getattr(sp, name), getattr(mp, name)), name
    assert torch.equal(ref.lm_head.lm_head.weight, mine.lm_head.lm_head.weight)
    assert torch.equal(
        ref.model.embed_tokens.embed_tokens.weight, mine.model.embed_tokens.embed_tokens.weight
    )
    n = mine.model.rope_cos.shape[0]
    assert torch.equal(ref.model.rope_cos[:n], mine.model.rope_cos), "rope cos"
    assert torch.equal(ref.model.rope_sin[:n], mine.model.rope_sin), "rope sin"


def weight_fingerprint(model) -> dict:
    sp = model.stacked_params
    out = {}
    for name in ("qkv_proj", "o_proj", "up_proj", "gate_proj", "down_proj"):
        t = getattr(sp, name)
        out[name] = hashlib.sha256(t.view(torch.int16).numpy().tobytes()).hexdigest()
    return out


def seeded_kv(model, prefill: int):
    gen = torch.Generator().manual_seed(SEED_KV)
    k, v = model.stacked_kv_cache
    k.zero_()
    v.zero_()
    k[:, :, :prefill] = torch.randn(k[:, :, :prefill].shape, generator=gen, dtype=torch.float32)
    v[:, :, :prefill] = torch.randn(v[:, :, :prefill].shape, generator=gen, dtype=torch.float32)


def seeded_tokens(vocab: int, n: int) -> list[int]:
    gen = torch.Generator().manual_seed(SEED_TOKENS)
    return torch.randint(0, vocab, (n,), generator=gen).tolist()


@torch.no_grad()
def run_reference_pyvm(model: RefLlama, prefill: int, tokens: list[int]):
    builder = make_schedule_builder("latency")
    schedule = builder.build(model)
    globs = schedule.globs
    instructions = schedule.get_linear_instructions()
    tensorize_instructions(globs, assign_to_sms("rr", schedule=schedule))
    seeded_kv(model, prefill)
    embed = model.model.embed_tokens.embed_tokens.weight
    steps = []
    for i, tok in enumerate(tokens):
        pos = prefill + i
        globs.hidden_states[:] = embed[tok]
        globs.barriers.zero_()
        globs.pos_id = pos
        interpret_with_pyvm(globs, instructions, INSTRUCTION_TO_SOLVER)
        steps.append(
            dict(
                pos=pos,
                token=tok,
                logits=globs.logits.clone(),
                hidden_states=globs.hidden_states.clone(),
                post_ln_rope_q=globs.post_ln_rope_q.clone(),
                attn_out=globs.attn_out.clone(),
                silu_out=globs.silu_out.clone(),
                k_new=globs.k_cache[:, 0, pos].clone(),
                v_new=globs.v_cache[:, 0, pos].clone(),
                barriers=globs.barriers.clone(),
            )
        )
    return steps, globs.instructions.clone()


@torch.no_grad()
def run_reference_torch(model: RefLlama, prefill: int, tokens: list[int]):
    seeded_kv(model, prefill)
    captured = {}
    handle = model.lm_head.lm_head.register_forward_hook(
        lambda mod, inp, out: captured.__setitem__("logits", out.detach().clone())
    )
    steps = []
    for i, tok in enumerate(tokens):
        pos = prefill + i
        bs = BatchState(
            input_ids=torch.tensor([[tok]]),
            position_ids=torch.tensor([[pos]]),
            seq_len=pos + 1,
        )
        out = model(bs)
        steps.append(
            dict(
                pos=pos,
                token=tok,
                logits=captured["logits"].reshape(-1),
                output_id=int(out.output_ids.reshape(-1)[0]),
                k_new=model.stacked_kv_cache[0][:, 0, pos].clone(),
                v_new=model.stacked_kv_cache[1][:, 0, pos].clone(),
            )
        )
    handle.remove()
    return steps


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().numpy().tobytes()).hexdigest()


def make_schedule_hashes():
    cfg = LlamaConfig.llama_3_2_1b()
    model = build_reference_model(cfg, max_len=64, seeded=False)
    builder = make_schedule_builder("latency")
    out = {"sm_count": 148, "shape": "llama-3.2-1b", "modes": {}}
    for mode in ("rr", "zz", "wave", "dag"):
        schedule = builder.build(model)
        schedule.globs.pos_id = 41
        queues = assign_to_sms(mode, schedule=schedule)
        tensorize_instructions(schedule.globs, queues)
        t = schedule.globs.instructions
        out["modes"][mode] = {"shape": list(t.shape), "sha256": sha(t)}
        print(mode, list(t.shape), out["modes"][mode]["sha256"][:16])
    out["num_instructions"] = len(schedule.get_linear_instructions())
    (HERE / "sched_1b.json").write_text(json.dumps(out, indent=1) + "\n")


def make_model_fixture(name: str, cfg: LlamaConfig, max_len: int, prefill: int, with_pyvm: bool):
    ref = build_reference_model(cfg, max_len)
    mine = LlamaForCausalLM.from_random(
        cfg,
        ExtraModelConfig(interleave_rope=True, max_len_override=max_len),
        device="cpu",
        seed=SEED_WEIGHTS,
    )
    check_same_weights(ref, mine)
    tokens = seeded_tokens(cfg.vocab_size, 3)
    fixture = dict(
        config=vars(cfg),
        max_len=max_len,
        prefill=prefill,
        tokens=tokens,
        seeds=dict(weights=SEED_WEIGHTS, kv=SEED_KV, tokens=SEED_TOKENS),
        weight_sha256=weight_fingerprint(ref),
        rope_rows=ROPE_ROWS,
        rope_cos=ref.model.rope_cos[ROPE_ROWS].clone(),
        rope_sin=ref.model.rope_sin[ROPE_ROWS].clone(),
    )
    if with_pyvm:
        steps, instr = run_reference_pyvm(ref, prefill, tokens)
        fixture["pyvm_steps"] = steps
        fixture["instructions_rr_sha256"] = sha(instr)
        fixture["instructions_shape"] = list(instr.shape)
    fixture["torch_steps"] = run_reference_torch(ref, prefill, tokens)
    torch.save(fixture, HERE / name)
    print(name, (HERE / name).stat().st_size, "bytes")


def main():
    make_schedule_hashes()
    small_1b = LlamaConfig.llama_3_2_1b(num_hidden_layers=2, vocab_size=4096)
    make_model_fixture("pyvm_1b_w2.pt", small_1b, max_len=64, prefill=20, with_pyvm=True)
    small_8b = LlamaConfig.llama_3_1_8b(num_hidden_layers=1, vocab_size=4096)
    make_model_fixture("torch_8b_w1.pt", small_8b, max_len=64, prefill=20, with_pyvm=False)


if __name__ == "__main__":
    main()
