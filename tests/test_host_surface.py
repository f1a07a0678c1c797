"""Host-side surface around the kernel: command line of the generate script, checkpoint
loading with tensor-parallel slicing, and (on a GPU) one script run and one recorded trace."""

import json

import pytest
import torch

from megakernels_b200.llama import LlamaConfig, LlamaForCausalLM
from megakernels_b200.model_types import ExtraModelConfig
from megakernels_b200.scripts.generate import ScriptConfig, main, parse_cli

TINY = dict(
    hidden_size=2048, intermediate_size=2048, num_hidden_layers=2, num_attention_heads=8,
    num_key_value_heads=2, head_dim=128, vocab_size=512, tie_word_embeddings=False,
)


# ---- scripts/generate.py: the key=value command line (reference: scripts/generate.py:28-66) ---- #
def test_parse_cli_defaults_follow_the_reference_script():
    cfg = parse_cli([])
    assert (cfg.mode, cfg.setting, cfg.sched, cfg.ntok) == ("mk", "latency", "rr", 100)
    assert (cfg.num_warmup, cfg.num_iters, cfg.max_len_override) == (5, 10, 16384)
    assert cfg.interleave_rope is True and cfg.batch_size == 1 and cfg.barrier_fill_val == 0


def test_parse_cli_types_and_presets():
    cfg = parse_cli(["l8", "once", "ntok=8", "layers=2", "tokens=false", "memory_fraction=0.25",
                     "prompt_ids=1,2,3", "sched=wave", "coalesce_o_proj=true", "merge_in_last_partial=true"])
    assert cfg.model == "llama-8b" and (cfg.num_warmup, cfg.num_iters) == (0, 1)
    assert cfg.ntok == 8 and cfg.layers == 2 and cfg.tokens is False and cfg.coalesce_o_proj is True
    assert cfg.merge_in_last_partial is True and parse_cli([]).merge_in_last_partial is False
    assert cfg.memory_fraction == 0.25 and cfg.prompt_ids == "1,2,3" and cfg.sched == "wave"
    assert isinstance(cfg, ScriptConfig)


@pytest.mark.parametrize("argv", [["mode=torch"], ["mode=pyvm"], ["nonsense=1"], ["ntok"], ["bogus_preset"]])
def test_parse_cli_rejects_what_the_package_does_not_have(argv):
    with pytest.raises(SystemExit):
        parse_cli(argv)


def test_parse_cli_requires_interleaved_rope_and_batch_one():
    with pytest.raises(AssertionError):
        parse_cli(["interleave_rope=false"])
    with pytest.raises(AssertionError):
        parse_cli(["batch_size=2"])


# ---- checkpoint loading (reference: llama.py:583-711, utils.py:34-97) ---- #
def write_checkpoint(path, cfg: LlamaConfig, seed=0, std=0.02):
    """A Hugging Face style directory holding exactly the tensors ``from_random`` draws."""
    from safetensors.torch import save_file

    gen = torch.Generator().manual_seed(seed)
    draw = lambda *shape: (torch.randn(shape, generator=gen, dtype=torch.float32) * std).to(torch.bfloat16)  # noqa: E731
    H, I, D = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim
    Hq, Hkv, V = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.vocab_size
    tensors = {"model.embed_tokens.weight": draw(V, H)}
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        tensors[p + "self_attn.q_proj.weight"] = draw(Hq * D, H)
        tensors[p + "self_attn.k_proj.weight"] = draw(Hkv * D, H)
        tensors[p + "self_attn.v_proj.weight"] = draw(Hkv * D, H)
        tensors[p + "self_attn.o_proj.weight"] = draw(H, Hq * D)
        tensors[p + "mlp.up_proj.weight"] = draw(I, H)
        tensors[p + "mlp.gate_proj.weight"] = draw(I, H)
        tensors[p + "mlp.down_proj.weight"] = draw(H, I)
        tensors[p + "input_layernorm.weight"] = torch.ones(H, dtype=torch.bfloat16)
        tensors[p + "post_attention_layernorm.weight"] = torch.ones(H, dtype=torch.bfloat16)
    tensors["lm_head.weight"] = draw(V, H)
    tensors["model.norm.weight"] = torch.ones(H, dtype=torch.bfloat16)
    names = sorted(tensors)
    half = len(names) // 2  # two shard files, as real checkpoints have
    save_file({k: tensors[k] for k in names[:half]}, str(path / "model-00001-of-00002.safetensors"))
    save_file({k: tensors[k] for k in names[half:]}, str(path / "model-00002-of-00002.safetensors"))
    (path / "config.json").write_text(json.dumps(dict(
        hidden_size=H, intermediate_size=I, num_hidden_layers=cfg.num_hidden_layers,
        num_attention_heads=Hq, num_key_value_heads=Hkv, head_dim=D, vocab_size=V,
        max_position_embeddings=cfg.max_position_embeddings, rms_norm_eps=cfg.rms_norm_eps,
        rope_theta=cfg.rope_theta, tie_word_embeddings=False, rope_scaling=cfg.rope_scaling,
    )))


@pytest.mark.parametrize("tp,rank", [(1, 0), (2, 0), (2, 1)])
def test_from_pretrained_equals_from_random_on_the_same_tensors(tmp_path, tp, rank):
    """Name map, q/k row interleave and tensor-parallel slices of the loader."""
    cfg = LlamaConfig(**TINY)
    write_checkpoint(tmp_path, cfg)
    extra = ExtraModelConfig(interleave_rope=True, max_len_override=32, tp_size=tp, tp_rank=rank)
    loaded = LlamaForCausalLM.from_pretrained(tmp_path, extra, device="cpu")
    drawn = LlamaForCausalLM.from_random(cfg, extra, device="cpu", seed=0)
    for name in ("qkv_proj", "o_proj", "up_proj", "gate_proj", "down_proj", "attn_ln_weight", "mlp_ln_weight"):
        a, b = getattr(loaded.stacked_params, name), getattr(drawn.stacked_params, name)
        assert a.shape == b.shape and torch.equal(a, b), name
    assert torch.equal(loaded.lm_head.lm_head.weight, drawn.lm_head.lm_head.weight)
    assert torch.equal(loaded.model.embed_tokens.embed_tokens.weight, drawn.model.embed_tokens.embed_tokens.weight)
    assert torch.equal(loaded.model.rope_cos, drawn.model.rope_cos)
    assert loaded.stacked_kv_cache[0].shape == (2, 1, 32, TINY["num_key_value_heads"] // tp, 128)


# ---- on a GPU: the script end to end, and a recorded timing trace ---- #
@pytest.mark.gpu
def test_generate_script_runs_and_repeats_itself(capsys):
    argv = ["model=llama-1b", "layers=2", "ntok=8", "once", "prompt_len=6", "max_len_override=64"]
    first = main(parse_cli(argv)).cpu()
    out = capsys.readouterr().out
    assert "Tokens per second" in out and "Output ids" in out
    assert first.shape == (1, 8) and int(first.min()) >= 0 and int(first.max()) < 128256
    assert torch.equal(main(parse_cli(argv + ["sched=wave"])).cpu(), first), "greedy decoding is deterministic"


@pytest.mark.gpu
def test_recorded_trace_covers_every_instruction():
    from megakernels_b200 import trace
    from megakernels_b200.demos.latency.scheduler import LatencyScheduleOptions
    from tests.gpu_utils import make_pair, run_gpu_step

    cfg = LlamaConfig.llama_3_2_1b(num_hidden_layers=2, vocab_size=4096)
    opts = LatencyScheduleOptions(num_attention_partitions=2, coalesce_o_proj=True)
    cpu_model, _, _, sched = make_pair(cfg, 200, 150, options=opts)
    g = sched.globs
    st = run_gpu_step(sched, cpu_model.model.embed_tokens.embed_tokens.weight[5], 150, record_timings=True)
    assert st.code == 0
    ins, tim = g.instructions.cpu(), g.timings.cpu().to(torch.int64) & 0xFFFFFFFF
    real = ins[:, :, 0] != 0
    start, wait, done = tim[:, :, 0][real], tim[:, :, 1][real], tim[:, :, 4][real]
    assert bool((start > 0).all()), "every non-NoOp instruction has a consumer start stamp"
    # stamps are the low 32 bits of a nanosecond counter: compare modulo 2^32
    assert bool((((wait - start) & 0xFFFFFFFF) < 10**8).all()), "barrier wait ends after the start"
    assert bool((((done - wait) & 0xFFFFFFFF) < 10**8).all()), "instruction ends after its wait"
    assert int(tim[:, :, 0][~real].abs().sum()) == 0, "NoOps leave no stamps"
    summary = trace.summarize(g)
    names = set(summary["stats"])
    assert {"qkv_rope_append", "partial_attention", "attention_reduction", "o_proj_residual",
            "upgate_silu", "down_proj_residual", "lm_head"} <= names
    n_real = int(real.sum())
    assert sum(max(v[2] for v in d.values()) for d in summary["stats"].values()) == n_real
    assert 0 < summary["total_us"] < 50_000
    assert "kernel span" in trace.format_summary(summary, layers=(0, 1))
