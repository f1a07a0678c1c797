"""Host logic: the instruction stream must equal the reference's, word for word."""

import hashlib
import json

import pytest
import torch

from megakernels_b200.demos.latency.instructions import (
    AttentionReduction,
    DownProjResidual,
    LayerNorm_QKV_MatVecRopeAppend,
    LayerNormDoubleMatVecSiLU,
    O_ProjResidual,
    PartialAttention,
    RMS_LM_Head,
)
from megakernels_b200.demos.latency.scheduler import (
    LatencyScheduleBuilder,
    LatencyScheduleOptions,
)
from megakernels_b200.dispatch import make_schedule_builder
from megakernels_b200.instructions import NoOp
from megakernels_b200.llama import LlamaConfig, LlamaForCausalLM
from megakernels_b200.model_types import ExtraModelConfig
from megakernels_b200.scheduler import (
    assign_to_sms,
    serialize_and_pad,
    tensorize_instructions,
)
from megakernels_b200.utils import set_sm_count_override


def shape_model(cfg, tp_size=1, tp_rank=0, max_len=64):
    extra = ExtraModelConfig(
        interleave_rope=True, max_len_override=max_len, tp_size=tp_size, tp_rank=tp_rank
    )
    return LlamaForCausalLM.from_random(cfg, extra, device="cpu", draw_on="zeros")


def sha(t):
    return hashlib.sha256(t.contiguous().numpy().tobytes()).hexdigest()


@pytest.fixture(scope="module")
def model_1b():
    return shape_model(LlamaConfig.llama_3_2_1b())


@pytest.mark.parametrize("mode", ["rr", "zz", "wave", "dag"])
def test_1b_instruction_tensor_equals_reference(model_1b, golden_dir, mode):
    set_sm_count_override(148)
    golden = json.loads((golden_dir / "sched_1b.json").read_text())
    schedule = make_schedule_builder("latency").build(model_1b)
    schedule.globs.pos_id = 41
    assert len(schedule.get_linear_instructions()) == golden["num_instructions"]
    tensorize_instructions(schedule.globs, assign_to_sms(mode, schedule=schedule))
    t = schedule.globs.instructions
    assert list(t.shape) == golden["modes"][mode]["shape"]
    assert sha(t) == golden["modes"][mode]["sha256"]
    assert schedule.globs.timings.shape == (148, t.shape[1], 128)


def test_serialize_layouts():
    assert NoOp().serialize() == [0]
    assert LayerNorm_QKV_MatVecRopeAppend(3, 5, 9).serialize() == [1, 3, 5, 9]
    assert PartialAttention(2, 7, 4, 1).serialize() == [2, 2, 7, 4, 1]
    assert AttentionReduction(1, 8, 3, True, [0, 1, 2], None).serialize() == [
        3, 1, 8, 3, 1, 3, 0, 1, 2, 0,
    ]
    assert O_ProjResidual(0, 4, 5, 0).serialize() == [4, 0, 4, 5, 0]
    assert LayerNormDoubleMatVecSiLU(1, [3, 151]).serialize() == [5, 1, 2, 3, 151]
    assert DownProjResidual(9, 0, 3, 2).serialize() == [6, 9, 0, 3, 2]
    assert RMS_LM_Head(10, 20).serialize() == [7, 10, 20]
    assert len(serialize_and_pad(RMS_LM_Head(1, 2))) == 32
    with pytest.raises(AssertionError):
        serialize_and_pad(LayerNormDoubleMatVecSiLU(0, list(range(40))))


def covered_blocks(instructions, cls, layer):
    return [i for i in instructions if isinstance(i, cls) and getattr(i, "layer_idx", layer) == layer]


@pytest.mark.parametrize(
    "cfg_fn,tp",
    [
        (LlamaConfig.llama_3_2_1b, 1),
        (LlamaConfig.llama_3_1_8b, 1),
        (LlamaConfig.llama_3_1_70b, 2),
        (LlamaConfig.llama_3_1_70b, 4),
        (LlamaConfig.llama_3_1_70b, 8),
    ],
)
@pytest.mark.parametrize("tuned", [False, True])
def test_every_output_block_is_covered_exactly_once(cfg_fn, tp, tuned):
    """Shape-generic builder: each projection row block x column slice appears once."""
    set_sm_count_override(148)
    cfg = cfg_fn(num_hidden_layers=2, vocab_size=128256)
    model = shape_model(cfg, tp_size=tp, tp_rank=tp - 1)
    opts = LatencyScheduleOptions(
        num_attention_partitions=4 if tuned else 1, coalesce_o_proj=bool(tuned)
    )
    schedule = LatencyScheduleBuilder(opts).build(model)
    g = schedule.globs
    ins = schedule.get_linear_instructions()
    Hq, Hkv, D = g.num_attention_heads, g.num_kv_heads, g.head_dim
    for layer in range(2):
        qkv = sorted(b for i in covered_blocks(ins, LayerNorm_QKV_MatVecRopeAppend, layer) for b in i.block_indices())
        assert qkv == list(range((Hq + 2 * Hkv) * D // 16))
        up = sorted(b for i in covered_blocks(ins, LayerNormDoubleMatVecSiLU, layer) for b in i.block_idxs)
        assert up == list(range(g.intermediate_size // 16))
        assert all(len(i.serialize()) <= 32 for i in covered_blocks(ins, LayerNormDoubleMatVecSiLU, layer))
        for cls, splits in ((O_ProjResidual, g.num_o_proj_col_splits()), (DownProjResidual, g.num_down_proj_col_splits())):
            jobs = sorted(
                (i.reduction_block_idx, b)
                for i in covered_blocks(ins, cls, layer)
                for b in range(i.start_block_idx, i.end_block_idx)
            )
            assert jobs == [(c, b) for c in range(splits) for b in range(g.hidden_size // 16)]
        parts = covered_blocks(ins, PartialAttention, layer)
        assert len(parts) == Hkv * opts.num_attention_partitions
        reds = covered_blocks(ins, AttentionReduction, layer)
        assert len(reds) == (0 if not tuned else Hq // 4)
    head = sorted(b for i in ins if isinstance(i, RMS_LM_Head) for b in range(i.start_output_block_idx, i.end_output_block_idx))
    assert head == list(range(cfg.vocab_size // 16))
    th = g.barrier_thresholds()
    assert th["attn_waits_qkv_per_head"] == D // 16
    assert g.barriers.shape == (2, 10, Hq + 2 * Hkv)
    for mode in ("rr", "wave"):
        queues = assign_to_sms(mode, schedule=schedule)
        assert sum(len(q) for q in queues) == len(ins)


def test_1b_thresholds_are_the_reference_constants(model_1b):
    g = make_schedule_builder("latency").build(model_1b, layer_limit=1).globs
    assert g.barrier_thresholds() == {
        "qkv_waits_downproj": 512,
        "attn_waits_qkv_per_head": 4,
        "oproj_waits_attn": 32,
        "upgate_waits_oproj": 128,
        "downproj_waits_upgate": 128,
    }
    assert g.matvec_reduction_size == 2048
