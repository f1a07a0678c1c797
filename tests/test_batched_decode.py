"""Batched decode: B independent sequences per launch, ragged lengths.

The reference has no kernel for this (its latency kernel decodes one sequence; its batched
instruction set needs batches that are multiples of 128, demos/throughput/instructions.py:30-31;
its torch path shares one length across the batch, llama.py:121-130), so the oracle is B
independent single-sequence runs of the pinned torch restatement on the same weights.
"""

import pytest
import torch

from megakernels_b200.demos.latency.instructions import (
    AttentionReduction,
    PartialAttention,
    RMS_Norm,
)
from megakernels_b200.demos.latency.scheduler import LatencyScheduleBuilder, LatencyScheduleOptions
from megakernels_b200.llama import LlamaConfig, LlamaForCausalLM
from megakernels_b200.model_types import ExtraModelConfig
from megakernels_b200.scheduler import assign_to_sms, serialize_and_pad, tensorize_instructions
from megakernels_b200.utils import set_sm_count_override


def batched_schedule(cfg, batch, parts, max_len, device="cpu", draw_on="zeros"):
    extra = ExtraModelConfig(interleave_rope=True, max_len_override=max_len, max_batch_size=batch)
    model = LlamaForCausalLM.from_random(cfg, extra, device=device, seed=0, draw_on=draw_on)
    opts = LatencyScheduleOptions(num_attention_partitions=parts, coalesce_o_proj=True, batch_size=batch)
    schedule = LatencyScheduleBuilder(opts).build(model)
    tensorize_instructions(schedule.globs, assign_to_sms("rr", schedule=schedule))
    return model, schedule


def test_single_sequence_words_are_unchanged_by_the_batch_fields():
    """A sequence index of 0 lands in the zero padding: the padded words equal the reference's."""
    assert serialize_and_pad(PartialAttention(3, 5, 4, 2))[:7] == [2, 3, 5, 4, 2, 0, 0]
    assert serialize_and_pad(PartialAttention(3, 5, 4, 2, 6))[:7] == [2, 3, 5, 4, 2, 6, 0]
    words = serialize_and_pad(AttentionReduction(1, 8, 3, True, [0, 1, 2], None, 5))
    assert words[:11] == [3, 1, 8, 3, 1, 3, 0, 1, 2, 0, 5]
    assert serialize_and_pad(RMS_Norm(7, 1, 3))[:5] == [9, 7, 1, 3, 0]


def test_more_than_eight_sequences_schedule_blocks_of_128_rows():
    """The tcgen05 build multiplies blocks of 128 weight rows: block indices, counts and barrier
    thresholds of the schedule follow."""
    set_sm_count_override(148)
    cfg = LlamaConfig.llama_3_1_8b(num_hidden_layers=1, vocab_size=4096)
    _, schedule = batched_schedule(cfg, 16, 1, 64)
    g = schedule.globs
    assert (g.qkv_block_size, g.o_proj_block_size, g.up_gate_proj_block_size, g.down_proj_block_size,
            g.lm_head_block_size) == (128,) * 5
    th = g.barrier_thresholds()
    assert th["attn_waits_qkv_per_head"] == 1 and th["downproj_waits_upgate"] == 2048 // 128
    assert th["qkv_waits_downproj"] == (4096 // 128) * 7 and th["upgate_waits_oproj"] == (4096 // 128) * 2
    ins = schedule.get_linear_instructions()
    qkv = sorted(b for i in ins if type(i).__name__ == "LayerNorm_QKV_MatVecRopeAppend" for b in i.block_indices())
    assert qkv == list(range((32 + 16) * 128 // 128))
    up = sorted(b for i in ins if type(i).__name__ == "LayerNormDoubleMatVecSiLU" for b in i.block_idxs)
    assert up == list(range(14336 // 128))
    assert g.barriers.shape[2] >= 16 * 32


@pytest.mark.parametrize("batch,parts", [(4, 1), (8, 3)])
def test_batched_schedule_covers_every_sequence(batch, parts):
    set_sm_count_override(148)
    cfg = LlamaConfig.llama_3_1_8b(num_hidden_layers=2, vocab_size=4096)
    _, schedule = batched_schedule(cfg, batch, parts, 64)
    g = schedule.globs
    ins = schedule.get_linear_instructions()
    assert g.batch_size == batch and g.hidden_states.shape == (batch, cfg.hidden_size)
    assert g.residual_acc.shape == (batch, cfg.hidden_size) and g.normed_states.shape == (batch, cfg.hidden_size)
    assert g.barriers.shape[2] >= batch * cfg.num_attention_heads
    for layer in range(2):
        attn = {(i.batch_idx, i.kv_head_idx, i.partial_idx) for i in ins if isinstance(i, PartialAttention) and i.layer_idx == layer}
        assert attn == {(b, kv, p) for b in range(batch) for kv in range(cfg.num_key_value_heads) for p in range(parts)}
        reds = {(i.batch_idx, i.head_start_idx) for i in ins if isinstance(i, AttentionReduction) and i.layer_idx == layer}
        want = {(b, h) for b in range(batch) for h in range(0, cfg.num_attention_heads, 4)} if parts > 1 else set()
        assert reds == want
        norms = {(i.which, i.batch_idx) for i in ins if isinstance(i, RMS_Norm) and i.layer_idx == layer}
        assert norms >= {(w, b) for w in (0, 1) for b in range(batch)}
    assert sum(isinstance(i, RMS_Norm) and i.which == 2 for i in ins) == batch
    assert g.upgate_instructions_per_layer == 0
    # topological order: a sequence's attention follows the layer's QKV and precedes its o-proj
    order = [type(i).__name__ for i in ins if getattr(i, "layer_idx", None) == 0]
    assert order.index("PartialAttention") > order.index("LayerNorm_QKV_MatVecRopeAppend")
    assert order.index("O_ProjResidual") > len(order) - 1 - order[::-1].index("PartialAttention")


@pytest.mark.gpu
@pytest.mark.parametrize(
    "shape,batch,parts,merge",
    # up to 8 sequences: mma.sync with the sequences as B-operand columns; more: tcgen05 GEMMs
    # (128-row blocks, head_dim 128 only), incl. a batch that is not a multiple of the MMA's N step;
    # merge: no reduction instructions, the last partial of a (sequence, KV head) merges the rows
    [("8b", 4, 3, False), ("8b", 8, 1, False), ("1b", 5, 2, False), ("1b", 2, 4, False), ("8b", 16, 1, False),
     ("8b", 40, 2, False), ("8b", 64, 1, False), ("8b", 4, 3, True), ("1b", 5, 2, True), ("8b", 40, 2, True)],
)
def test_batched_decode_matches_independent_sequences(shape, batch, parts, merge):
    from megakernels_b200.generators import MK_Generator
    from oracle.llama_ref import TorchReferenceModel, assert_logits_parity
    from tests.gpu_utils import interpreter

    dev = "cuda:0"
    cfg = (LlamaConfig.llama_3_1_8b if shape == "8b" else LlamaConfig.llama_3_2_1b)(num_hidden_layers=2, vocab_size=4096)
    lens = torch.randint(5, 300, (batch,), generator=torch.Generator().manual_seed(4)).tolist()
    max_len = max(lens) + 8
    extra = ExtraModelConfig(interleave_rope=True, max_len_override=max_len, max_batch_size=batch)
    model = LlamaForCausalLM.from_random(cfg, extra, device=dev, seed=0, draw_on="device")
    gen = torch.Generator(device=dev).manual_seed(2)
    for c in model.stacked_kv_cache:  # N(0,1) prefix per sequence, poison beyond it
        c.copy_((torch.randn(c.shape, generator=gen, device=dev) * 100).to(c.dtype))
        for b, n in enumerate(lens):
            c[:, b, :n] = torch.randn(c[:, b, :n].shape, generator=gen, device=dev).to(c.dtype)
    # one copy of the weights on the host, one KV cache per sequence swapped in for its run
    ref = TorchReferenceModel(model, kv_len=max_len)
    caches = [tuple(c[:, b : b + 1].cpu().clone() for c in model.stacked_kv_cache) for b in range(batch)]
    opts = LatencyScheduleOptions(num_attention_partitions=parts, coalesce_o_proj=True, batch_size=batch,
                                  merge_in_last_partial=merge)
    schedule = LatencyScheduleBuilder(opts).build(model)
    tensorize_instructions(schedule.globs, assign_to_sms("rr", schedule=schedule))
    g = schedule.globs
    assert any(isinstance(i, AttentionReduction) for i in schedule.get_linear_instructions()) == (parts > 1 and not merge)
    mk = MK_Generator(model, interpreter(), schedule)
    ids = torch.randint(0, cfg.vocab_size, (3, batch), generator=torch.Generator().manual_seed(3))
    for step in range(3):
        pos = [n + step for n in lens]
        out = mk.run(ids[step].view(batch, 1).to(dev), pos)
        mk.check()
        assert out.shape == (batch,)
        for b in range(batch):
            ref.k_cache, ref.v_cache = caches[b]
            # 2e-2 / 0.999 as everywhere (the bounds never go below the stated values); with so
            # many (sequence, step) samples some top-2 pairs are one bf16 step apart, and for
            # those the float32 restatement says whether the oracle itself can tell them apart
            exact = ref.decode_token_exact(int(ids[step, b]), pos[b])
            want = ref.decode_token(int(ids[step, b]), pos[b])
            assert_logits_parity(g.logits[b], want, f"step {step}, sequence {b} at position {pos[b]}", exact=exact)
            assert int(out[b]) == int(torch.argmax(g.logits[b])), f"fused argmax, sequence {b}"
            # the appended K/V row, and nothing beyond it
            assert torch.equal(g.k_cache[:, b, pos[b] + 1 :].cpu(), ref.k_cache[:, 0, pos[b] + 1 :])
