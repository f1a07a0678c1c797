"""Pin the checker's split-KV solvers to scaled-dot-product attention (CPU).

The reference ships `partial_attention` and `attention_reduction` solvers
(demos/latency/python_vm.py:277-393) but never schedules more than one partition
(its builder asserts `skip_attn_reduction`, demos/latency/scheduler.py:276-277), so its
golden outputs cover `num_partials == 1` only.  Here hand-built instruction lists with
several partitions - a flat terminal reduction and a two-level tree through non-terminal
reductions - must reproduce attention over the whole cache.
"""

import math

import pytest
import torch
import torch.nn.functional as F

from megakernels_b200.demos.latency.instructions import AttentionReduction, PartialAttention
from megakernels_b200.demos.latency.scheduler import LatencyScheduleOptions
from megakernels_b200.llama import LlamaConfig
from oracle.python_vm import attention_reduction, partial_attention
from tests.oracle_utils import build_model, build_schedule, fill_kv


def setup(num_partials, seq_len, shape="1b"):
    cfg = (LlamaConfig.llama_3_2_1b if shape == "1b" else LlamaConfig.llama_3_1_8b)(
        num_hidden_layers=1, vocab_size=4096
    )
    model = build_model(cfg, seq_len + 4)
    fill_kv(model, seq_len, poison=True)
    opts = LatencyScheduleOptions(num_attention_partitions=max(2, num_partials))
    g = build_schedule(model, opts, layer_limit=1).globs
    gen = torch.Generator().manual_seed(5)
    g.post_ln_rope_q[:] = torch.randn(g.post_ln_rope_q.shape, generator=gen).to(g.post_ln_rope_q.dtype)
    g.pos_id = seq_len - 1
    g.barriers[0, 0, :] = g.barrier_thresholds()["attn_waits_qkv_per_head"]  # the QKV op is done
    return cfg, g


def sdpa(g, cfg):
    n = g.pos_id + 1
    q = g.post_ln_rope_q.view(1, g.num_attention_heads, 1, cfg.head_dim).float()
    k = g.k_cache[0, :, :n].transpose(1, 2).float()
    v = g.v_cache[0, :, :n].transpose(1, 2).float()
    out = F.scaled_dot_product_attention(q, k, v, is_causal=False, enable_gqa=True)
    return out.reshape(-1)


@pytest.mark.parametrize("shape,num_partials,seq_len", [("1b", 1, 40), ("1b", 4, 333), ("1b", 7, 100), ("8b", 3, 257), ("1b", 6, 17)])
def test_partials_and_terminal_reduction_equal_full_attention(shape, num_partials, seq_len):
    cfg, g = setup(num_partials, seq_len, shape)
    for kv in range(g.num_kv_heads):
        for p in range(num_partials):
            partial_attention(g, PartialAttention(0, kv, num_partials, p))
    assert int(g.barriers[0, 1, : g.num_attention_heads].min()) == num_partials
    for h0 in range(0, g.num_attention_heads, g.attn_reduction_size):
        attention_reduction(g, AttentionReduction(0, h0, num_partials, True, list(range(num_partials)), None))
    assert int(g.barriers[0, 2, 0]) == g.num_attention_heads
    want = sdpa(g, cfg)
    err = (g.attn_out.float() - want).abs().max() / want.abs().max()
    assert err <= 1e-2, err  # attn_out is bf16: one rounding of an fp32 result


def test_two_level_reduction_tree_equals_full_attention():
    """Non-terminal reductions write merged (O, LSE) pairs that a later reduction consumes."""
    num_partials, seq_len = 6, 500
    cfg, g = setup(num_partials, seq_len)
    for kv in range(g.num_kv_heads):
        for p in range(num_partials):
            partial_attention(g, PartialAttention(0, kv, num_partials, p))
    for h0 in range(0, g.num_attention_heads, g.attn_reduction_size):
        # merge {0,1,2} into slot 6 and {3,4,5} into slot 7, then those two terminally; each
        # non-terminal reduction counts as one more arrival on the partial-attention row
        attention_reduction(g, AttentionReduction(0, h0, num_partials, False, [0, 1, 2], 6))
        attention_reduction(g, AttentionReduction(0, h0, num_partials + 1, False, [3, 4, 5], 7))
        attention_reduction(g, AttentionReduction(0, h0, num_partials + 2, True, [6, 7], None))
    want = sdpa(g, cfg)
    err = (g.attn_out.float() - want).abs().max() / want.abs().max()
    assert err <= 1e-2, err
    lse = g.attn_lse_intermediates[:, 6]
    assert bool(torch.isfinite(lse).all()) and not math.isnan(float(lse.sum()))


@pytest.mark.parametrize("shape,partitions,prefill", [("1b", 4, 90), ("8b", 3, 70)])
def test_merge_in_last_partial_equals_separate_reduction(shape, partitions, prefill):
    """Schedules without AttentionReduction instructions (`merge_in_last_partial`: the partial of a
    KV head that arrives last merges the rows) leave the same logits, bit for bit, as partials +
    terminal reductions, and the same o-proj barrier count."""
    from oracle.python_vm import PyVM_Interpreter

    cfg = (LlamaConfig.llama_3_2_1b if shape == "1b" else LlamaConfig.llama_3_1_8b)(
        num_hidden_layers=2, vocab_size=4096
    )
    logits = []
    for merge in (False, True):
        model = build_model(cfg, prefill + 4)
        fill_kv(model, prefill, poison=True)
        opts = LatencyScheduleOptions(num_attention_partitions=partitions, coalesce_o_proj=True,
                                      merge_in_last_partial=merge)
        sched = build_schedule(model, opts)
        g = sched.globs
        ops = [type(i).__name__ for i in sched.get_linear_instructions()]
        assert ("AttentionReduction" in ops) != merge
        g.hidden_states[:] = model.model.embed_tokens.embed_tokens.weight[11]
        g.pos_id = prefill
        PyVM_Interpreter().interpret(g, sched.get_linear_instructions())
        assert int(g.barriers[:, 2, 0].sum()) == 2 * g.num_attention_heads
        logits.append(g.logits.clone())
    assert torch.equal(logits[0], logits[1])
