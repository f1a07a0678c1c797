"""``mkb_launch_no_alloc`` against ``mkb_launch`` (collected last on purpose).

Some hosts of the decode kernel cannot allocate device memory while they run:
their memory plan is fixed before the first token, or every byte already
belongs to their own pool.  For them the library offers one entry point that
calls no allocator at all and keeps the split-KV attention scratch and the
error record in a static device array.  This test drives that entry point
through the C ABI with the attention intermediates set to NULL, on a schedule
that really uses the scratch (several attention partitions plus reductions),
twice in a row, and compares every output with the ordinary entry point on
the same inputs.  The array keeps the previous call's contents, so the second
call also shows that nothing stale leaks into the result.
"""

import sys

import pytest
import torch

from megakernels_b200.demos.latency.scheduler import LatencyScheduleOptions
from megakernels_b200.llama import LlamaConfig
from tests.gpu_utils import interpreter, make_pair, rel_err, run_gpu_step
from tests.oracle_utils import seeded_tokens

pytestmark = pytest.mark.gpu

TOL = 2e-2  # the tolerance of the parity tests: max|a-b| / max|b|


def launch_no_alloc(g, hidden, pos, max_partials):
    mk = sys.modules["mk_llama"]
    g.hidden_states[:] = hidden.to(g.hidden_states.device)
    g.barriers.zero_()
    g.pos_id = pos
    L, B, T, Hkv, D = g.k_cache.shape
    status = torch.zeros(16, dtype=torch.int32, device=g.hidden_states.device)
    call = mk.mk_llama_no_alloc(
        g.barriers, g.instructions, g.timings,
        g.qkv_proj_weights, g.attn_ln_weights, g.o_proj_weights, g.mlp_ln_weights,
        g.up_proj_weights, g.gate_proj_weights, g.down_proj_weights,
        g.lm_head_norm_weights, g.lm_head_weights,
        g.k_cache.view(L * B, T, Hkv, D), g.v_cache.view(L * B, T, Hkv, D),
        g.rope_cos, g.rope_sin,
        g.hidden_states, g.post_ln_rope_q, g.attn_out,
        None, None,  # the attention scratch is the library's static array
        g.silu_out, g.logits,
        g.pos_id, g.attn_scale, g.rms_norm_eps, g.skip_attn_reduction,
        matvec_reduction_size=g.matvec_reduction_size,
        status=status,
        num_attention_heads=g.num_attention_heads,
        max_partials=max_partials,
    )
    return mk.sync_status(call)


def test_no_alloc_entry_point_matches_the_allocating_one():
    interpreter()
    cfg = LlamaConfig.llama_3_2_1b(num_hidden_layers=2, vocab_size=4096)
    parts = 5
    opts = LatencyScheduleOptions(num_attention_partitions=parts, coalesce_o_proj=True)
    prefill = 150
    _, _, model_a, sched_a = make_pair(cfg, prefill + 8, prefill, options=opts)
    _, _, model_b, sched_b = make_pair(cfg, prefill + 8, prefill, options=opts)
    embed = model_a.model.embed_tokens.embed_tokens.weight.cpu()
    ga, gb = sched_a.globs, sched_b.globs
    for i, tok in enumerate(seeded_tokens(cfg.vocab_size, 2)):  # two calls in a row
        pos = prefill + i
        st = run_gpu_step(sched_a, embed[tok], pos)
        assert st.code == 0
        st = launch_no_alloc(gb, embed[tok], pos, max_partials=parts)
        assert st.code == 0
        for name in ("logits", "hidden_states", "post_ln_rope_q", "attn_out", "silu_out"):
            assert rel_err(getattr(gb, name), getattr(ga, name)) <= TOL, f"{name} at pos {pos}"
        assert rel_err(gb.k_cache[:, 0, pos], ga.k_cache[:, 0, pos]) <= TOL
        assert rel_err(gb.v_cache[:, 0, pos], ga.v_cache[:, 0, pos]) <= TOL
        assert torch.equal(gb.barriers, ga.barriers)
        assert int(gb.logits.argmax()) == int(ga.logits.argmax())


def test_no_alloc_entry_point_rejects_oversized_scratch():
    interpreter()
    mk = sys.modules["mk_llama"]
    cfg = LlamaConfig.llama_3_2_1b(num_hidden_layers=1, vocab_size=4096)
    _, _, _, sched = make_pair(cfg, 64, 8)
    with pytest.raises(mk.MegakernelError) as err:
        launch_no_alloc(sched.globs, torch.zeros(cfg.hidden_size, dtype=torch.bfloat16), 8, max_partials=148)
    assert "MKB_ERR_UNSUPPORTED" in str(err.value) and "MKB_NO_ALLOC_SCRATCH_BYTES" in str(err.value)
