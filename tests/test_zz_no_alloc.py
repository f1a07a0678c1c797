"""``mkb_launch_no_alloc`` against ``mkb_launch`` and the CPU oracle (collected last on purpose).

Some hosts of the decode kernel cannot allocate device memory while they run:
their memory plan is fixed before the first token, or every byte already
belongs to their own pool.  For them the library offers one entry point that
calls no allocator at all and keeps the split-KV attention scratch, the
residual accumulators and the error record in a static device array.  These
tests drive that entry point through the C ABI with the attention
intermediates set to NULL, on a schedule that really uses the scratch (several
attention partitions plus reductions), twice in a row, and compare every
output with the ordinary entry point and with the oracle on the same inputs.
The array keeps the previous call's contents, so the second call also shows
that nothing stale leaks into the result.  One test repeats this in a fresh
process where the no-alloc call is the very first thing the library does on
the device, with the error record left inside the static array as well.
"""

import subprocess
import sys
from pathlib import Path

import pytest
import torch

from megakernels_b200.demos.latency.scheduler import LatencyScheduleOptions
from megakernels_b200.llama import LlamaConfig
from oracle.llama_ref import assert_logits_parity
from tests.gpu_utils import interpreter, make_pair, rel_err, run_cpu_step, run_gpu_step
from tests.oracle_utils import seeded_tokens

pytestmark = pytest.mark.gpu

TOL = 2e-2  # the tolerance of the parity tests: max|a-b| / max|b|
PARTS, PREFILL = 5, 150
OUTPUTS = ("logits", "post_ln_rope_q", "attn_out", "silu_out")


def launch_no_alloc(g, hidden, pos, max_partials, own_status=True):
    mk = sys.modules["mk_llama"]
    g.hidden_states[:] = hidden.to(g.hidden_states.device)
    g.barriers.zero_()
    g.pos_id = pos
    L, B, T, Hkv, D = g.k_cache.shape
    status = torch.zeros(16, dtype=torch.int32, device=g.hidden_states.device) if own_status else None
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
        upgate_instructions_per_layer=g.upgate_instructions_per_layer,
    )
    return mk.sync_status(call, no_alloc=True)


def small_case():
    cfg = LlamaConfig.llama_3_2_1b(num_hidden_layers=2, vocab_size=4096)
    opts = LatencyScheduleOptions(num_attention_partitions=PARTS, coalesce_o_proj=True)
    return cfg, opts


def test_no_alloc_entry_point_matches_the_allocating_one():
    interpreter()
    cfg, opts = small_case()
    cpu_model, cpu_sched, model_a, sched_a = make_pair(cfg, PREFILL + 8, PREFILL, options=opts)
    _, _, model_b, sched_b = make_pair(cfg, PREFILL + 8, PREFILL, options=opts)
    embed = cpu_model.model.embed_tokens.embed_tokens.weight
    ga, gb = sched_a.globs, sched_b.globs
    for i, tok in enumerate(seeded_tokens(cfg.vocab_size, 2)):  # two calls in a row
        pos = PREFILL + i
        run_cpu_step(cpu_model, cpu_sched, embed[tok], pos)
        st = run_gpu_step(sched_a, embed[tok], pos)
        assert st.code == 0
        st = launch_no_alloc(gb, embed[tok], pos, max_partials=PARTS)
        assert st.code == 0
        # integer accumulation makes the two entry points agree exactly, not just within TOL
        for name in OUTPUTS:
            assert rel_err(getattr(gb, name), getattr(ga, name)) <= TOL, f"{name} at pos {pos}"
            assert torch.equal(getattr(gb, name), getattr(ga, name)), f"{name} at pos {pos}"
        assert torch.equal(gb.k_cache[:, 0, pos], ga.k_cache[:, 0, pos])
        assert torch.equal(gb.v_cache[:, 0, pos], ga.v_cache[:, 0, pos])
        assert torch.equal(gb.barriers, ga.barriers)
        assert_logits_parity(gb.logits, cpu_sched.globs.logits, f"no-alloc vs oracle, pos {pos}")


def fresh_process_body():
    """Runs in a child process: the no-alloc call is the library's first act on the device."""
    interpreter()  # loads the library; launches nothing
    cfg, opts = small_case()
    cpu_model, cpu_sched, model_a, sched_a = make_pair(cfg, PREFILL + 8, PREFILL, options=opts)
    _, _, model_b, sched_b = make_pair(cfg, PREFILL + 8, PREFILL, options=opts)
    embed = cpu_model.model.embed_tokens.embed_tokens.weight
    ga, gb = sched_a.globs, sched_b.globs
    for i, tok in enumerate(seeded_tokens(cfg.vocab_size, 2)):
        pos = PREFILL + i
        # error record inside the static array too (status=None), read back without allocating
        st = launch_no_alloc(gb, embed[tok], pos, max_partials=PARTS, own_status=False)
        assert st.code == 0
        run_cpu_step(cpu_model, cpu_sched, embed[tok], pos)
        assert_logits_parity(gb.logits, cpu_sched.globs.logits, f"fresh process vs oracle, pos {pos}")
        st = run_gpu_step(sched_a, embed[tok], pos)  # only now the allocating entry point
        assert st.code == 0
        for name in OUTPUTS:
            assert torch.equal(getattr(gb, name), getattr(ga, name)), f"{name} at pos {pos}"
    print("FRESH-PROCESS-OK")


def test_no_alloc_entry_point_as_first_call_in_a_fresh_process():
    root = Path(__file__).resolve().parent.parent
    code = (
        "import sys; sys.path.insert(0, %r)\n"
        "import torch\n"
        "from megakernels_b200.utils import set_sm_count_override\n"
        "set_sm_count_override(torch.cuda.get_device_properties(0).multi_processor_count)\n"
        "from tests.test_zz_no_alloc import fresh_process_body\n"
        "fresh_process_body()\n"
    ) % str(root)
    res = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0 and "FRESH-PROCESS-OK" in res.stdout, res.stdout[-2000:] + res.stderr[-4000:]


def test_no_alloc_entry_point_rejects_oversized_scratch():
    interpreter()
    mk = sys.modules["mk_llama"]
    cfg = LlamaConfig.llama_3_2_1b(num_hidden_layers=1, vocab_size=4096)
    _, _, _, sched = make_pair(cfg, 64, 8)
    with pytest.raises(mk.MegakernelError) as err:
        launch_no_alloc(sched.globs, torch.zeros(cfg.hidden_size, dtype=torch.bfloat16), 8, max_partials=148)
    assert "MKB_ERR_UNSUPPORTED" in str(err.value) and "MKB_NO_ALLOC_SCRATCH_BYTES" in str(err.value)
