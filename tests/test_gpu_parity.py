"""GPU parity: the CUDA megakernel (through the C ABI) against the CPU oracle
and against the golden vectors produced by the reference itself.

Tolerances (bf16): per-step logits max|a-b|/max|b| <= 2e-2 and cosine >= 0.999;
greedy argmax equal wherever the oracle's top-2 margin exceeds 1e-2.  Integer
state (barrier counters) must match exactly.
"""

import sys

import pytest
import torch

from megakernels_b200.demos.latency.scheduler import LatencyScheduleOptions
from megakernels_b200.llama import LlamaConfig
from oracle.llama_ref import parity_metrics, TorchReferenceModel, assert_logits_parity
from tests.gpu_utils import (
    compare_globals,
    tensor_of,
    interpreter,
    make_pair,
    rel_err,
    run_cpu_step,
    run_gpu_step,
)
from tests.oracle_utils import config_from_fixture, load_fixture, seeded_tokens

pytestmark = pytest.mark.gpu


def small_1b(**kw):
    base = dict(num_hidden_layers=2, vocab_size=4096)
    base.update(kw)
    return LlamaConfig.llama_3_2_1b(**base)


def small_8b(**kw):
    base = dict(num_hidden_layers=2, vocab_size=4096)
    base.update(kw)
    return LlamaConfig.llama_3_1_8b(**base)


def small_70b(**kw):
    base = dict(num_hidden_layers=1, vocab_size=4096)
    base.update(kw)
    return LlamaConfig.llama_3_1_70b(**base)


def test_library_reports_b200_geometry():
    interpreter()
    mk = sys.modules["mk_llama"]
    lib = mk.load_library()
    assert lib.mkb_sm_count() == torch.cuda.get_device_properties(0).multi_processor_count
    assert lib.mkb_block_threads() == 576
    assert lib.mkb_smem_bytes() <= 227 * 1024


def test_all_noop_queue_runs_clean():
    _, _, gpu_model, gpu_sched = make_pair(small_1b(), 64, 8)
    g = gpu_sched.globs
    g.instructions.zero_()
    before = g.logits.clone()
    st = run_gpu_step(gpu_sched, torch.zeros_like(g.hidden_states).cpu(), 8)
    assert st.code == 0
    assert torch.equal(g.logits, before)
    assert int(g.barriers.abs().sum()) == 0


@pytest.mark.parametrize("stop_after_op", ["qkv", "partial", "oproj", "upgate", "downproj"])
@pytest.mark.parametrize("shape", ["1b", "8b"])
def test_each_op_against_oracle(shape, stop_after_op):
    """diff_test-style bisecting: run the stream up to one op on both sides."""
    cfg = small_1b() if shape == "1b" else small_8b()
    prefill = 37
    cpu_model, cpu_sched, gpu_model, gpu_sched = make_pair(
        cfg, 128, prefill, stop_after_op=stop_after_op, layer_limit=1
    )
    gen = torch.Generator().manual_seed(11)
    hidden = torch.randn(cfg.hidden_size, generator=gen).to(torch.bfloat16)
    run_cpu_step(cpu_model, cpu_sched, hidden, prefill)
    st = run_gpu_step(gpu_sched, hidden, prefill)
    assert st.code == 0
    names = {
        "qkv": ("post_ln_rope_q",),
        "partial": ("post_ln_rope_q", "attn_out"),
        "oproj": ("attn_out", "hidden_states"),
        "upgate": ("hidden_states", "silu_out"),
        "downproj": ("hidden_states", "silu_out"),
    }[stop_after_op]
    compare_globals(gpu_sched.globs, cpu_sched.globs, prefill, names=names)
    assert torch.equal(gpu_sched.globs.barriers.cpu(), cpu_sched.globs.barriers)
    # nothing may be written beyond the appended position
    assert torch.equal(
        gpu_sched.globs.k_cache[:, :, prefill + 1 :].cpu(), cpu_sched.globs.k_cache[:, :, prefill + 1 :]
    )


@pytest.mark.parametrize("sched", ["rr", "zz", "wave", "dag"])
def test_golden_1b_widths_all_assignments(golden_dir, sched):
    """Three teacher-forced steps against the reference VM's own logits."""
    fx = load_fixture(golden_dir / "pyvm_1b_w2.pt")
    cfg = config_from_fixture(fx)
    cpu_model, cpu_sched, gpu_model, gpu_sched = make_pair(
        cfg, fx["max_len"], fx["prefill"], sched=sched, poison=True
    )
    embed = cpu_model.model.embed_tokens.embed_tokens.weight
    for step, tstep in zip(fx["pyvm_steps"], fx["torch_steps"]):
        st = run_gpu_step(gpu_sched, embed[step["token"]], step["pos"])
        assert st.code == 0
        g = gpu_sched.globs
        assert_logits_parity(g.logits, step["logits"], f"vs reference VM, pos {step['pos']}")
        assert_logits_parity(g.logits, tstep["logits"], f"vs reference torch, pos {step['pos']}")
        for name in ("hidden_states", "post_ln_rope_q", "attn_out", "silu_out"):
            assert rel_err(tensor_of(g, name), step[name]) <= 2e-2, name
        assert rel_err(g.k_cache[:, 0, step["pos"]], step["k_new"]) <= 2e-2
        assert rel_err(g.v_cache[:, 0, step["pos"]], step["v_new"]) <= 2e-2
        ours, ref = g.barriers.cpu().clone(), step["barriers"].clone()
        assert torch.equal(ours[:, 4].sum(-1), ref[:, 4].sum(-1))
        ours[:, 4] = 0
        ref[:, 4] = 0
        ours[:, 8] = 0  # residual-read arrivals: no counterpart in the reference
        assert torch.equal(ours, ref)


def test_golden_8b_widths(golden_dir):
    fx = load_fixture(golden_dir / "torch_8b_w1.pt")
    cfg = config_from_fixture(fx)
    cpu_model, cpu_sched, gpu_model, gpu_sched = make_pair(cfg, fx["max_len"], fx["prefill"])
    embed = cpu_model.model.embed_tokens.embed_tokens.weight
    for step in fx["torch_steps"]:
        st = run_gpu_step(gpu_sched, embed[step["token"]], step["pos"])
        assert st.code == 0
        assert_logits_parity(gpu_sched.globs.logits, step["logits"], f"pos {step['pos']}")
        assert rel_err(gpu_sched.globs.k_cache[:, 0, step["pos"]], step["k_new"]) <= 2e-2


@pytest.mark.parametrize(
    "shape,prefill,partitions,merge",
    [("1b", 5, 1, False), ("1b", 300, 4, False), ("1b", 1000, 18, False), ("8b", 130, 3, False),
     ("8b", 700, 16, False), ("1b", 17, 6, False),
     ("1b", 300, 4, True), ("1b", 1000, 18, True), ("8b", 130, 3, True), ("8b", 700, 16, True),
     ("1b", 17, 6, True), ("8b", 1500, 24, True)],
)
def test_split_kv_attention_and_reduction(shape, prefill, partitions, merge):
    """Multi-partition schedules (partials + reduction instructions, or the last partial of a KV
    head merging the rows) and empty partitions."""
    cfg = small_1b(num_hidden_layers=1) if shape == "1b" else small_8b(num_hidden_layers=1)
    opts = LatencyScheduleOptions(num_attention_partitions=partitions, coalesce_o_proj=True,
                                  merge_in_last_partial=merge)
    cpu_model, cpu_sched, gpu_model, gpu_sched = make_pair(cfg, prefill + 8, prefill, options=opts)
    embed = cpu_model.model.embed_tokens.embed_tokens.weight
    # the multi-partition VM solvers are this repository's generalisation; the torch path
    # (attention over the whole cache in one call) is pinned to the reference, so it is the
    # anchor for both the VM and the kernel here
    ref = TorchReferenceModel(cpu_model)
    ref.load_kv(*cpu_model.stacked_kv_cache)
    for i, tok in enumerate(seeded_tokens(cfg.vocab_size, 2)):
        pos = prefill + i
        run_cpu_step(cpu_model, cpu_sched, embed[tok], pos)
        st = run_gpu_step(gpu_sched, embed[tok], pos)
        assert st.code == 0
        compare_globals(gpu_sched.globs, cpu_sched.globs, pos)
        assert_logits_parity(gpu_sched.globs.logits, cpu_sched.globs.logits, f"pos {pos}")
        want = ref.decode_token(tok, pos)
        assert_logits_parity(cpu_sched.globs.logits, want, f"VM vs torch path, pos {pos}")
        assert_logits_parity(gpu_sched.globs.logits, want, f"kernel vs torch path, pos {pos}")
        assert torch.equal(gpu_sched.globs.barriers.cpu(), cpu_sched.globs.barriers)


def test_70b_widths_one_layer():
    """hidden 8192 (two chunks per thread) and GQA ratio 8."""
    cfg = small_70b()
    opts = LatencyScheduleOptions(num_attention_partitions=2, coalesce_o_proj=True)
    cpu_model, cpu_sched, gpu_model, gpu_sched = make_pair(cfg, 200, 150, options=opts)
    embed = cpu_model.model.embed_tokens.embed_tokens.weight
    run_cpu_step(cpu_model, cpu_sched, embed[77], 150)
    st = run_gpu_step(gpu_sched, embed[77], 150)
    assert st.code == 0
    compare_globals(gpu_sched.globs, cpu_sched.globs, 150)
    assert_logits_parity(gpu_sched.globs.logits, cpu_sched.globs.logits, "70b widths")


@pytest.mark.parametrize("width,tp", [("70b", 2), ("70b", 8), ("8b", 2), ("8b", 4), ("8b", 8)])
def test_tensor_parallel_shard_shapes(width, tp):
    """One rank's shard, run on its own: input-column slices of 2048 (70B widths, tp 2), 512
    (70B tp 8, 8B tp 4), 1024 (8B tp 2) and 256 (8B tp 8: fewer heads than down-proj slices)."""
    from tests.oracle_utils import build_model, build_schedule, fill_kv
    from megakernels_b200.scheduler import assign_to_sms, tensorize_instructions

    cfg = small_70b() if width == "70b" else small_8b(num_hidden_layers=1)
    opts = LatencyScheduleOptions(num_attention_partitions=1, coalesce_o_proj=True)
    cpu_model = build_model(cfg, 64, device="cpu", tp_size=tp, tp_rank=tp - 1)
    fill_kv(cpu_model, 40, poison=True)
    gpu_model = build_model(cfg, 64, device="cuda:0", tp_size=tp, tp_rank=tp - 1)
    for a, b in zip(gpu_model.stacked_kv_cache, cpu_model.stacked_kv_cache):
        a.copy_(b)
    cpu_sched, gpu_sched = build_schedule(cpu_model, opts), build_schedule(gpu_model, opts)
    for s in (cpu_sched, gpu_sched):
        tensorize_instructions(s.globs, assign_to_sms("wave", schedule=s))
    embed = cpu_model.model.embed_tokens.embed_tokens.weight
    run_cpu_step(cpu_model, cpu_sched, embed[5], 40)
    st = run_gpu_step(gpu_sched, embed[5], 40)
    assert st.code == 0
    compare_globals(gpu_sched.globs, cpu_sched.globs, 40)
    assert torch.equal(gpu_sched.globs.barriers.cpu(), cpu_sched.globs.barriers)


def test_bounded_wait_reports_instead_of_hanging():
    """A counter nothing increments: the wait gives up, the status says where."""
    cfg = small_1b(num_hidden_layers=1)
    _, _, gpu_model, gpu_sched = make_pair(cfg, 64, 8, stop_after_op="oproj", layer_limit=1)
    g = gpu_sched.globs
    # keep only the O-proj instructions: their attention producers never run
    ins = g.instructions
    keep = ins[:, :, 0] == 4
    ins[~keep] = 0
    mk = sys.modules.get("mk_llama")
    with pytest.raises(Exception) as err:
        run_gpu_step(gpu_sched, torch.zeros(cfg.hidden_size, dtype=torch.bfloat16), 8, wait_timeout_ms=50)
    assert "MKB_ERR_DEVICE_TIMEOUT" in str(err.value)
    status = err.value.status
    assert status.opcode == 4 and status.role == 1
    assert list(status.detail)[:3] == [0, 2, 0]  # layer 0, attention-reduction row, slot 0
    # the context is still usable and the next launch runs clean
    _, _, _, sched2 = make_pair(cfg, 64, 8)
    st = run_gpu_step(sched2, torch.zeros(cfg.hidden_size, dtype=torch.bfloat16), 8)
    assert st.code == 0


def test_host_validation_rejects_bad_arguments():
    cfg = small_1b(num_hidden_layers=1)
    _, _, gpu_model, gpu_sched = make_pair(cfg, 64, 8)
    g = gpu_sched.globs
    mk = sys.modules["mk_llama"]
    g.pos_id = 64  # beyond the KV cache
    with pytest.raises(ValueError):
        interpreter().interpret(g)
    g.pos_id = 8
    bad = torch.zeros(148 + 1000, 1, 32, dtype=torch.int32, device="cuda:0")
    good = g.instructions
    g.instructions = bad
    with pytest.raises(mk.MegakernelError) as err:
        interpreter().interpret(g)
    assert "co-resident" in str(err.value)
    g.instructions = good


def test_greedy_generation_matches_oracle():
    """MK_Generator end to end: prefill + greedy decode vs the torch oracle."""
    from megakernels_b200.generators import MK_Generator

    cfg = small_1b()
    cpu_model, cpu_sched, gpu_model, gpu_sched = make_pair(cfg, 64, 0, poison=False)
    prompt = torch.tensor(seeded_tokens(cfg.vocab_size, 6, seed=1))
    ref = TorchReferenceModel(cpu_model)
    gen = MK_Generator(gpu_model, interpreter(), gpu_sched)
    first = gen.prefill(prompt.cuda())
    ntok = 8
    out = torch.zeros(1, ntok, dtype=torch.long, device="cuda:0")
    out[:, 0] = first
    gen.generate(out, prompt_len=prompt.numel(), ntok=ntok - 1)
    gen.check()
    got = out.cpu()[0].tolist()
    # teacher-force the oracle with the kernel's tokens; argmax must agree where the margin allows
    for pos, tok in enumerate(prompt.tolist()):
        logits = ref.decode_token(tok, pos)
    for i in range(ntok):
        want = int(logits.argmax())
        m = parity_metrics(logits, logits)  # margin and bf16 spacing of the oracle's own logits
        if m["top2_margin"] > 1e-2:
            assert got[i] == want, f"token {i}: {got[i]} vs {want}"
        if i + 1 < ntok:
            logits = ref.decode_token(got[i], prompt.numel() + i)


def test_fused_argmax_equals_torch_argmax_of_the_logits():
    """The LM-head epilogue's own argmax (all CTAs merge through the last one to finish) must be
    exactly torch.argmax of the logits the same launch wrote, launch after launch, also when
    ties exist (smallest index wins) and in CUDA-graph replay."""
    from megakernels_b200.generators import MK_Generator

    cfg = small_1b()
    _, _, gpu_model, gpu_sched = make_pair(cfg, 64, 0, poison=False)
    gen = MK_Generator(gpu_model, interpreter(), gpu_sched)
    globs = gpu_sched.globs
    assert globs.argmax_out is not None
    toks = seeded_tokens(cfg.vocab_size, 6, seed=5)
    for pos, tok in enumerate(toks):
        got = gen.run(torch.tensor([[tok]], device="cuda:0"), pos)
        gen.check()
        assert int(got) == int(torch.argmax(globs.logits)), f"position {pos}"
    # ties: a zero LM head makes every logit equal, so index 0 must win
    head = globs.lm_head_weights.data
    saved = head.clone()
    head.zero_()
    got = gen.run(torch.tensor([[toks[0]]], device="cuda:0"), len(toks))
    gen.check()
    assert int(got) == 0 == int(torch.argmax(globs.logits))
    head.copy_(saved)
    gen.enable_cuda_graph(warmup_pos=len(toks))
    for i, tok in enumerate(toks[:3]):
        got = gen.run(torch.tensor([[tok]], device="cuda:0"), len(toks) + 1 + i)
        gen.check()
        assert int(got) == int(torch.argmax(globs.logits)), f"graph replay {i}"
    # opting out restores the reference's host-side reduction
    _, _, gpu_model2, gpu_sched2 = make_pair(cfg, 64, 0, poison=False)
    gen2 = MK_Generator(gpu_model2, interpreter(), gpu_sched2, fused_argmax=False)
    assert gpu_sched2.globs.argmax_out is None
    got = gen2.run(torch.tensor([[toks[0]]], device="cuda:0"), 0)
    assert int(got) == int(torch.argmax(gpu_sched2.globs.logits))
