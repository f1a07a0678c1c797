"""Tensor parallelism: stream splitting on CPU, gloo ranks on CPU, emulated ranks on one GPU."""

import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from megakernels_b200.demos.latency.instructions import (
    DownProjResidual,
    LayerNormDoubleMatVecSiLU,
    O_ProjResidual,
    TP_AllReduce,
)
from megakernels_b200.demos.latency.scheduler import (
    LatencyScheduleOptions,
    split_at_collectives,
)
from megakernels_b200.llama import LlamaConfig
from megakernels_b200.utils import set_sm_count_override
from oracle.llama_ref import TorchReferenceModel, assert_logits_parity
from oracle.python_vm import PyVM_Interpreter
from tests.oracle_utils import build_model, build_schedule, fill_kv, seeded_tokens

CFG = dict(
    hidden_size=2048, intermediate_size=4096, num_hidden_layers=2, num_attention_heads=16,
    num_key_value_heads=4, head_dim=128, vocab_size=4096, tie_word_embeddings=False,
)
PREFILL = 24


def tp_model(rank, tp, device="cpu"):
    model = build_model(LlamaConfig(**CFG), 64, device=device, tp_size=tp, tp_rank=rank)
    # every rank holds its own KV heads of the same seeded cache
    full = build_model(LlamaConfig(**CFG), 64, device="cpu")
    fill_kv(full, PREFILL, poison=True)
    per = CFG["num_key_value_heads"] // tp
    for dst, src in zip(model.stacked_kv_cache, full.stacked_kv_cache):
        dst.copy_(src[:, :, :, rank * per : (rank + 1) * per])
    return model


def reference_logits(tokens):
    full = build_model(LlamaConfig(**CFG), 64, device="cpu")
    fill_kv(full, PREFILL, poison=True)
    ref = TorchReferenceModel(full)
    ref.load_kv(*full.stacked_kv_cache)
    return [ref.decode_token(t, PREFILL + i) for i, t in enumerate(tokens)]


def test_stream_is_cut_after_every_row_split_projection():
    set_sm_count_override(148)
    model = build_model(LlamaConfig(**CFG), 64, tp_size=2, tp_rank=0)
    sched = build_schedule(model, LatencyScheduleOptions(coalesce_o_proj=True))
    segs = split_at_collectives(sched.get_linear_instructions())
    assert len(segs) == 2 * CFG["num_hidden_layers"] + 1
    assert [ar for _, ar in segs] == [True] * (2 * CFG["num_hidden_layers"]) + [False]
    for (ins, ar), kind in zip(segs[:-1], [O_ProjResidual, DownProjResidual] * CFG["num_hidden_layers"]):
        assert isinstance(ins[-1], kind)
    assert sum(len(s) for s, _ in segs) == len(sched.get_linear_instructions())


def _gloo_rank(rank, world, port, tokens, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    set_sm_count_override(148)
    model = tp_model(rank, world)
    sched = build_schedule(model, LatencyScheduleOptions(coalesce_o_proj=True))
    g = sched.globs
    g.residual_scale = float(world)
    vm = PyVM_Interpreter()
    embed = model.model.embed_tokens.embed_tokens.weight
    logits = []
    for i, tok in enumerate(tokens):
        g.hidden_states[:] = embed[tok]
        g.barriers.zero_()
        g.pos_id = PREFILL + i
        for ins, needs_all_reduce in split_at_collectives(sched.get_linear_instructions()):
            vm.interpret(g, ins)
            if needs_all_reduce:  # gloo has no AVG: sum in fp32, divide, round once
                h = g.hidden_states.float()
                dist.all_reduce(h)
                g.hidden_states.copy_((h / world).to(g.hidden_states.dtype))
        logits.append(g.logits.clone())
    if rank == 0:
        torch.save(logits, out)
    dist.barrier()
    dist.destroy_process_group()


def test_two_gloo_ranks_reproduce_the_unsharded_model(tmp_path):
    """The sharding + scaled-residual + averaging scheme, with the CPU oracle as the kernel."""
    tokens = seeded_tokens(CFG["vocab_size"], 2)
    out = tmp_path / "logits.pt"
    mp.spawn(_gloo_rank, args=(2, 29517, tokens, str(out)), nprocs=2, join=True)
    got = torch.load(out)
    for a, b in zip(got, reference_logits(tokens)):
        assert_logits_parity(a, b, "tp=2 on gloo")


@pytest.mark.gpu
@pytest.mark.parametrize("tp", [2, 4])
def test_emulated_ranks_on_one_gpu(tp):
    """All ranks' megakernels run on one GPU, segment by segment; the all-reduce is a host loop."""
    from megakernels_b200.dispatch import make_mk_interpreter
    from megakernels_b200.generators import TP_MK_Generator

    tokens = seeded_tokens(CFG["vocab_size"], 2)
    gens = []
    for rank in range(tp):
        model = tp_model(rank, tp, device="cuda:0")
        sched = build_schedule(model, LatencyScheduleOptions(coalesce_o_proj=True))
        gens.append(TP_MK_Generator(model, make_mk_interpreter("latency"), sched, all_reduce=lambda t: None))
    want = reference_logits(tokens)
    for i, tok in enumerate(tokens):
        ids = torch.tensor([[tok]], device="cuda:0")
        for g in gens:
            g.begin_token(ids, PREFILL + i)
        for k in range(len(gens[0].segments)):
            flags = [g.launch_segment(k) for g in gens]
            if flags[0]:  # what TP_MK_Generator._nccl_average does across processes
                total = torch.stack([g.schedule.globs.residual_acc for g in gens]).sum(0)
                assert int((total % tp).abs().sum()) == 0, "every term is a multiple of the degree"
                for g in gens:
                    g.schedule.globs.residual_acc.copy_(total // tp)
        for g in gens:
            g.check()
            assert_logits_parity(g.schedule.globs.logits, want[i], f"tp={tp} step {i}")


def _nccl_rank(rank, world, port, tokens, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from megakernels_b200.dispatch import make_mk_interpreter
    from megakernels_b200.generators import TP_MK_Generator

    set_sm_count_override(torch.cuda.get_device_properties(rank).multi_processor_count)
    model = tp_model(rank, world, device=f"cuda:{rank}")
    sched = build_schedule(model, LatencyScheduleOptions(coalesce_o_proj=True))
    gen = TP_MK_Generator(model, make_mk_interpreter("latency"), sched)
    logits = []
    for i, tok in enumerate(tokens):
        gen.run(torch.tensor([[tok]], device=f"cuda:{rank}"), PREFILL + i)
        gen.check()
        logits.append(sched.globs.logits.cpu())
    if rank == 0:
        torch.save(logits, out)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.gpu
def test_nccl_ranks_on_real_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    tokens = seeded_tokens(CFG["vocab_size"], 2)
    out = tmp_path / "logits.pt"
    mp.spawn(_nccl_rank, args=(2, 29519, tokens, str(out)), nprocs=2, join=True)
    for a, b in zip(torch.load(out), reference_logits(tokens)):
        assert_logits_parity(a, b, "tp=2 on NCCL")


# --------------------------------------------------------------------------- #
# all-reduce inside the kernel (TP_AllReduce instructions, one launch per token)
# --------------------------------------------------------------------------- #
PEER_OPTIONS = dict(coalesce_o_proj=True, tp_all_reduce_chunks=4)


def test_all_reduce_instructions_follow_every_row_split_projection():
    set_sm_count_override(148)
    model = build_model(LlamaConfig(**CFG), 64, tp_size=2, tp_rank=1)
    sched = build_schedule(model, LatencyScheduleOptions(**PEER_OPTIONS))
    tp = sched.globs.tp
    assert (tp.size, tp.rank, tp.num_chunks) == (2, 1, 4)
    ins = sched.get_linear_instructions()
    ars = [i for i in ins if isinstance(i, TP_AllReduce)]
    assert len(ars) == 2 * CFG["num_hidden_layers"] * 4
    assert ars[0].serialize()[:5] == [8, 0, 0, 0, 4]
    # topological order: each group of chunks sits between its producer and its consumer
    kinds = [type(i) for i in ins]
    first_ar = kinds.index(TP_AllReduce)
    assert kinds[first_ar - 1] is O_ProjResidual
    assert kinds[first_ar + 4] is LayerNormDoubleMatVecSiLU
    # an unsharded model never gets them
    plain = build_schedule(build_model(LlamaConfig(**CFG), 64), LatencyScheduleOptions(**PEER_OPTIONS))
    assert plain.globs.tp is None
    assert not any(isinstance(i, TP_AllReduce) for i in plain.get_linear_instructions())


@pytest.mark.parametrize("mode", ["rr", "zz", "wave", "dag"])
def test_every_assignment_mode_keeps_all_reduce_chunks_in_order(mode):
    """Whatever the SM assignment, within a queue an all-reduce chunk comes after the row-split
    projections of its layer and before the RMSNorm op that consumes it (in-order queues)."""
    from megakernels_b200.scheduler import assign_to_sms

    set_sm_count_override(148)
    model = build_model(LlamaConfig(**CFG), 64, tp_size=2, tp_rank=0)
    sched = build_schedule(model, LatencyScheduleOptions(**PEER_OPTIONS))
    queues = assign_to_sms(mode, schedule=sched)
    seen = 0
    for q in queues:
        stage = {}  # layer -> furthest point reached: o-proj 0, ar0 1, upgate 2, down 3, ar1 4
        for ins in q:
            if isinstance(ins, TP_AllReduce):
                seen += 1
                rank_in_layer = 1 if ins.which == 0 else 4
            elif isinstance(ins, O_ProjResidual):
                rank_in_layer = 0
            elif isinstance(ins, LayerNormDoubleMatVecSiLU):
                rank_in_layer = 2
            elif isinstance(ins, DownProjResidual):
                rank_in_layer = 3
            else:
                continue
            layer = ins.layer_idx
            assert stage.get(layer, -1) <= rank_in_layer, f"{mode}: {ins} after stage {stage[layer]}"
            stage[layer] = rank_in_layer
    assert seen == 2 * CFG["num_hidden_layers"] * 4


def _attach_cpu_exchange(globs):
    """What megakernels_b200.peer.connect does on GPUs, for the CPU checker: local buffers
    and a gloo sum standing in for the stores into peer memory."""
    from megakernels_b200.instructions import TP_MAX_CHUNKS

    tp = globs.tp
    slices = max(globs.num_o_proj_col_splits(), globs.num_down_proj_col_splits())
    tp.partial = torch.zeros(slices, globs.hidden_size, dtype=torch.float32)
    tp.counters = torch.zeros(globs.num_hidden_layers, 2, 1 + TP_MAX_CHUNKS, dtype=torch.int32)

    def exchange(t):
        t = t.clone()
        dist.all_reduce(t)
        return t

    tp.exchange = exchange


def _gloo_peer_rank(rank, world, port, tokens, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    set_sm_count_override(148)
    model = tp_model(rank, world)
    sched = build_schedule(model, LatencyScheduleOptions(**PEER_OPTIONS))
    g = sched.globs
    _attach_cpu_exchange(g)
    vm = PyVM_Interpreter()
    embed = model.model.embed_tokens.embed_tokens.weight
    logits = []
    for i, tok in enumerate(tokens):
        g.hidden_states[:] = embed[tok]
        g.barriers.zero_()  # the tensor-parallel counters are NOT reset: they count up
        g.pos_id = PREFILL + i
        vm.interpret(g, sched.get_linear_instructions())
        g.tp.epoch += 1
        logits.append(g.logits.clone())
    assert int(g.tp.counters[0, 0, 0]) == 4 * len(tokens)
    if rank == 0:
        torch.save(logits, out)
    dist.barrier()
    dist.destroy_process_group()


def test_two_gloo_ranks_with_in_stream_all_reduce(tmp_path):
    """TP_AllReduce semantics (fp32 partial sums, one rounding, epoch counters) on the CPU checker."""
    tokens = seeded_tokens(CFG["vocab_size"], 3)
    out = tmp_path / "logits.pt"
    mp.spawn(_gloo_peer_rank, args=(2, 29521, tokens, str(out)), nprocs=2, join=True)
    for a, b in zip(torch.load(out), reference_logits(tokens)):
        assert_logits_parity(a, b, "tp=2, in-stream all-reduce on gloo")


def _peer_rank(rank, world, port, tokens, out, use_graph):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from megakernels_b200.dispatch import make_mk_interpreter
    from megakernels_b200.generators import TP_Peer_MK_Generator
    from megakernels_b200.scheduler import assign_to_sms, tensorize_instructions

    dev = f"cuda:{rank}"
    set_sm_count_override(torch.cuda.get_device_properties(rank).multi_processor_count)
    model = tp_model(rank, world, device=dev)
    sched = build_schedule(model, LatencyScheduleOptions(**PEER_OPTIONS))
    tensorize_instructions(sched.globs, assign_to_sms("rr", schedule=sched))
    gen = TP_Peer_MK_Generator(model, make_mk_interpreter("latency"), sched)
    if use_graph:
        gen.enable_cuda_graph(warmup_pos=PREFILL)
    logits, hidden = [], []
    for i, tok in enumerate(tokens):
        gen.run(torch.tensor([[tok]], device=dev), PREFILL + i)
        gen.check()
        logits.append(sched.globs.logits.cpu())
        hidden.append(sched.globs.tp.hidden_tagged[:, 0].cpu())  # the residual stream's bf16 pairs
    # every rank must hold the same residual stream, bit for bit
    gathered = [None] * world
    dist.all_gather_object(gathered, hidden)
    if rank == 0:
        for other in gathered[1:]:
            for a, b in zip(gathered[0], other):
                assert torch.equal(a, b), "ranks disagree on the residual stream"
        torch.save(logits, out)
    dist.barrier()
    gen.close()
    dist.destroy_process_group()


@pytest.mark.gpu
@pytest.mark.parametrize("use_graph", [False, True])
def test_peer_ranks_on_real_gpus(tmp_path, use_graph):
    """One launch per token and rank; the all-reduce runs inside the kernels over peer memory."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    tokens = seeded_tokens(CFG["vocab_size"], 3)
    out = tmp_path / "logits.pt"
    mp.spawn(_peer_rank, args=(2, 29523 + int(use_graph), tokens, str(out), use_graph), nprocs=2, join=True)
    for a, b in zip(torch.load(out), reference_logits(tokens)):
        assert_logits_parity(a, b, "tp=2, in-kernel all-reduce")


def _peer_rank_with_a_silent_peer(rank, world, port, tokens, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from megakernels_b200.dispatch import make_mk_interpreter
    from megakernels_b200.generators import TP_Peer_MK_Generator
    from megakernels_b200.scheduler import assign_to_sms, tensorize_instructions

    dev = f"cuda:{rank}"
    set_sm_count_override(torch.cuda.get_device_properties(rank).multi_processor_count)
    model = tp_model(rank, world, device=dev)
    sched = build_schedule(model, LatencyScheduleOptions(**PEER_OPTIONS))
    tensorize_instructions(sched.globs, assign_to_sms("rr", schedule=sched))
    gen = TP_Peer_MK_Generator(model, make_mk_interpreter("latency"), sched)
    import mk_llama  # the module make_mk_interpreter put on the path

    g = sched.globs
    verdict = "not run"
    if rank == 0:
        # rank 1 never launches: rank 0's waits for its partial sums must run out (50 ms
        # budget) and come back as a status record, not as a hang
        g.hidden_states[:] = model.model.embed_tokens.embed_tokens.weight[tokens[0]]
        g.barriers.zero_()
        g.pos_id = PREFILL
        call = gen.interpreter.interpret(g, wait_timeout_ms=50)
        try:
            mk_llama.sync_status(call)
            verdict = "no error"
        except mk_llama.MegakernelError as err:
            verdict = f"code {err.code} opcode {err.status.opcode}"
    dist.barrier()  # rank 1 sat here on the host the whole time, nothing of it in flight
    # Recovery rule: the aborted launch left partial sums with the current launch counter's
    # tags in the owners' receive buffers, so both ranks move to a counter value nobody used.
    assert gen.resync_epoch() == 1
    # the context is still usable and the exchange recovers.  The retry decodes a DIFFERENT
    # token than the aborted launch (same position, so the half-written K/V row is
    # overwritten): stale sums taken for fresh ones would now show in the logits
    logits = []
    for i, tok in enumerate(tokens[1:]):
        gen.run(torch.tensor([[tok]], device=dev), PREFILL + i)
        gen.check()
        logits.append(g.logits.cpu())
    if rank == 0:
        torch.save((verdict, logits), out)
    dist.barrier()
    gen.close()
    dist.destroy_process_group()


@pytest.mark.gpu
def test_peer_rank_that_never_launches_is_reported_not_hung(tmp_path):
    """Failure detection across GPUs without faulting one: the missing rank is simulated on the
    host (it simply does not launch); the waiting rank's polls are bounded."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    tokens = seeded_tokens(CFG["vocab_size"], 3)
    out = tmp_path / "result.pt"
    mp.spawn(_peer_rank_with_a_silent_peer, args=(2, 29527, tokens, str(out)), nprocs=2, join=True)
    verdict, logits = torch.load(out)
    assert verdict.startswith("code 3"), verdict  # MKB_ERR_DEVICE_TIMEOUT
    for a, b in zip(logits, reference_logits(tokens[1:])):
        assert_logits_parity(a, b, "tp=2 after a timed-out launch")
