"""Latency DAG builder: one token of Llama decode as a DAG of instructions.

Reference: megakernels/demos/latency/scheduler.py.  At the Llama-3.2-1B shape
with default options this emits the reference's instruction stream word for
word.  Differences are generalisations the reference does not have:

* every count is derived from the model shape (the reference's builder and
  Python VM hard-code 1B constants), so 8B / 70B / tensor-parallel shards build;
* ``num_attention_partitions > 1`` emits split-KV ``PartialAttention``
  instructions plus one terminal ``AttentionReduction`` per group of 4 Q heads
  (the reference asserts ``skip_attn_reduction``, latency/scheduler.py:276-277);
* ``coalesce_o_proj`` emits one block-range O-proj instruction per SM instead
  of one per 16-row block (latency/scheduler.py:344-354);
* ``merge_in_last_partial`` drops the terminal reductions: the partial-attention
  instruction of a KV head that arrives last merges the partial rows itself;
* ``tp_all_reduce_chunks`` (tensor-parallel shards only) emits ``TP_AllReduce``
  instructions after every o-proj and down-proj group, so that the ranks
  exchange their partial sums inside the kernel and a token stays one launch.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from megakernels_b200.demos.latency.instructions import (
    AttentionReduction,
    DownProjResidual,
    Globals,
    Instruction,
    LayerNorm_QKV_MatVecRopeAppend,
    LayerNormDoubleMatVecSiLU,
    O_ProjResidual,
    PartialAttention,
    RMS_LM_Head,
    RMS_Norm,
    TP_AllReduce,
)
from megakernels_b200.instructions import NoOp, TensorParallelState
from megakernels_b200.scheduler import DAG_Node, ScheduleBuilder
from megakernels_b200.utils import assert_div, get_sm_count

MAX_REDUCTION_LIST = 24  # idx list + 7 fixed words must fit the 32-word instruction


@dataclass
class LatencyScheduleOptions:
    """Knobs of the DAG builder; the defaults reproduce the reference stream."""

    num_attention_partitions: int = 1
    coalesce_o_proj: bool = False
    # with more than one attention partition: no AttentionReduction instructions; the partial of a
    # KV head that arrives last merges the partial rows itself and signals the o-proj (one barrier
    # hop and one instruction less on the critical path of a layer)
    merge_in_last_partial: bool = False
    # > 1: batched decode, that many independent sequences per launch (at most 64; more than 8
    # switches the schedule to 128-row blocks for the tcgen05 build of the kernel); the model's
    # KV cache must hold them (ExtraModelConfig.max_batch_size)
    batch_size: int = 1
    # > 0 on a tensor-parallel shard: all-reduce the residual stream inside the kernel,
    # split into this many chunks (a multiple of the TP degree); 0 leaves the exchange
    # to the host (generators.TP_MK_Generator cuts the stream and calls NCCL)
    tp_all_reduce_chunks: int = 0


def pick_num_attention_partitions(
    prompt_len: int, ntok: int, device=None, num_kv_heads: int = 8, min_chunk_size: int = 256
):
    """Partitions per KV head for a generation of ``prompt_len + ntok`` tokens.

    Reference heuristic: one partition per 256 positions, at most 24
    (latency/scheduler.py:21-35).  Additionally capped so that all partials of
    a layer fit one wave of SMs.  On B200 a chunk of 128 positions measures
    slightly faster (a partial then spans at most two 64-position KV stages).
    """
    full_len = prompt_len + ntok
    n = min(math.ceil(full_len / min_chunk_size), MAX_REDUCTION_LIST)
    n = min(n, max(1, get_sm_count(device) // num_kv_heads))
    return max(1, n)


def pick_matvec_reduction_size(o_in_features: int, intermediate_size: int) -> int:
    """Largest input-column slice (<= 2048) dividing both row-split projections."""
    for r in (2048, 1024, 512, 256):
        if o_in_features % r == 0 and intermediate_size % r == 0:
            return r
    raise ValueError(
        f"o-proj inputs {o_in_features} and intermediate {intermediate_size} "
        "must both be multiples of 256"
    )


def make_globals(
    model, skip_attn_reduction: bool = True, max_attn_partitions: int | None = None, batch_size: int = 1
):
    """Allocate activation buffers and barriers; gather weights (scheduler.py:38-115).

    ``batch_size`` > 1 gives every activation buffer a leading batch dimension.
    """
    config = model.config
    device = model.device
    dtype = model.dtype
    assert 1 <= batch_size <= 64 and batch_size <= model.extra_config.max_batch_size
    # 9..64 sequences run the tcgen05 build of the kernel, whose blocks are 128 weight rows
    # (the M side of the MMA); everything else counts blocks of 16 rows as the reference does
    block = 128 if batch_size > 8 else 16
    if batch_size > 8:
        assert config.head_dim == 128 and config.vocab_size % 128 == 0, "the GEMM build needs 128-row blocks"

    def make_buffer(shape, buffer_dtype=dtype):
        shape = [shape] if isinstance(shape, int) else list(shape)
        if batch_size > 1:
            shape = [batch_size] + shape
        return torch.zeros(shape, device=device, dtype=buffer_dtype)

    sp = model.stacked_params
    n_q = model.num_qo_heads()
    n_kv = model.num_kv_heads()
    inter = model.local_intermediate_size()
    if max_attn_partitions is None:
        max_attn_partitions = get_sm_count(device) if batch_size == 1 else 24

    # barrier counters and residual accumulators share one buffer: one fill resets both
    # one slot per head as in the reference (latency/scheduler.py:59); small tensor-parallel
    # shards can have more down-proj input slices than heads, and every slice needs a slot
    reduction = pick_matvec_reduction_size(n_q * config.head_dim, inter)
    # (and a batched launch one slot per sequence and Q head in the partial-attention row)
    width = max(n_q + 2 * n_kv, inter // reduction, batch_size * n_q if batch_size > 1 else 0)
    bar_shape = [config.num_hidden_layers, 10, width]
    n_bar = math.prod(bar_shape)
    acc_off = (n_bar + 3) // 4 * 4  # int64 view needs 8-byte, the kernel's loads 16-byte alignment
    vm_state = torch.zeros(acc_off + 2 * batch_size * config.hidden_size, dtype=torch.int32, device=device)
    barriers = vm_state[:n_bar].view(bar_shape)

    globs = Globals(
        qkv_proj_weights=sp.qkv_proj,
        o_proj_weights=sp.o_proj,
        attn_ln_weights=sp.attn_ln_weight,
        mlp_ln_weights=sp.mlp_ln_weight,
        up_proj_weights=sp.up_proj,
        gate_proj_weights=sp.gate_proj,
        down_proj_weights=sp.down_proj,
        lm_head_norm_weights=model.lm_head.input_norm.weight,
        lm_head_weights=model.lm_head.lm_head.weight,
        k_cache=model.stacked_kv_cache[0],
        v_cache=model.stacked_kv_cache[1],
        rope_cos=model.model.rope_cos,
        rope_sin=model.model.rope_sin,
        hidden_states=make_buffer(config.hidden_size),
        post_ln_rope_q=make_buffer(n_q * config.head_dim),
        attn_out=make_buffer(n_q * config.head_dim),
        attn_out_intermediates=make_buffer(
            [n_q, max_attn_partitions, config.head_dim], buffer_dtype=torch.float32
        ),
        attn_lse_intermediates=make_buffer(
            [n_q, max_attn_partitions], buffer_dtype=torch.float32
        ),
        silu_out=make_buffer(inter),
        logits=make_buffer(config.vocab_size),
        pos_id=0,
        attn_scale=1 / math.sqrt(config.head_dim),
        rms_norm_eps=config.rms_norm_eps,
        skip_attn_reduction=skip_attn_reduction,
        num_hidden_layers=config.num_hidden_layers,
        num_attention_heads=n_q,
        num_kv_heads=n_kv,
        head_dim=config.head_dim,
        hidden_size=config.hidden_size,
        intermediate_size=inter,
        up_gate_proj_block_size=block,
        down_proj_block_size=block,
        qkv_block_size=block,
        o_proj_block_size=block,
        lm_head_block_size=block,
        matvec_reduction_size=reduction,
        attn_kv_block_size=16,
        attn_reduction_size=4,
        vocab_size=config.vocab_size,
        device=device,
        barriers=barriers,
    )
    globs.vm_state = vm_state
    globs.residual_acc = vm_state[acc_off:].view(torch.int64)
    if batch_size > 1:
        globs.batch_size = batch_size
        globs.residual_acc = globs.residual_acc.view(batch_size, config.hidden_size)
        globs.normed_states = make_buffer(config.hidden_size)
        globs.pos_ids = [0] * batch_size
    return globs


def _even_ranges(num_blocks: int, parts: int):
    # fewer blocks than SMs (small tensor-parallel shards): one block each
    parts = min(parts, num_blocks)
    per = num_blocks / parts
    return [(round(i * per), round((i + 1) * per)) for i in range(parts)]


def schedule_qkv(globs: Globals, layer_idx: int):
    """One contiguous block range per SM (reference: scheduler.py:118-144)."""
    out_dim = (globs.num_attention_heads + 2 * globs.num_kv_heads) * globs.head_dim
    n_blocks = assert_div(out_dim, globs.qkv_block_size)
    return [
        LayerNorm_QKV_MatVecRopeAppend(layer_idx, s, e)
        for s, e in _even_ranges(n_blocks, globs.sm_count())
    ]


def schedule_upgate(globs: Globals, layer_idx: int):
    """Strided block lists, SM ``i`` gets blocks ``i, i+N, ...`` (scheduler.py:147-166)."""
    n_blocks = assert_div(globs.intermediate_size, globs.up_gate_proj_block_size)
    sm_count = min(globs.sm_count(), n_blocks)
    return [
        LayerNormDoubleMatVecSiLU(layer_idx, list(range(sm, n_blocks, sm_count)))
        for sm in range(sm_count)
    ]


def _split_jobs_within_columns(num_col_splits: int, num_row_blocks: int, sm_count: int):
    """Deal ``(col, row_block)`` jobs to SMs in contiguous runs of one column.

    Same greedy walk as the reference's down-proj scheduling
    (scheduler.py:169-216): each SM takes ``round(jobs_left / sms_left)`` jobs,
    truncated at the first change of column.
    """
    jobs = [(c, b) for c in range(num_col_splits) for b in range(num_row_blocks)]
    out = []
    done = 0
    for sm in range(sm_count):
        per = (len(jobs) - done) / (sm_count - sm)
        if per <= 1:
            return None  # the reference asserts here; the caller falls back to exact runs
        take = jobs[done : done + round(per)]
        col = take[0][0]
        take = [j for j in take if j[0] == col]
        start = take[0][1]
        out.append((col, start, start + len(take)))
        done += len(take)
    return out


def schedule_downproj(globs: Globals, layer_idx: int):
    n_blocks = assert_div(globs.hidden_size, globs.down_proj_block_size)
    splits = globs.num_down_proj_col_splits()
    runs = None
    if splits * n_blocks > globs.sm_count():
        runs = _split_jobs_within_columns(splits, n_blocks, globs.sm_count())
        if runs is not None and sum(e - s for _, s, e in runs) != n_blocks * splits:
            runs = None  # the truncating walk stranded jobs (shapes far from 1B)
    if runs is None:
        runs = _exact_runs(splits, n_blocks, globs.sm_count())
    return [DownProjResidual(layer_idx, s, e, c) for c, s, e in runs]


def _exact_runs(num_col_splits: int, num_row_blocks: int, sm_count: int):
    """Cover every ``(col, row_block)`` job with contiguous same-column runs."""
    total = num_col_splits * num_row_blocks
    sm_count = min(sm_count, total)
    per = total / sm_count
    runs = []
    for i in range(sm_count):
        lo, hi = round(i * per), round((i + 1) * per)
        while lo < hi:
            col, start = divmod(lo, num_row_blocks)
            end = min(num_row_blocks, start + (hi - lo))
            runs.append((col, start, end))
            lo += end - start
    return runs


def schedule_oproj(globs: Globals, layer_idx: int, coalesce: bool):
    n_blocks = assert_div(globs.hidden_size, globs.o_proj_block_size)
    splits = globs.num_o_proj_col_splits()
    if not coalesce:
        return [
            O_ProjResidual(layer_idx, b, b + 1, c) for c in range(splits) for b in range(n_blocks)
        ]
    return [
        O_ProjResidual(layer_idx, s, e, c)
        for c, s, e in _exact_runs(splits, n_blocks, globs.sm_count())
    ]


def schedule_lm_head(globs: Globals):
    n_blocks = assert_div(globs.vocab_size, globs.lm_head_block_size)
    return [RMS_LM_Head(s, e) for s, e in _even_ranges(n_blocks, globs.sm_count())]


def make_dag_layer(
    globs: Globals,
    layer_idx: int,
    prev_layer_outputs: list[DAG_Node],
    stop_after_op: str | None = None,
    options: LatencyScheduleOptions | None = None,
):
    """Reference: megakernels/demos/latency/scheduler.py:270-386."""
    options = options or LatencyScheduleOptions()
    n_part = options.num_attention_partitions
    if globs.skip_attn_reduction:
        assert n_part == 1, "skip_attn_reduction requires a single attention partition"
    assert 1 <= n_part <= MAX_REDUCTION_LIST
    assert n_part <= globs.attn_lse_intermediates.shape[-1]

    new_nodes: list[DAG_Node] = []

    qkv_nodes = [DAG_Node(ins, prev_layer_outputs) for ins in schedule_qkv(globs, layer_idx)]
    block_owner = {}
    for node in qkv_nodes:
        for b in node.instruction.block_indices():
            block_owner[b] = node
    new_nodes.extend(qkv_nodes)
    if stop_after_op == "qkv":
        return new_nodes, qkv_nodes

    blocks_per_head = assert_div(globs.head_dim, globs.qkv_block_size)
    partial_nodes: list[DAG_Node] = []
    partials_of_head: dict[int, list[DAG_Node]] = {}
    for kv in range(globs.num_kv_heads):
        k0 = (globs.num_attention_heads + kv) * blocks_per_head
        v0 = (globs.num_attention_heads + globs.num_kv_heads + kv) * blocks_per_head
        needed = list(range(k0, k0 + blocks_per_head)) + list(range(v0, v0 + blocks_per_head))
        deps = list({id(block_owner[b]): block_owner[b] for b in needed}.values())
        for p in range(n_part):
            node = DAG_Node(PartialAttention(layer_idx, kv, n_part, p), deps)
            partial_nodes.append(node)
            partials_of_head.setdefault(kv, []).append(node)
    new_nodes.extend(partial_nodes)
    if stop_after_op == "partial":
        return new_nodes, partial_nodes

    attn_outputs = partial_nodes
    if not globs.skip_attn_reduction and not globs.merge_in_last_partial:
        gqa = assert_div(globs.num_attention_heads, globs.num_kv_heads)
        red_nodes: list[DAG_Node] = []
        for head_start in range(0, globs.num_attention_heads, globs.attn_reduction_size):
            ins = AttentionReduction(
                layer_idx=layer_idx,
                head_start_idx=head_start,
                num_partials=n_part,
                is_terminal=True,
                reduction_list=list(range(n_part)),
                output_partial_idx=None,
            )
            red_nodes.append(DAG_Node(ins, partials_of_head[head_start // gqa]))
        new_nodes.extend(red_nodes)
        attn_outputs = red_nodes
        if stop_after_op == "reduction":
            return new_nodes, red_nodes

    o_nodes = [
        DAG_Node(ins, attn_outputs)
        for ins in schedule_oproj(globs, layer_idx, options.coalesce_o_proj)
    ]
    new_nodes.extend(o_nodes)
    if stop_after_op == "oproj":
        return new_nodes, o_nodes
    if globs.tp is not None:
        n = globs.tp.num_chunks
        o_nodes = [DAG_Node(TP_AllReduce(layer_idx, 0, c, n), o_nodes) for c in range(n)]
        new_nodes.extend(o_nodes)

    upgate_nodes = [DAG_Node(ins, o_nodes) for ins in schedule_upgate(globs, layer_idx)]
    new_nodes.extend(upgate_nodes)
    if stop_after_op == "upgate":
        return new_nodes, upgate_nodes

    down_nodes = [DAG_Node(ins, upgate_nodes) for ins in schedule_downproj(globs, layer_idx)]
    new_nodes.extend(down_nodes)
    if stop_after_op == "downproj":
        return new_nodes, down_nodes
    if globs.tp is not None:
        n = globs.tp.num_chunks
        down_nodes = [DAG_Node(TP_AllReduce(layer_idx, 1, c, n), down_nodes) for c in range(n)]
        new_nodes.extend(down_nodes)

    assert stop_after_op is None
    return new_nodes, down_nodes


def make_batched_dag(globs: Globals, options: LatencyScheduleOptions, layer_limit: int | None = None):
    """One decode step of ``globs.batch_size`` independent sequences (no counterpart in the
    reference).  The projections are the same instructions as for one sequence - a block is
    multiplied with every sequence's activation vector while it is in shared memory - and
    wait for ``RMS_Norm`` instructions instead of normalising; attention and its reduction are
    emitted per sequence, each over that sequence's own length."""
    B, n_part = globs.batch_size, options.num_attention_partitions
    assert globs.tp is None, "batched decode has no tensor-parallel variant"
    assert 1 <= n_part <= MAX_REDUCTION_LIST and n_part <= globs.attn_lse_intermediates.shape[-1]
    assert globs.skip_attn_reduction == (n_part == 1)
    nodes: list[DAG_Node] = []
    nlayers = globs.num_hidden_layers if layer_limit is None else layer_limit
    gqa = assert_div(globs.num_attention_heads, globs.num_kv_heads)
    last: list[DAG_Node] = []

    def emit(instructions, deps):
        new = [DAG_Node(ins, deps) for ins in instructions]
        nodes.extend(new)
        return new

    for layer in range(nlayers):
        norm = emit([RMS_Norm(layer, 0, b) for b in range(B)], last)
        qkv = emit(schedule_qkv(globs, layer), norm)
        attn_out: list[DAG_Node] = []
        for b in range(B):
            for kv in range(globs.num_kv_heads):
                parts = emit([PartialAttention(layer, kv, n_part, p, b) for p in range(n_part)], qkv)
                if globs.skip_attn_reduction or globs.merge_in_last_partial:
                    attn_out.extend(parts)  # (the last partial to arrive merges the rows)
                    continue
                for h0 in range(kv * gqa, (kv + 1) * gqa, globs.attn_reduction_size):
                    attn_out.extend(
                        emit([AttentionReduction(layer, h0, n_part, True, list(range(n_part)), None, b)], parts)
                    )
        o = emit(schedule_oproj(globs, layer, options.coalesce_o_proj), attn_out)
        norm = emit([RMS_Norm(layer, 1, b) for b in range(B)], o)
        up = emit(schedule_upgate(globs, layer), norm)
        last = emit(schedule_downproj(globs, layer), up)
    if nlayers == globs.num_hidden_layers:
        norm = emit([RMS_Norm(nlayers - 1, 2, b) for b in range(B)], last)
        last = emit(schedule_lm_head(globs), norm)
    return nodes, DAG_Node(NoOp(), last)


def make_dag(
    globs: Globals,
    stop_after_op: str | None = None,
    layer_limit: int | None = None,
    options: LatencyScheduleOptions | None = None,
):
    """Reference: megakernels/demos/latency/scheduler.py:235-267."""
    if globs.batch_size > 1:
        assert stop_after_op is None, "the batched builder emits whole layers"
        return make_batched_dag(globs, options or LatencyScheduleOptions(), layer_limit)
    nodes: list[DAG_Node] = []
    nlayers = globs.num_hidden_layers if layer_limit is None else layer_limit
    last_outputs: list[DAG_Node] = []
    for layer_idx in range(nlayers):
        new_nodes, last_outputs = make_dag_layer(
            globs, layer_idx, last_outputs, stop_after_op, options
        )
        nodes.extend(new_nodes)
    if nlayers == globs.num_hidden_layers:
        head_nodes = [DAG_Node(ins, last_outputs) for ins in schedule_lm_head(globs)]
        nodes.extend(head_nodes)
        last_outputs = head_nodes
    return nodes, DAG_Node(NoOp(), last_outputs)


class LatencyScheduleBuilder(ScheduleBuilder):
    """Builder with reference-identical defaults; set ``options`` to tune."""

    options = LatencyScheduleOptions()

    def __init__(self, options: LatencyScheduleOptions | None = None):
        if options is not None:
            self.options = options

    # ``build`` is usable on the class (as in the reference) and on an
    # instance carrying non-default options.
    def build(self, model, stop_after_op=None, layer_limit=None):  # type: ignore[override]
        from megakernels_b200.scheduler import Schedule

        globs = self.make_globals(model)
        nodes, end = make_dag(globs, stop_after_op, layer_limit, self.options)
        # (a batched launch orders the down-proj behind the norm through the up/gate itself)
        globs.upgate_instructions_per_layer = 0 if globs.batch_size > 1 else sum(
            1
            for n in nodes
            if isinstance(n.instruction, LayerNormDoubleMatVecSiLU) and n.instruction.layer_idx == 0
        )
        return Schedule(globs, nodes, end)

    def make_globals(self, model):  # type: ignore[override]
        skip = self.options.num_attention_partitions == 1
        globs = make_globals(model, skip_attn_reduction=skip, batch_size=self.options.batch_size)
        globs.merge_in_last_partial = bool(self.options.merge_in_last_partial) and not skip
        extra = model.extra_config
        if self.options.tp_all_reduce_chunks and extra.tp_size > 1:
            globs.tp = TensorParallelState(extra.tp_size, extra.tp_rank, self.options.tp_all_reduce_chunks)
        return globs

    def with_new_globals(self, schedule, model):  # type: ignore[override]
        from dataclasses import replace

        return replace(schedule, globs=self.make_globals(model))

    def make_dag(self, globs, stop_after_op=None, layer_limit=None):  # type: ignore[override]
        return make_dag(globs, stop_after_op, layer_limit, self.options)


def split_at_collectives(instructions: list[Instruction]) -> list[tuple[list[Instruction], bool]]:
    """Cut a topologically ordered stream where tensor parallelism needs an all-reduce.

    Row-split projections (o-proj, down-proj) leave every rank with a partial sum of
    the residual stream, so the stream is cut after each layer's o-proj group and
    after each down-proj group.  Returns ``[(segment, needs_all_reduce_after), ...]``;
    barrier counters carry over from one segment to the next.
    """
    segments: list[tuple[list[Instruction], bool]] = []
    cur: list[Instruction] = []
    for ins in instructions:
        if cur and cur[-1].opcode() in (O_ProjResidual.opcode(), DownProjResidual.opcode()) and (
            ins.opcode() != cur[-1].opcode()
        ):
            segments.append((cur, True))
            cur = []
        cur.append(ins)
    if cur:
        last = cur[-1].opcode()
        segments.append((cur, last in (O_ProjResidual.opcode(), DownProjResidual.opcode())))
    return segments
