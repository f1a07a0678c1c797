"""Timeline-model schedule builder: balances every phase against a cost model.

The reference splits each projection evenly over the SMs (latency/scheduler.py:
118-232).  With 16-row blocks that leaves whole-block remainders - 896 up/gate
block pairs over 148 SMs is 6 or 7 pairs, 16 % more for eight SMs - and because
almost every phase ends in a global barrier, the slowest SM of every phase is on
the critical path.  This builder keeps a simulated clock per SM and

* hands each phase's jobs to the SMs by water-filling over the times at which
  the SMs become free (an SM that ran an attention instruction gets fewer
  o-proj jobs, an SM with a seventh up/gate pair gets fewer down-proj jobs);
* deals up/gate blocks in index order so that the column slices of the
  intermediate vector complete one after the other, and releases the down-proj
  jobs of a slice as soon as that slice is complete, so the remainder of one
  phase overlaps the start of the next;
* pins every instruction to its SM (attribute ``sm_hint``, honoured by
  ``assign_to_sms("hint", ...)``).

The instruction set is unchanged; only block ranges and the SM mapping differ
from the reference stream.
"""

from __future__ import annotations

import heapq
from dataclasses import dataclass

from megakernels_b200.demos.latency.instructions import (
    AttentionReduction,
    DownProjResidual,
    Globals,
    LayerNorm_QKV_MatVecRopeAppend,
    LayerNormDoubleMatVecSiLU,
    O_ProjResidual,
    PartialAttention,
    RMS_LM_Head,
)
from megakernels_b200.instructions import Instruction, NoOp
from megakernels_b200.scheduler import DAG_Node

MAX_UPGATE_LIST = 29  # block list + 3 fixed words must fit the 32-word instruction


@dataclass
class CostModel:
    """Microseconds, measured on B200 with the timing trace (8B shape)."""

    bytes_per_us: float = 51e3  # one SM's share of HBM bandwidth
    hop: float = 2.0  # producer's last store -> consumer sees the counter
    rms_setup: float = 2.5  # barrier seen -> RMS-normalised activations ready
    plain_setup: float = 0.8  # barrier seen -> activation slice ready
    attention: float = 6.0  # one partial-attention instruction
    reduction: float = 3.5  # one attention-reduction instruction


def _waterfill(avail: list[float], n_jobs: int, cost: float, release: float = 0.0) -> list[int]:
    """Jobs per SM so that all SMs finish as evenly as possible.

    SM ``i`` can start at ``max(avail[i], release)``; every job costs ``cost``.
    """
    start = [max(a, release) for a in avail]
    counts = [0] * len(avail)
    heap = [(s + cost, i) for i, s in enumerate(start)]  # finish time if given one more job
    heapq.heapify(heap)
    for _ in range(n_jobs):
        finish, i = heapq.heappop(heap)
        counts[i] += 1
        heapq.heappush(heap, (finish + cost, i))
    return counts


class _Timeline:
    def __init__(self, globs: Globals, model: CostModel):
        self.g = globs
        self.m = model
        self.n = globs.sm_count()
        self.t = [0.0] * self.n  # when each SM is free
        self.nodes: list[DAG_Node] = []

    def emit(self, ins: Instruction, sm: int, deps: list[DAG_Node]) -> DAG_Node:
        ins.sm_hint = sm  # not a dataclass field: never serialised
        node = DAG_Node(ins, deps)
        self.nodes.append(node)
        return node

    # ---- phases ---------------------------------------------------------- #
    def ranges_phase(self, n_blocks, block_bytes, release, setup, make, deps):
        """Contiguous block ranges, water-filled; returns (nodes, per-block finish times)."""
        cost = block_bytes / self.m.bytes_per_us
        avail = [max(t, release) + setup for t in self.t]
        counts = _waterfill(avail, n_blocks, cost)
        order = sorted(range(self.n), key=lambda i: (avail[i], i))
        nodes, finish, blk = [], [0.0] * n_blocks, 0
        for sm in order:
            if counts[sm] == 0:
                continue
            s, e = blk, blk + counts[sm]
            nodes.append(self.emit(make(s, e), sm, deps))
            for k in range(s, e):
                finish[k] = avail[sm] + (k - s + 1) * cost
            self.t[sm] = avail[sm] + counts[sm] * cost
            blk = e
        assert blk == n_blocks
        return nodes, finish

    def sliced_phase(self, n_row_blocks, n_slices, job_bytes, releases, setup, make, deps):
        """(slice, row block) jobs with a release time per slice.

        The number of jobs per SM comes from water-filling over the SMs' free times; the
        jobs are then walked in release order (slices as they complete, rows ascending)
        and handed out as contiguous runs to the SMs in the order in which they become
        free, so early SMs work on early slices and an SM runs one instruction per slice
        it touches (usually one or two).
        """
        cost = job_bytes / self.m.bytes_per_us
        first_release = min(releases)
        avail = [max(t, first_release) + setup for t in self.t]
        counts = _waterfill(avail, n_row_blocks * n_slices, cost)
        order = sorted(range(self.n), key=lambda i: (avail[i], i))
        slice_order = sorted(range(n_slices), key=lambda s: (releases[s], s))
        nodes, pos, end_time = [], 0, 0.0  # pos indexes the (slice, row) sequence
        for sm in order:
            left, now = counts[sm], self.t[sm]
            while left > 0:
                sl = slice_order[pos // n_row_blocks]
                rb = pos % n_row_blocks
                n = min(left, n_row_blocks - rb)
                nodes.append(self.emit(make(rb, rb + n, sl), sm, deps))
                now = max(now, releases[sl]) + setup + n * cost
                pos += n
                left -= n
            if counts[sm]:
                self.t[sm] = now
                end_time = max(end_time, now)
        assert pos == n_row_blocks * n_slices
        return nodes, end_time

    def single_phase(self, jobs, cost):
        """One instruction each, earliest-free SM first.  jobs: [(release, make, deps)]."""
        nodes = []
        heap = [(t, i) for i, t in enumerate(self.t)]
        heapq.heapify(heap)
        finish = []
        for release, make, deps in jobs:
            a, sm = heapq.heappop(heap)
            done = max(a, release) + cost
            nodes.append(self.emit(make(), sm, deps))
            finish.append(done)
            self.t[sm] = done
            heapq.heappush(heap, (done, sm))
        return nodes, finish


def make_balanced_dag(globs: Globals, options, layer_limit: int | None = None, model: CostModel | None = None):
    """Whole-token DAG with pinned, cost-balanced instructions (see module docstring)."""
    g, m = globs, model or CostModel()
    tl = _Timeline(g, m)
    n_part = options.num_attention_partitions
    H, D, R = g.hidden_size, g.head_dim, g.matvec_reduction_size
    Hq, Hkv = g.num_attention_heads, g.num_kv_heads
    gqa = Hq // Hkv
    bph = D // 16  # qkv blocks per head
    nlayers = g.num_hidden_layers if layer_limit is None else layer_limit
    last: list[DAG_Node] = []
    release = 0.0
    for layer in range(nlayers):
        # ---- qkv ----
        qkv_blocks = (Hq + 2 * Hkv) * D // 16
        qkv_nodes, qkv_done = tl.ranges_phase(
            qkv_blocks, 16 * H * 2, release, m.rms_setup,
            lambda s, e, layer=layer: LayerNorm_QKV_MatVecRopeAppend(layer, s, e), last,
        )
        head_done = [max(qkv_done[h * bph : (h + 1) * bph]) for h in range(Hq + 2 * Hkv)]
        # ---- attention ----
        jobs = []
        for kv in range(Hkv):
            ready = max(
                max(head_done[kv * gqa : (kv + 1) * gqa]), head_done[Hq + kv], head_done[Hq + Hkv + kv]
            ) + m.hop
            for p in range(n_part):
                jobs.append((ready, lambda layer=layer, kv=kv, p=p: PartialAttention(layer, kv, n_part, p), qkv_nodes))
        part_nodes, part_done = tl.single_phase(jobs, m.attention)
        attn_nodes, attn_done = part_nodes, max(part_done)
        if not g.skip_attn_reduction:
            jobs = []
            for h0 in range(0, Hq, g.attn_reduction_size):
                kv = h0 // gqa
                ready = max(part_done[kv * n_part : (kv + 1) * n_part]) + m.hop
                jobs.append((
                    ready,
                    lambda layer=layer, h0=h0: AttentionReduction(layer, h0, n_part, True, list(range(n_part)), None),
                    part_nodes[kv * n_part : (kv + 1) * n_part],
                ))
            attn_nodes, red_done = tl.single_phase(jobs, m.reduction)
            attn_done = max(red_done)
        # ---- o-proj: every job waits for all heads ----
        o_slices = g.num_o_proj_col_splits()
        o_nodes, o_done = tl.sliced_phase(
            H // 16, o_slices, 16 * R * 2, [attn_done + m.hop] * o_slices, m.plain_setup,
            lambda s, e, sl, layer=layer: O_ProjResidual(layer, s, e, sl), attn_nodes,
        )
        # ---- up/gate: blocks dealt in index order, water-filled counts ----
        n_up = g.intermediate_size // 16
        pair_cost = 2 * 16 * H * 2 / m.bytes_per_us
        avail = [max(t, o_done + m.hop) + m.rms_setup for t in tl.t]
        counts = _waterfill(avail, n_up, pair_cost)
        order = sorted(range(tl.n), key=lambda i: (avail[i], i))
        lists: dict[int, list[int]] = {sm: [] for sm in order}
        blk = 0
        for rnd in range(max(counts)):
            for sm in order:
                if counts[sm] > rnd and blk < n_up:
                    lists[sm].append(blk)
                    blk += 1
        assert blk == n_up
        up_nodes, blk_done = [], [0.0] * n_up
        for sm in order:
            blocks = lists[sm]
            for c0 in range(0, len(blocks), MAX_UPGATE_LIST):
                up_nodes.append(tl.emit(LayerNormDoubleMatVecSiLU(layer, blocks[c0 : c0 + MAX_UPGATE_LIST]), sm, o_nodes))
            for k, b in enumerate(blocks):
                blk_done[b] = avail[sm] + (k + 1) * pair_cost
            if blocks:
                tl.t[sm] = avail[sm] + len(blocks) * pair_cost
        # ---- down-proj: a slice is released when its up/gate blocks are done ----
        d_slices = g.num_down_proj_col_splits()
        per_slice = R // 16
        releases = [max(blk_done[s * per_slice : (s + 1) * per_slice]) + m.hop for s in range(d_slices)]
        down_nodes, down_done = tl.sliced_phase(
            H // 16, d_slices, 16 * R * 2, releases, m.plain_setup,
            lambda s, e, sl, layer=layer: DownProjResidual(layer, s, e, sl), up_nodes,
        )
        last, release = down_nodes, down_done + m.hop
    if nlayers == g.num_hidden_layers:
        last, _ = tl.ranges_phase(
            g.vocab_size // 16, 16 * H * 2, release, m.rms_setup,
            lambda s, e: RMS_LM_Head(s, e), last,
        )
    return tl.nodes, DAG_Node(NoOp(), last)
