"""Reader of the megakernel's per-instruction timing trace.

The kernel, when launched with ``record_timings=True``, stamps event times
(low 32 bits of the GPU's nanosecond timer) into ``globs.timings[sm, slot]`` at
the slots listed in ``include/mkb200.h`` (``MKB_T_*``).  The reference records
a similar trace (include/util.cuh:190-246) but only pickles it
(scripts/diff_test.py:231-242); this module turns it into per-opcode phase
statistics and a per-layer timeline.
"""

from __future__ import annotations

from collections import defaultdict

import torch

T_CONSUMER_START, T_WAIT_DONE, T_ACT_READY, T_FIRST_STAGE, T_CONSUMER_DONE = 0, 1, 2, 3, 4
T_LOADER_START, T_LOADER_DONE, T_STORER_START, T_STORER_DONE = 8, 9, 16, 17

OP_NAMES = {
    1: "qkv_rope_append",
    2: "partial_attention",
    3: "attention_reduction",
    4: "o_proj_residual",
    5: "upgate_silu",
    6: "down_proj_residual",
    7: "lm_head",
    8: "tp_all_reduce",
    9: "rms_norm",
}


def _layer_of(words) -> int:
    return int(words[1]) if int(words[0]) != 7 else -1


def summarize(globs) -> dict:
    """Per-opcode mean phase durations (us) and per-(layer, opcode) wall spans."""
    ins = globs.instructions.cpu()
    tim = globs.timings.cpu().to(torch.int64) & 0xFFFFFFFF
    valid = ins[:, :, 0] != 0
    t0 = int(tim[:, :, T_CONSUMER_START][valid].min())
    per_op = defaultdict(lambda: defaultdict(list))
    spans = defaultdict(lambda: [float("inf"), 0.0, float("inf"), 0.0])
    n_sm, qlen = ins.shape[0], ins.shape[1]
    for sm in range(n_sm):
        for i in range(qlen):
            op = int(ins[sm, i, 0])
            if op == 0:
                continue
            t = tim[sm, i]
            us = lambda slot: (int(t[slot]) - t0) / 1e3  # noqa: E731
            d = per_op[op]
            d["wait"].append(us(T_WAIT_DONE) - us(T_CONSUMER_START))
            if op in (1, 4, 5, 6, 7) and getattr(globs, "batch_size", 1) > 8:
                # tcgen05 build: the second loader waits for the producer, one thread issues the MMAs
                # (slot 5: all issued), four warps run the epilogues (slot 6: first accumulator
                # complete, slot 7: last epilogue done)
                d["first_stage"].append(us(T_FIRST_STAGE) - us(T_WAIT_DONE))
                d["mma_issue"].append(us(5) - us(T_FIRST_STAGE))
                d["first_accumulator"].append(us(6) - us(T_FIRST_STAGE))
                d["epilogue_after_issue"].append(us(7) - us(5))
                d["tail"].append(us(T_CONSUMER_DONE) - us(7))
            elif op in (1, 4, 5, 6, 7):
                d["activation"].append(us(T_ACT_READY) - us(T_WAIT_DONE))
                if op in (1, 5, 7) and getattr(globs, "batch_size", 1) == 1:
                    d["act:load"].append(us(6) - us(T_WAIT_DONE))
                    d["act:sync"].append(us(7) - us(6))
                    d["act:norm"].append(us(T_ACT_READY) - us(7))
                d["first_stage"].append(us(T_FIRST_STAGE) - us(T_ACT_READY))
                d["stream"].append(us(T_CONSUMER_DONE) - us(T_FIRST_STAGE))
                d["loader_lead"].append(us(T_CONSUMER_START) - us(T_LOADER_START))
                d["storer_tail"].append(us(T_STORER_DONE) - us(T_CONSUMER_DONE))
            elif op == 2:
                d["stages"].append(us(5) - us(T_WAIT_DONE))
                d["merge_store"].append(us(T_CONSUMER_DONE) - us(5))
            elif op == 8:
                d["send"].append(us(5) - us(T_WAIT_DONE))
                if int(t[6]) != 0:  # only the chunk's owner waits for arrivals and broadcasts
                    d["arrivals"].append(us(6) - us(5))
                    d["reduce_bcast"].append(us(T_CONSUMER_DONE) - us(6))
            elif op == 9:  # batched launches: one sequence's RMSNorm for all SMs
                d["load"].append(us(6) - us(T_WAIT_DONE))
                d["sync"].append(us(7) - us(6))
                d["norm_store_signal"].append(us(T_CONSUMER_DONE) - us(7))
            else:
                d["work"].append(us(T_CONSUMER_DONE) - us(T_WAIT_DONE))
            key = (_layer_of(ins[sm, i]), op)
            s = spans[key]
            s[0] = min(s[0], us(T_CONSUMER_START))
            s[1] = max(s[1], us(T_CONSUMER_DONE))
            s[2] = min(s[2], us(T_WAIT_DONE))
            s[3] = max(s[3], us(T_WAIT_DONE))
    stats = {
        OP_NAMES[op]: {k: (sum(v) / len(v), max(v), len(v)) for k, v in d.items()}
        for op, d in sorted(per_op.items())
    }
    total = (int(tim[:, :, T_CONSUMER_DONE][valid].max()) - t0) / 1e3
    return {"stats": stats, "spans": dict(spans), "total_us": total}


def format_summary(summary: dict, layers=(1,)) -> str:
    lines = [f"kernel span {summary['total_us']:.1f} us"]
    lines.append("per opcode: phase mean / max (us) over instructions")
    for name, d in summary["stats"].items():
        parts = [f"{k} {m:.2f}/{mx:.2f}" for k, (m, mx, _) in d.items()]
        n = max(v[2] for v in d.values())
        lines.append(f"  {name:20s} n={n:5d}  " + "  ".join(parts))
    for layer in layers:
        lines.append(f"layer {layer}: first start .. last done | barrier satisfied first .. last (us)")
        for (l, op), s in sorted(summary["spans"].items()):
            if l == layer:
                lines.append(
                    f"  {OP_NAMES[op]:20s} {s[0]:9.2f} .. {s[1]:9.2f} | {s[2]:9.2f} .. {s[3]:9.2f}"
                )
    return "\n".join(lines)
