"""DAG of instructions -> per-SM instruction queues -> int32 tensor.

Reference: megakernels/scheduler.py.  Same public names and results:
``DAG_Node``/``Schedule``/``ScheduleBuilder`` (:17-91), the assignment modes
``rr``/``zz``/``wave``/``dag``/``pool`` (:94-271) and
``tensorize_instructions`` (:281-308).
"""

from __future__ import annotations

import heapq
from dataclasses import dataclass, field, replace

import torch

from megakernels_b200.instructions import BaseGlobals, Instruction, NoOp

INTS_PER_INSTRUCTION = 32
TIMING_SLOTS = 128


@dataclass(eq=False)
class DAG_Node:
    instruction: Instruction
    dependencies: list["DAG_Node"]
    children: set["DAG_Node"] = field(default_factory=set)
    start_time: float = float("inf")
    end_time: float = float("inf")
    remaining_dependencies: set["DAG_Node"] = field(default_factory=set)
    priority: float = 0

    def earliest_ready_time(self, globs: BaseGlobals):
        return max((d.end_time for d in self.dependencies), default=0)

    def register_with_parents(self):
        for d in self.dependencies:
            d.children.add(self)


@dataclass
class Schedule:
    globs: BaseGlobals
    dag_nodes: list[DAG_Node]
    end_node: DAG_Node

    def get_linear_instructions(self) -> list[Instruction]:
        # dag_nodes are emitted in topological order by the builders
        return [n.instruction for n in self.dag_nodes]

    def smart_assign_to_sms(self):
        return assign_dag_to_sms(self)

    def round_robin_assign_to_sms(self):
        return round_robin_assign_to_sms(self.get_linear_instructions(), self.globs.sm_count())


class ScheduleBuilder:
    @classmethod
    def make_globals(cls, model):
        raise NotImplementedError

    @classmethod
    def make_dag(cls, globs, stop_after_op: str | None = None, layer_limit: int | None = None):
        raise NotImplementedError

    @classmethod
    def build(cls, model, stop_after_op: str | None = None, layer_limit: int | None = None):
        globs = cls.make_globals(model)
        nodes, end = cls.make_dag(globs, stop_after_op, layer_limit)
        return Schedule(globs, nodes, end)

    @classmethod
    def with_new_globals(cls, schedule: Schedule, model):
        return replace(schedule, globs=cls.make_globals(model))


def assign_dag_to_sms(schedule: Schedule) -> list[list[Instruction]]:
    """Greedy list scheduling: most expensive ready node onto the SM that frees first.

    Reference: megakernels/scheduler.py:94-151 (ties are broken by node index
    and SM index through the heap tuples, which this keeps).
    """
    nodes, globs = schedule.dag_nodes, schedule.globs
    index = {id(n): i for i, n in enumerate(nodes)}
    for n in nodes:
        n.children = set()
    for n in nodes:
        n.register_with_parents()
        n.remaining_dependencies = set(n.dependencies)

    sm_count = globs.sm_count()
    queues: list[list[Instruction]] = [[] for _ in range(sm_count)]
    sm_heap = [(0, i) for i in range(sm_count)]
    heapq.heapify(sm_heap)
    ready = [(-n.instruction.cost(globs), i) for i, n in enumerate(nodes) if not n.dependencies]
    heapq.heapify(ready)

    while ready:
        _, i = heapq.heappop(ready)
        node = nodes[i]
        sm_time, sm = heapq.heappop(sm_heap)
        node.start_time = sm_time
        node.end_time = sm_time + node.instruction.cost(globs)
        queues[sm].append(node.instruction)
        heapq.heappush(sm_heap, (node.end_time, sm))
        for child in node.children:
            child.remaining_dependencies.remove(node)
            if not child.remaining_dependencies:
                heapq.heappush(ready, (-child.instruction.cost(globs), index[id(child)]))
    return queues


def round_robin_assign_to_sms(instructions: list[Instruction], sm_count: int):
    """Reference: megakernels/scheduler.py:154-161."""
    queues: list[list[Instruction]] = [[] for _ in range(sm_count)]
    for i, ins in enumerate(instructions):
        queues[i % sm_count].append(ins)
    return queues


def zig_zag_assign_to_sms(instructions: list[Instruction], sm_count: int):
    """Boustrophedon order over the SMs (reference: scheduler.py:164-176)."""
    queues: list[list[Instruction]] = [[] for _ in range(sm_count)]
    for i, ins in enumerate(instructions):
        k = i % (2 * sm_count)
        queues[k if k < sm_count else 2 * sm_count - 1 - k].append(ins)
    return queues


def collect_into_waves(instructions: list[Instruction]) -> list[list[Instruction]]:
    """Maximal runs of equal opcode (reference: scheduler.py:179-193)."""
    waves: list[list[Instruction]] = []
    for ins in instructions:
        if waves and waves[-1][-1].opcode() == ins.opcode():
            waves[-1].append(ins)
        else:
            waves.append([ins])
    return waves


def wave_assign_to_sms(schedule: Schedule):
    """Per wave, longest-processing-time first onto the least-loaded SM.

    The load is cumulative over waves, so the per-SM byte totals stay balanced
    over the whole token (reference: scheduler.py:196-221).
    """
    globs = schedule.globs
    sm_count = globs.sm_count()
    queues: list[list[Instruction]] = [[] for _ in range(sm_count)]
    heap = [(0, i) for i in range(sm_count)]
    heapq.heapify(heap)
    for wave in collect_into_waves(schedule.get_linear_instructions()):
        for ins in sorted(wave, key=lambda x: x.cost(globs), reverse=True):
            load, sm = heapq.heappop(heap)
            heapq.heappush(heap, (load + ins.cost(globs), sm))
            queues[sm].append(ins)
    return queues


def pool_assign_to_sms(instructions: list[Instruction], sm_count: int, memory_fraction: float):
    """Split SMs into a memory pool and a compute pool (scheduler.py:224-246)."""
    pools: dict[str, list[Instruction]] = {"memory": [], "compute": []}
    for ins in instructions:
        pool = ins.tags()["pool"]
        if pool not in pools:
            raise ValueError(f"Unknown pool: {pool}")
        pools[pool].append(ins)
    mem_sms = round(sm_count * memory_fraction)
    return round_robin_assign_to_sms(pools["memory"], mem_sms) + round_robin_assign_to_sms(
        pools["compute"], sm_count - mem_sms
    )


def assign_to_sms(
    mode: str,
    schedule: Schedule | None = None,
    instructions: list[Instruction] | None = None,
    sm_count: int | None = None,
    memory_fraction: float | None = None,
):
    """Reference: megakernels/scheduler.py:249-271."""
    if schedule is not None:
        instructions = schedule.get_linear_instructions()
        sm_count = schedule.globs.sm_count()
    if mode == "rr":
        return round_robin_assign_to_sms(instructions, sm_count)
    if mode == "zz":
        return zig_zag_assign_to_sms(instructions, sm_count)
    if mode == "wave":
        return wave_assign_to_sms(schedule)
    if mode == "dag":
        return assign_dag_to_sms(schedule)
    if mode == "pool":
        assert memory_fraction is not None
        return pool_assign_to_sms(instructions, sm_count, memory_fraction=memory_fraction)
    raise ValueError(f"Unknown mode: {mode}")


def serialize_and_pad(instruction: Instruction) -> list[int]:
    words = instruction.serialize()
    if len(words) > INTS_PER_INSTRUCTION:
        raise AssertionError(
            f"{type(instruction).__name__} needs {len(words)} words > {INTS_PER_INSTRUCTION}"
        )
    return words + [0] * (INTS_PER_INSTRUCTION - len(words))


def tensorize_instructions(globs: BaseGlobals, instruction_queues: list[list[Instruction]]):
    """Pad queues with NoOps and attach ``instructions``/``timings`` to ``globs``.

    ``instructions`` is int32 ``[num_sms, queue_len, 32]``; ``timings`` is
    int32 ``[num_sms, queue_len, 128]`` (reference: scheduler.py:281-308).
    """
    num_sms = globs.sm_count()
    assert len(instruction_queues) == num_sms
    qlen = max(1, max(len(q) for q in instruction_queues))
    for q in instruction_queues:
        q.extend([NoOp()] * (qlen - len(q)))
    flat = [serialize_and_pad(ins) for q in instruction_queues for ins in q]
    globs.instructions = torch.tensor(flat, dtype=torch.int32, device=globs.device).view(
        num_sms, qlen, INTS_PER_INSTRUCTION
    )
    globs.timings = torch.zeros(
        [num_sms, qlen, TIMING_SLOTS], dtype=torch.int32, device=globs.device
    )
