"""Dependency graph of instructions, worker assignment, and the queue tensors
the kernel reads.

API-compatible with the reference's ``megakernels/scheduler.py``: ``DAG_Node``
(:16-46), ``Schedule`` (:49-63), ``ScheduleBuilder`` (:66-91), the assignment
policies ``rr`` / ``zz`` / ``wave`` / ``dag`` / ``pool`` (:94-163, :224-369),
``validate_queues`` (:166-221), ``serialize_and_pad`` (:372-377) and
``tensorize_instructions`` (:380-413).  For equal inputs every policy yields
the same queues as the reference, so an instruction tensor built here is
interchangeable with one built there.
"""
from __future__ import annotations

import heapq
from dataclasses import dataclass, field, replace
from typing import TYPE_CHECKING

if TYPE_CHECKING:  # pragma: no cover
    from .instructions import BaseGlobals, Instruction

INTS_PER_INSTRUCTION = 32
TIMING_SLOTS = 128


@dataclass(eq=False)
class DAG_Node:
    instruction: "Instruction"
    dependencies: list["DAG_Node"]

    children: set["DAG_Node"] = field(default_factory=set)
    start_time: float = float("inf")
    end_time: float = float("inf")
    remaining_dependencies: set["DAG_Node"] = field(default_factory=set)
    priority: float = 0

    def __hash__(self):
        return id(self)

    def earliest_ready_time(self, globs) -> float:
        return max((d.end_time for d in self.dependencies), default=0)

    def register_with_parents(self):
        for parent in self.dependencies:
            parent.children.add(self)

    def calc_priority(self, globs):
        for parent in self.dependencies:
            parent.priority = max(parent.priority, self.priority + parent.instruction.cost(globs))
            parent.calc_priority(globs)


@dataclass
class Schedule:
    globs: "BaseGlobals"
    dag_nodes: list[DAG_Node]
    end_node: DAG_Node

    def get_linear_instructions(self):
        """Instructions in DAG-list order, which builders keep topological."""
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


# ---------------------------------------------------------------------------
# assignment policies
# ---------------------------------------------------------------------------

def _require_workers(count: int):
    if count <= 0:
        raise ValueError("active worker count must be positive")


def _check_closed_graph(nodes: list[DAG_Node]) -> set[DAG_Node]:
    members = set(nodes)
    if len(members) != len(nodes):
        raise ValueError("duplicate DAG node")
    for n in nodes:
        for parent in n.dependencies:
            if parent not in members:
                raise ValueError("dependency missing from schedule")
    return members


def assign_dag_to_sms(schedule: Schedule) -> list[list["Instruction"]]:
    """List scheduling: the costliest ready instruction goes to the worker that
    frees up first (reference scheduler.py:94-163)."""
    nodes, globs = schedule.dag_nodes, schedule.globs
    workers = globs.sm_count()
    _require_workers(workers)
    _check_closed_graph(nodes)

    for n in nodes:
        n.children.clear()
        n.start_time = n.end_time = float("inf")
    for n in nodes:
        n.register_with_parents()
        n.remaining_dependencies = set(n.dependencies)

    index_of = {n: i for i, n in enumerate(nodes)}
    queues: list[list] = [[] for _ in range(workers)]
    free_at = [(0, w) for w in range(workers)]
    heapq.heapify(free_at)
    ready = [(-n.instruction.cost(globs), i) for i, n in enumerate(nodes) if not n.dependencies]
    heapq.heapify(ready)

    placed = 0
    while ready:
        _, i = heapq.heappop(ready)
        node = nodes[i]
        worker_time, w = heapq.heappop(free_at)
        node.start_time = max(worker_time, node.earliest_ready_time(globs))
        node.end_time = node.start_time + node.instruction.cost(globs)
        queues[w].append(node.instruction)
        placed += 1
        heapq.heappush(free_at, (node.end_time, w))
        for child in node.children:
            child.remaining_dependencies.remove(node)
            if not child.remaining_dependencies:
                heapq.heappush(ready, (-child.instruction.cost(globs), index_of[child]))

    if placed != len(nodes):
        raise ValueError("dependency graph contains a cycle")
    validate_queues(schedule, queues)
    return queues


def validate_queues(schedule: Schedule, queues: list[list["Instruction"]]) -> None:
    """Check that the queues cover every DAG node exactly once and that the DAG
    edges together with each queue's program order admit a topological order
    (i.e. an in-order worker can never wait for work queued behind it).
    Padding entries must have opcode 0.  (reference scheduler.py:166-221)"""
    if not queues or len(queues) != schedule.globs.sm_count():
        raise ValueError("queue count must equal positive active worker count")
    nodes = schedule.dag_nodes
    members = _check_closed_graph(nodes)

    node_of = {}
    for n in nodes:
        key = id(n.instruction)
        if key in node_of:
            raise ValueError("DAG operations must have distinct instruction objects")
        node_of[key] = n

    successors = {n: set() for n in nodes}
    for n in nodes:
        for parent in n.dependencies:
            successors[parent].add(n)

    assigned = set()
    for q in queues:
        last = None
        for ins in q:
            n = node_of.get(id(ins))
            if n is None:
                if ins.opcode() != 0:
                    raise ValueError("queue contains an unknown operation")
                continue
            if n in assigned:
                raise ValueError("operation assigned more than once")
            assigned.add(n)
            if last is not None:
                successors[last].add(n)
            last = n
    if assigned != members:
        raise ValueError("schedule has unassigned operations")

    indegree = dict.fromkeys(nodes, 0)
    for outs in successors.values():
        for n in outs:
            indegree[n] += 1
    frontier = [n for n in nodes if indegree[n] == 0]
    done = 0
    while frontier:
        n = frontier.pop()
        done += 1
        for m in successors[n]:
            indegree[m] -= 1
            if indegree[m] == 0:
                frontier.append(m)
    if done != len(nodes):
        raise ValueError("DAG plus worker queue ordering contains a deadlock cycle")


def round_robin_assign_to_sms(instructions, sm_count: int):
    _require_workers(sm_count)
    queues = [[] for _ in range(sm_count)]
    for i, ins in enumerate(instructions):
        queues[i % sm_count].append(ins)
    return queues


def row_keeping_assign_to_sms(instructions, sm_count: int):
    """Round robin, except that instructions which reduce different column
    slices into the SAME output rows of a layer (``reduction_block_idx`` differs,
    layer and row blocks equal) all go to the worker that got the first of them.
    With a builder that lists the slices of a row range one after the other
    (``down_rows_together``), a worker then holds every slice of its rows in
    slice order and can add them up itself.  Not a reference policy."""
    _require_workers(sm_count)
    queues = [[] for _ in range(sm_count)]
    home: dict = {}
    cursor = 0
    for ins in instructions:
        if hasattr(ins, "reduction_block_idx"):
            key = (type(ins), ins.layer_idx, ins.start_block_idx, ins.end_block_idx)
            if key not in home:
                home[key] = cursor % sm_count
                cursor += 1
            queues[home[key]].append(ins)
        else:
            queues[cursor % sm_count].append(ins)
            cursor += 1
    return queues


def zig_zag_assign_to_sms(instructions, sm_count: int):
    """Boustrophedon order: 0..n-1, n-1..0, 0..n-1, ..."""
    _require_workers(sm_count)
    queues = [[] for _ in range(sm_count)]
    period = 2 * sm_count
    for i, ins in enumerate(instructions):
        p = i % period
        queues[p if p < sm_count else period - 1 - p].append(ins)
    return queues


def collect_into_waves(instructions):
    """Split the linear order into maximal runs of one opcode."""
    waves: list[list] = []
    for ins in instructions:
        if waves and waves[-1][-1].opcode() == ins.opcode():
            waves[-1].append(ins)
        else:
            waves.append([ins])
    return waves


def wave_assign_to_sms(schedule: Schedule):
    """Per opcode wave, longest-processing-time-first onto the least loaded
    worker, never placing an instruction before a same-wave producer
    (reference scheduler.py:270-318)."""
    globs = schedule.globs
    workers = globs.sm_count()
    queues = [[] for _ in range(workers)]
    load = [(0, w) for w in range(workers)]
    heapq.heapify(load)
    node_of = {id(n.instruction): n for n in schedule.dag_nodes}

    for wave in collect_into_waves(schedule.get_linear_instructions()):
        nodes = [node_of[id(ins)] for ins in wave]
        inside = set(nodes)
        slot = {n: i for i, n in enumerate(nodes)}
        waiting = {}
        kids = {n: [] for n in nodes}
        for n in nodes:
            parents = set(n.dependencies) & inside
            waiting[n] = len(parents)
            for p in parents:
                kids[p].append(n)
        ready = [(-n.instruction.cost(globs), slot[n]) for n in nodes if waiting[n] == 0]
        heapq.heapify(ready)
        placed = 0
        while ready:
            _, i = heapq.heappop(ready)
            n = nodes[i]
            cost_so_far, w = heapq.heappop(load)
            heapq.heappush(load, (cost_so_far + n.instruction.cost(globs), w))
            queues[w].append(n.instruction)
            placed += 1
            for c in kids[n]:
                waiting[c] -= 1
                if waiting[c] == 0:
                    heapq.heappush(ready, (-c.instruction.cost(globs), slot[c]))
        if placed != len(nodes):
            raise ValueError("dependency cycle within opcode wave")
    return queues


def pool_assign_to_sms(instructions, sm_count: int, memory_fraction: float):
    """Dedicated worker pools for memory-tagged and compute-tagged instructions."""
    pools = {"memory": [], "compute": []}
    for ins in instructions:
        tag = ins.tags()["pool"]
        if tag not in pools:
            raise ValueError(f"Unknown pool: {tag}")
        pools[tag].append(ins)
    mem_workers = round(sm_count * memory_fraction)
    return round_robin_assign_to_sms(pools["memory"], mem_workers) + round_robin_assign_to_sms(
        pools["compute"], sm_count - mem_workers
    )


def assign_to_sms(
    mode: str,
    schedule: Schedule | None = None,
    instructions=None,
    sm_count: int | None = None,
    memory_fraction: float | None = None,
):
    if schedule is not None:
        instructions = schedule.get_linear_instructions()
        sm_count = schedule.globs.sm_count()

    if mode == "rr":
        queues = round_robin_assign_to_sms(instructions, sm_count)
    elif mode == "rrk":
        queues = row_keeping_assign_to_sms(instructions, sm_count)
    elif mode == "zz":
        queues = zig_zag_assign_to_sms(instructions, sm_count)
    elif mode == "wave":
        queues = wave_assign_to_sms(schedule)
    elif mode == "dag":
        queues = assign_dag_to_sms(schedule)
    elif mode == "pool":
        if memory_fraction is None:
            raise ValueError("pool scheduler requires memory_fraction")
        queues = pool_assign_to_sms(instructions, sm_count, memory_fraction)
    else:
        raise ValueError(f"Unknown mode: {mode}")
    if schedule is not None:
        validate_queues(schedule, queues)
    return queues


# ---------------------------------------------------------------------------
# queue tensors
# ---------------------------------------------------------------------------

def serialize_and_pad(instruction) -> list[int]:
    words = instruction.serialize()
    if len(words) > INTS_PER_INSTRUCTION:
        raise ValueError("serialized instruction exceeds instruction width")
    return words + [0] * (INTS_PER_INSTRUCTION - len(words))


def tensorize_instructions(globs, instruction_queues):
    """Write ``globs.instructions`` (int32 ``[workers, len, 32]``, short queues
    padded with all-zero no-ops) and ``globs.timings`` (int32 zeros
    ``[workers, len, 128]``).  The queues passed in are left untouched."""
    import torch

    workers = globs.sm_count()
    if workers <= 0 or len(instruction_queues) != workers:
        raise ValueError("queue count must equal positive active worker count")
    depth = max(len(q) for q in instruction_queues)
    blank = [0] * INTS_PER_INSTRUCTION
    rows = []
    for q in instruction_queues:
        rows.extend(serialize_and_pad(ins) for ins in q)
        rows.extend(blank for _ in range(depth - len(q)))

    globs.instructions = torch.tensor(rows, dtype=torch.int32, device=globs.device).view(
        workers, depth, INTS_PER_INSTRUCTION
    )
    globs.timings = torch.zeros((workers, depth, TIMING_SLOTS), dtype=torch.int32, device=globs.device)
