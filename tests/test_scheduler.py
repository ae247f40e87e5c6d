"""Host-side scheduling rules, mirroring the reference's own unit tests
(tests/test_thor_scheduler.py:20-98): dependencies respected, cycles and missing
producers rejected, queue validation catches duplicates, omissions and
reversed order."""
import random
from types import SimpleNamespace

import pytest

from thor_megakernels_b200.scheduler import (
    DAG_Node,
    Schedule,
    assign_dag_to_sms,
    assign_to_sms,
    collect_into_waves,
    round_robin_assign_to_sms,
    validate_queues,
    wave_assign_to_sms,
    zig_zag_assign_to_sms,
)


class Op:
    def __init__(self, cost, code=1):
        self.duration = cost
        self.code = code

    def cost(self, globs):
        return self.duration

    def opcode(self):
        return self.code

    def serialize(self):
        return [self.code]


def schedule(nodes, workers=2):
    return Schedule(SimpleNamespace(sm_count=lambda: workers), nodes, nodes[-1])


def test_dependency_ready_time_and_repeat():
    a = DAG_Node(Op(100), [])
    b = DAG_Node(Op(1), [a])
    s = schedule([a, b])
    for _ in range(2):
        queues = assign_dag_to_sms(s)
        assert sum(map(len, queues)) == 2
        assert b.start_time >= a.end_time


def test_identical_serializations_are_distinct_nodes():
    nodes = [DAG_Node(Op(1), []) for _ in range(5)]
    assert sum(map(len, assign_dag_to_sms(schedule(nodes)))) == 5


def test_cycle_and_missing_producer():
    a = DAG_Node(Op(1), [])
    b = DAG_Node(Op(1), [a])
    with pytest.raises(ValueError):
        assign_dag_to_sms(schedule([b]))
    a.dependencies = [b]
    with pytest.raises(ValueError):
        assign_dag_to_sms(schedule([a, b]))


def test_wave_cost_order_respects_dependencies_within_opcode():
    a = DAG_Node(Op(1), [])
    b = DAG_Node(Op(100), [a])
    s = schedule([a, b], workers=1)
    queues = wave_assign_to_sms(s)
    assert queues == [[a.instruction, b.instruction]]
    validate_queues(s, queues)


def test_random_waves_remain_dependency_safe():
    rng = random.Random(19)
    for _ in range(100):
        nodes = []
        for _i in range(30):
            nodes.append(DAG_Node(Op(rng.randint(1, 1000)), [n for n in nodes if rng.random() < 0.1]))
        for workers in (1, 3, 7):
            s = schedule(nodes, workers)
            validate_queues(s, wave_assign_to_sms(s))


def test_reverse_queue_dependency_detected():
    a, b = DAG_Node(Op(1), []), DAG_Node(Op(1), [])
    b.dependencies = [a]
    s = Schedule(SimpleNamespace(sm_count=lambda: 1), [a, b], b)
    with pytest.raises(ValueError):
        validate_queues(s, [[b.instruction, a.instruction]])
    validate_queues(s, [[a.instruction, b.instruction]])


def test_duplicate_missing_and_random_dags():
    rng = random.Random(7)
    for _ in range(100):
        nodes = []
        for _i in range(25):
            nodes.append(DAG_Node(Op(rng.randint(1, 100)), [n for n in nodes if rng.random() < 0.12]))
        s = Schedule(SimpleNamespace(sm_count=lambda: 3), nodes, nodes[-1])
        queues = assign_dag_to_sms(s)
        validate_queues(s, queues)
        for n in nodes:
            for parent in n.dependencies:
                assert n.start_time >= parent.end_time
        broken = [list(q) for q in queues]
        broken[0].append(nodes[0].instruction)
        with pytest.raises(ValueError):
            validate_queues(s, broken)
        missing = [[ins for ins in q if ins is not nodes[0].instruction] for q in queues]
        with pytest.raises(ValueError):
            validate_queues(s, missing)


def test_round_robin_and_zig_zag_orders():
    items = list(range(7))
    assert round_robin_assign_to_sms(items, 3) == [[0, 3, 6], [1, 4], [2, 5]]
    assert zig_zag_assign_to_sms(items, 3) == [[0, 5, 6], [1, 4], [2, 3]]
    for fn in (round_robin_assign_to_sms, zig_zag_assign_to_sms):
        with pytest.raises(ValueError):
            fn(items, 0)


def test_waves_split_on_opcode_change():
    ops = [Op(1, 1), Op(1, 1), Op(1, 2), Op(1, 1)]
    assert [len(w) for w in collect_into_waves(ops)] == [2, 1, 1]


def test_unknown_mode_and_pool_requires_fraction():
    with pytest.raises(ValueError):
        assign_to_sms("nope", instructions=[], sm_count=1)
    with pytest.raises(ValueError):
        assign_to_sms("pool", instructions=[], sm_count=2)
