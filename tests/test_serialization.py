"""Queue tensors and the instruction wire format (reference
tests/test_thor_serialization.py:9-35, tests/test_thor_worker_budget.py:5-21)."""
from types import SimpleNamespace
from unittest.mock import patch

import pytest

from thor_megakernels_b200.demos.latency import instructions as li
from thor_megakernels_b200.instructions import BaseGlobals, NoOp
from thor_megakernels_b200.scheduler import serialize_and_pad, tensorize_instructions


def globs(workers):
    return SimpleNamespace(sm_count=lambda: workers, device="cpu")


def test_nonsquare_queues_padding_and_input_immutability():
    queues = [[NoOp()], [NoOp(), NoOp(), NoOp()], []]
    g = globs(3)
    tensorize_instructions(g, queues)
    assert tuple(g.instructions.shape) == (3, 3, 32)
    assert tuple(g.timings.shape) == (3, 3, 128)
    assert [len(q) for q in queues] == [1, 3, 0]
    assert g.instructions.count_nonzero().item() == 0


def test_empty_queues_have_explicit_zero_length():
    g = globs(2)
    tensorize_instructions(g, [[], []])
    assert tuple(g.instructions.shape) == (2, 0, 32)


def test_invalid_queue_count_and_oversize_instruction():
    with pytest.raises(ValueError):
        tensorize_instructions(globs(2), [[]])
    with pytest.raises(ValueError):
        serialize_and_pad(SimpleNamespace(serialize=lambda: [1] * 33))


def test_word_layouts():
    assert li.LayerNorm_QKV_MatVecRopeAppend(3, 4, 6).serialize() == [1, 3, 4, 6]
    assert li.PartialAttention(1, 2, 8, 5).serialize() == [2, 1, 2, 8, 5]
    assert li.AttentionReduction(1, 4, 3, True, [0, 1, 2], None).serialize() == [3, 1, 4, 3, 1, 3, 0, 1, 2, 0]
    assert li.O_ProjResidual(0, 7, 8, 0).serialize() == [4, 0, 7, 8, 0]
    assert li.LayerNormDoubleMatVecSiLU(2, [5, 153, 301]).serialize() == [5, 2, 3, 5, 153, 301]
    assert li.DownProjResidual(2, 10, 13, 3).serialize() == [6, 2, 10, 13, 3]
    assert li.RMS_LM_Head(54, 108).serialize() == [7, 54, 108]
    assert serialize_and_pad(NoOp()) == [0] * 32


def test_mixed_queue_tensor_contents():
    g = globs(2)
    tensorize_instructions(g, [[li.RMS_LM_Head(0, 2)], [li.O_ProjResidual(1, 2, 3, 0), NoOp()]])
    assert g.instructions[0, 0, :3].tolist() == [7, 0, 2]
    assert g.instructions[0, 1].count_nonzero().item() == 0
    assert g.instructions[1, 0, :5].tolist() == [4, 1, 2, 3, 0]


@patch.object(BaseGlobals, "physical_sm_count", return_value=20)
def test_residency_and_queue_invalidation(_physical):
    g = BaseGlobals.__new__(BaseGlobals)
    g.__post_init__()
    g.set_active_workers(20)
    instructions, timings = object(), object()
    g.instructions, g.timings = instructions, timings
    for value in (None, True, 1.5, 0, 21):
        with pytest.raises(ValueError):
            g.set_active_workers(value)
        assert g.sm_count() == 20
        assert g.instructions is instructions
        assert g.timings is timings
    g.set_active_workers(3)
    assert g.sm_count() == 3
    assert g.instructions is None and g.timings is None
