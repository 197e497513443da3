"""Admission policies: the three cases of the reference's tests/test_scheduler.py."""

from collections import deque

import torch

from quic_cu_b200.scheduler import ContinuousAdmissionPolicy, StaticAdmissionPolicy
from quic_cu_b200.sequence import SequenceState


def _seq(rid, max_tokens=10, generated=()):
    s = SequenceState(prompt_tokens=torch.tensor([[rid]]), request_id=rid, max_tokens=max_tokens)
    s.generated_tokens = list(generated)
    return s


def test_static_scheduler_admits_when_empty():
    decision = StaticAdmissionPolicy().decide(running=[], waiting=deque([_seq(1), _seq(2)]), max_batch_size=2)
    assert len(decision.admit) == 2 and len(decision.release) == 0


def test_static_scheduler_blocks_while_any_running():
    decision = StaticAdmissionPolicy().decide(running=[_seq(1, generated=[1, 2])], waiting=deque([_seq(2)]),
                                              max_batch_size=2)
    assert len(decision.admit) == 0 and len(decision.release) == 0


def test_continuous_scheduler_admits_into_vacant_slots():
    running = [_seq(1, max_tokens=2, generated=[10, 20]), _seq(2, generated=[30])]
    decision = ContinuousAdmissionPolicy().decide(running=running, waiting=deque([_seq(3), _seq(4)]),
                                                  max_batch_size=2)
    assert [s.request_id for s in decision.release] == [1]
    assert [s.request_id for s in decision.admit] == [3]


def test_sequence_state_finish_rule_and_equality():
    a, b = _seq(1, max_tokens=2), _seq(1, max_tokens=2)
    assert a == b and not a.is_finished
    a.generated_tokens.append(5)
    assert a != b
    a.finished_at = 0
    assert a.is_finished
    b.generated_tokens = [1, 2]
    assert b.is_finished
