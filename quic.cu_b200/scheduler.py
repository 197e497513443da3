"""Slot admission policies (same decisions as the reference's src/scheduler.py:11-65).

``decide`` looks at the running rows and the FIFO of waiting requests and says which
finished rows to release and which waiting requests to admit:

* static: nothing happens while any row is still generating; when all rows are finished
  they are released together and up to ``max_batch_size`` requests are admitted
  (src/scheduler.py:28-46);
* continuous: finished rows are released at once and every vacant slot is refilled from
  the head of the queue (src/scheduler.py:49-65).
"""

from __future__ import annotations

from abc import ABC, abstractmethod
from collections import deque
from dataclasses import dataclass
from itertools import islice

from .sequence import SequenceState


@dataclass
class AdmissionDecision:
    release: list[SequenceState]
    admit: list[SequenceState]


class BatchAdmissionPolicy(ABC):
    @abstractmethod
    def decide(self, running: list[SequenceState], waiting: deque[SequenceState],
               max_batch_size: int) -> AdmissionDecision:
        ...


def _split(running: list[SequenceState]) -> tuple[list[SequenceState], int]:
    done = [seq for seq in running if seq.is_finished]
    return done, len(running) - len(done)


class StaticAdmissionPolicy(BatchAdmissionPolicy):
    def decide(self, running, waiting, max_batch_size) -> AdmissionDecision:
        done, alive = _split(running)
        if alive:
            return AdmissionDecision([], [])
        return AdmissionDecision(done, list(islice(waiting, min(len(waiting), max_batch_size))))


class ContinuousAdmissionPolicy(BatchAdmissionPolicy):
    def decide(self, running, waiting, max_batch_size) -> AdmissionDecision:
        done, alive = _split(running)
        room = max(0, min(len(waiting), max_batch_size - alive))
        return AdmissionDecision(done, list(islice(waiting, room)))
