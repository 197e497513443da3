"""Per-request state (same fields and finish rule as the reference's src/sequence.py:7-30)."""

from __future__ import annotations

from dataclasses import dataclass, field

import torch


@dataclass
class SequenceState:
    prompt_tokens: torch.Tensor  # [1, T] token ids
    request_id: int
    max_tokens: int
    generated_tokens: list[int] = field(default_factory=list)
    finished_at: int | None = None
    slot: int | None = None  # KV slot while the request is running (new: slotted cache)

    @property
    def is_finished(self) -> bool:
        """Finished once EOS was seen or ``max_tokens`` tokens exist (src/sequence.py:15-19)."""
        return self.finished_at is not None or len(self.generated_tokens) >= self.max_tokens

    def __eq__(self, other: object) -> bool:
        if not isinstance(other, SequenceState):
            return False
        return (
            self.request_id == other.request_id
            and self.max_tokens == other.max_tokens
            and self.finished_at == other.finished_at
            and self.generated_tokens == other.generated_tokens
            and torch.equal(self.prompt_tokens, other.prompt_tokens)
        )

    __hash__ = None  # type: ignore[assignment]
