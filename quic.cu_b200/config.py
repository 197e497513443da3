"""Engine flags (the reference's EngineConfig, src/config.py:12-18, plus cache geometry)."""

from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Literal

MODEL_ROOT = os.environ.get("QWEN25_AWQ_PATH", os.environ.get("QWEN25_FP16_PATH", ""))


@dataclass(frozen=True)
class EngineConfig:
    batching: Literal["static", "continuous"] = "continuous"
    model_path: str | None = None
    tokenizer_path: str | None = None
    use_machete: bool = False  # accepted for compatibility; the Hopper-only backend is not built
    # kept for the reference's call sites ("pytorch" = torch SDPA, "quic" = its own kernel there);
    # here every value runs the library's causal prefill kernel, all admitted sequences in one launch
    prefill_backend: Literal["pytorch", "quic"] = "quic"
    # additions (defaults keep reference call sites valid)
    max_context: int = 2048   # tokens per KV slot (prompt + generated)
    decode_burst: int = 8     # greedy steps per graph launch between scheduling points
    # prefill newly admitted requests on a second CUDA stream while the rows already running
    # decode their next burst; the new rows join at the following iteration
    overlap_prefill: bool = True
    # chunked prefill: at most this many prompt tokens per sequence per iteration (None: the whole
    # prompt at once); the rows already running decode a burst between two chunks
    prefill_chunk: int | None = None
