"""Wall-clock spans around engine phases (the hook the reference's engine carries,
src/metrics.py:78-131: ``Span(name, registry)`` context managers feeding a registry)."""

from __future__ import annotations

import json
import time
from collections import defaultdict


class MetricsRegistry:
    def __init__(self) -> None:
        self.totals: dict[str, float] = defaultdict(float)
        self.counts: dict[str, int] = defaultdict(int)

    def record(self, name: str, seconds: float) -> None:
        self.totals[name] += seconds
        self.counts[name] += 1

    def summary(self) -> dict:
        return {k: {"seconds": self.totals[k], "count": self.counts[k]} for k in self.totals}

    def dump_json(self, path: str) -> None:
        with open(path, "w") as handle:
            json.dump(self.summary(), handle, indent=1)


class Span:
    def __init__(self, name: str, registry: MetricsRegistry | None = None) -> None:
        self.name, self.registry = name, registry

    def __enter__(self):
        self._t0 = time.perf_counter()
        return self

    def __exit__(self, *exc):
        if self.registry is not None:
            self.registry.record(self.name, time.perf_counter() - self._t0)
        return False
