"""Timers and nested spans around the engine's phases.

Same interface and JSON as the reference's registry (src/metrics.py:38-131):
``MetricsRegistry.add_timer / add_span / dump_json(file) -> {"timers": [...], "spans": [tree]}``,
``Timer(name, registry)`` and ``Span(name, registry)`` context managers that record nothing
when no registry is given.  A span opened inside another becomes its child
(``children_spans`` in the dump).  Differences: the stack of open spans is kept per thread
(the reference's is one class-level list, src/metrics.py:99), the tree is built in one pass
over an index instead of a scan per node, and ``summary()`` adds per-name totals.
"""

from __future__ import annotations

import itertools
import json
import threading
import time
from collections import defaultdict

_span_ids = itertools.count(1)
_open = threading.local()


def _stack() -> list:
    if not hasattr(_open, "spans"):
        _open.spans = []
    return _open.spans


class MetricsRegistry:
    def __init__(self) -> None:
        self._timers: list[dict] = []
        self._spans: list[dict] = []

    def add_timer(self, timer_log: dict) -> None:
        self._timers.append({"name": timer_log["name"], "duration": float(timer_log["duration"])})

    def add_span(self, span_log: dict) -> None:
        self._spans.append({"id": span_log["id"], "name": span_log["name"],
                            "duration": float(span_log["duration"]), "parent_id": span_log.get("parent_id")})

    def record(self, name: str, seconds: float) -> None:
        """A flat timer entry (shorthand for ``add_timer``)."""
        self.add_timer({"name": name, "duration": seconds})

    def to_json(self) -> dict:
        children: dict = defaultdict(list)
        for span in self._spans:
            children[span["parent_id"]].append(span)

        def node(span: dict) -> dict:
            out = {"name": span["name"], "duration": span["duration"]}
            kids = children.get(span["id"])
            if kids:
                out["children_spans"] = [node(k) for k in kids]
            return out

        return {"timers": [dict(t) for t in self._timers], "spans": [node(s) for s in children.get(None, [])]}

    def dump_json(self, file_name: str) -> dict:
        tree = self.to_json()
        with open(file_name, "w") as handle:
            json.dump(tree, handle, indent=4)
        return tree

    def summary(self) -> dict:
        """Total seconds and count per span / timer name."""
        totals: dict = defaultdict(lambda: {"seconds": 0.0, "count": 0})
        for entry in itertools.chain(self._spans, self._timers):
            slot = totals[entry["name"]]
            slot["seconds"] += entry["duration"]
            slot["count"] += 1
        return dict(totals)


class Timer:
    def __init__(self, name: str, registry: MetricsRegistry | None = None) -> None:
        self.name, self.registry = name, registry
        self.start_time = self.end_time = 0.0

    def __enter__(self) -> "Timer":
        if self.registry is not None:
            self.start_time = time.perf_counter()
        return self

    def __exit__(self, *exc) -> None:
        if self.registry is not None:
            self.end_time = time.perf_counter()
            self.registry.add_timer({"name": self.name, "duration": self.end_time - self.start_time})


class Span:
    def __init__(self, name: str, registry: MetricsRegistry | None = None) -> None:
        self.id = next(_span_ids)
        self.name, self.registry = name, registry
        self.parent_id: int | None = None
        self.start_time = self.end_time = 0.0

    def __enter__(self) -> "Span":
        if self.registry is None:
            return self
        stack = _stack()
        if stack:
            self.parent_id = stack[-1].id
        stack.append(self)
        self.start_time = time.perf_counter()
        return self

    def __exit__(self, *exc) -> None:
        if self.registry is None:
            return
        self.end_time = time.perf_counter()
        stack = _stack()
        if stack and stack[-1] is self:
            stack.pop()
        self.registry.add_span({"id": self.id, "name": self.name, "duration": self.end_time - self.start_time,
                                "parent_id": self.parent_id})
