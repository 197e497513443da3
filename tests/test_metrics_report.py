"""Metrics registry (src/metrics.py) and benchmark report schema (benchmarks/collect.py,
benchmarks/report.py) of the reference, as mirrored by this package.  CPU only."""

import json
import math
import threading

from quic_cu_b200 import report
from quic_cu_b200.engine import Engine
from quic_cu_b200.config import EngineConfig
from quic_cu_b200.metrics import MetricsRegistry, Span, Timer

from tests.fake_model import FakeModule


def test_spans_nest_and_dump_as_a_tree(tmp_path):
    reg = MetricsRegistry()
    with Span("request run", reg):
        with Span("scheduling", reg):
            pass
        with Span("step", reg):
            with Span("forward_pass", reg):
                pass
    with Timer("load", reg):
        pass
    tree = reg.dump_json(str(tmp_path / "m.json"))
    assert json.load(open(tmp_path / "m.json")) == tree
    assert [t["name"] for t in tree["timers"]] == ["load"]
    assert len(tree["spans"]) == 1
    root = tree["spans"][0]
    assert root["name"] == "request run" and root["duration"] >= 0
    assert [c["name"] for c in root["children_spans"]] == ["scheduling", "step"]
    assert "children_spans" not in root["children_spans"][0]
    assert [c["name"] for c in root["children_spans"][1]["children_spans"]] == ["forward_pass"]
    assert reg.summary()["step"]["count"] == 1


def test_without_registry_nothing_is_recorded_and_nothing_nests():
    reg = MetricsRegistry()
    with Span("outer"):  # no registry: not on the stack (src/metrics.py:112-113)
        with Span("inner", reg):
            pass
    with Timer("t"):
        pass
    tree = reg.to_json()
    assert tree == {"timers": [], "spans": [{"name": "inner", "duration": tree["spans"][0]["duration"]}]}


def test_span_stacks_are_per_thread():
    reg = MetricsRegistry()
    started, release = threading.Event(), threading.Event()

    def worker():
        with Span("worker", reg):
            started.set()
            release.wait(5)

    t = threading.Thread(target=worker)
    t.start()
    started.wait(5)
    with Span("main", reg):  # opened while "worker" is open on another thread
        pass
    release.set()
    t.join()
    assert sorted(s["name"] for s in reg.to_json()["spans"]) == ["main", "worker"]


def test_engine_feeds_the_registry_with_the_reference_span_names():
    reg = MetricsRegistry()
    engine = Engine(registry=reg, max_batch_size=2, config=EngineConfig(batching="continuous", max_context=64),
                    model_module=FakeModule(None))
    engine.max_tokens = 3
    for prompt in ([1, 2, 3], [4, 5], [6]):
        engine.add_request_ids(prompt)
    assert len(engine.run()) == 3
    tree = reg.to_json()
    assert [s["name"] for s in tree["spans"]] == ["request run"]  # src/engine.py:112
    names = {c["name"] for c in tree["spans"][0]["children_spans"]}
    assert {"scheduling", "prefill", "step"} <= names  # src/engine.py:114,144,79
    step = next(c for c in tree["spans"][0]["children_spans"] if c["name"] == "step")
    assert [c["name"] for c in step["children_spans"]] == ["prepare_decode", "forward_pass", "sample_and_update"]


def _rows():
    return [{"batch": 1, "context": 128, "ttft_ms": 1.5, "decode_tps": 2800.0, "peak_vram_mb": 900.0, "note": "x"},
            {"batch": 4, "context": 512, "ttft_ms": 5.4, "decode_tps": 4700.0, "peak_vram_mb": 950.0}]


def _batching(policy):
    return {"policy": policy, "max_batch_size": 4, "num_requests": 8, "total_tokens": 256, "elapsed_s": 0.05,
            "throughput_tps": 5120.0, "peak_vram_mb": 1000.0}


def test_results_follow_the_collector_schema(tmp_path):
    data = report.collect_results({"quic_quant": _rows()}, {p: _batching(p) for p in ("static", "continuous")})
    assert list(data) == ["quic_quant", "engine_batching"]
    assert list(data["quic_quant"]) == ["B1_C128", "B4_C512"]
    assert set(data["quic_quant"]["B1_C128"]) == {"ttft_ms", "decode_tps", "peak_vram_mb"}
    assert set(data["engine_batching"]["static"]) == set(report.BATCHING_KEYS)
    path = report.write_results(data, str(tmp_path / "results"))
    assert path.endswith("benchmark_results.json") and json.load(open(path)) == data


def test_markdown_report_tables(tmp_path):
    data = report.collect_results({"quic_quant": _rows(), "hf_quant": _rows()[:1]}, {"static": _batching("static")})
    data["hf_quant"]["B4_C512"] = report.failed_entry()
    json_path = report.write_results(data, str(tmp_path))
    text = report.generate_markdown_report(json_path, str(tmp_path / "REPORT.md"))
    assert open(tmp_path / "REPORT.md").read() == text
    lines = text.splitlines()
    assert lines[0] == "# QUIC 4-Path Benchmark Summary Report"
    assert lines[2] == ("| Batch | Context | quic_quant TTFT (ms) | hf_quant TTFT (ms) | quic_quant Dec TPS | "
                        "hf_quant Dec TPS | quic_quant VRAM (MB) | hf_quant VRAM (MB) |")
    assert lines[4] == "| 1 | 128 | 1.5 | 1.5 | 2800.0 | 2800.0 | 900.0 | 900.0 |"
    assert lines[5] == "| 4 | 512 | 5.4 | OOM | 4700.0 | OOM | 950.0 | OOM |"
    assert "| static | 4 | 8 | 256 | 0.05 | 5120.0 | 1000.0 |" in lines
    assert math.isnan(report.failed_entry()["ttft_ms"])
