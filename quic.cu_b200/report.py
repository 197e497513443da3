"""Benchmark results in the reference's JSON schema and its Markdown report.

The reference's collector writes ``benchmark_results.json`` as
``{path: {"B<batch>_C<context>": {"ttft_ms", "decode_tps", "peak_vram_mb"}}, "engine_batching":
{policy: {"policy", "max_batch_size", "num_requests", "total_tokens", "elapsed_s",
"throughput_tps", "peak_vram_mb"}}}`` (benchmarks/collect.py:106-117,170-178,243-247) and
its report turns that file into two Markdown tables (benchmarks/report.py:9-90).  The
functions here produce both from this library's own measurements, so result files of the two
code bases can be merged and reported side by side.
"""

from __future__ import annotations

import json
import math
import os

SWEEP_KEYS = ("ttft_ms", "decode_tps", "peak_vram_mb")
BATCHING_KEYS = ("policy", "max_batch_size", "num_requests", "total_tokens", "elapsed_s", "throughput_tps",
                 "peak_vram_mb")


def sweep_entry(ttft_ms: float, decode_tps: float, peak_vram_mb: float) -> dict:
    return {"ttft_ms": float(ttft_ms), "decode_tps": float(decode_tps), "peak_vram_mb": float(peak_vram_mb)}


def failed_entry() -> dict:
    """What the reference stores for a grid point that ran out of memory (benchmarks/collect.py:117)."""
    return sweep_entry(float("nan"), 0.0, float("nan"))


def collect_results(sweeps: dict[str, list[dict]], batching: dict[str, dict] | None = None) -> dict:
    """``sweeps``: execution path name -> rows with ``batch``, ``context`` and the three sweep keys.
    ``batching``: policy name -> a dict with the seven batching keys."""
    data: dict = {}
    for path_name, rows in sweeps.items():
        data[path_name] = {f"B{r['batch']}_C{r['context']}": sweep_entry(*(r[k] for k in SWEEP_KEYS)) for r in rows}
    if batching:
        for policy, info in batching.items():
            missing = [k for k in BATCHING_KEYS if k not in info]
            if missing:
                raise KeyError(f"engine_batching[{policy!r}] lacks {missing}")
        data["engine_batching"] = {p: {k: info[k] for k in BATCHING_KEYS} for p, info in batching.items()}
    return data


def write_results(data: dict, output_dir: str) -> str:
    os.makedirs(output_dir, exist_ok=True)
    json_path = os.path.join(output_dir, "benchmark_results.json")
    with open(json_path, "w") as handle:
        json.dump(data, handle, indent=2)
    return json_path


def _cell(value, oom: bool) -> str:
    return "OOM" if oom else f"{value:.1f}"


def _is_nan(value) -> bool:
    return value is None or (isinstance(value, float) and math.isnan(value))


def markdown_report(data: dict) -> str:
    """The reference's two tables: one row per grid point with TTFT, decode rate and peak memory
    of every path side by side, then one row per batching policy."""
    sections = []
    paths = [name for name in data if name != "engine_batching"]
    if paths:
        def header(label: str) -> str:
            return " | ".join(f"{p} {label}" for p in paths)

        n_cols = 3 * len(paths)
        lines = ["# QUIC 4-Path Benchmark Summary Report\n",
                 f"| Batch | Context | {header('TTFT (ms)')} | {header('Dec TPS')} | {header('VRAM (MB)')} |",
                 "| :---: | :---: | " + " | ".join([":---:"] * n_cols) + " |"]
        for key in data[paths[0]]:
            batch, context = key.split("_")
            cells = []
            for p in paths:
                point = data[p].get(key, failed_entry())
                cells.append(_cell(point["ttft_ms"], _is_nan(point["ttft_ms"])))
            for p in paths:
                point = data[p].get(key, failed_entry())
                cells.append(_cell(point["decode_tps"], not point["decode_tps"] > 0))
            for p in paths:
                point = data[p].get(key, failed_entry())
                vram = point.get("peak_vram_mb")
                cells.append(_cell(vram, _is_nan(vram) or not vram))
            lines.append(f"| {batch[1:]} | {context[1:]} | " + " | ".join(cells) + " |")
        sections.append("\n".join(lines))
    if "engine_batching" in data:
        lines = ["## Serving Engine Batching Policies (Static vs Continuous)\n",
                 "| Policy | Max Batch Size | Requests | Total Tokens | Latency (s) | Throughput (tok/s) | "
                 "Peak VRAM (MB) |",
                 "| :---: | :---: | :---: | :---: | :---: | :---: | :---: |"]
        for info in data["engine_batching"].values():
            lines.append(f"| {info['policy']} | {info['max_batch_size']} | {info['num_requests']} | "
                         f"{info['total_tokens']} | {info['elapsed_s']:.2f} | {info['throughput_tps']:.1f} | "
                         f"{info['peak_vram_mb']:.1f} |")
        sections.append("\n".join(lines))
    return "\n\n".join(sections) + "\n"


def generate_markdown_report(json_path: str, out_md_path: str) -> str:
    with open(json_path) as handle:
        data = json.load(handle)
    text = markdown_report(data)
    with open(out_md_path, "w") as handle:
        handle.write(text)
    return text


if __name__ == "__main__":
    import sys

    json_file = sys.argv[1] if len(sys.argv) > 1 else "results/benchmark_results.json"
    md_file = sys.argv[2] if len(sys.argv) > 2 else "results/REPORT.md"
    if os.path.exists(json_file):
        print(generate_markdown_report(json_file, md_file))
    else:
        print(f"No results found at {json_file}")
