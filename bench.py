"""Decode-throughput benchmark of the W4A16 path (and the reference's CPU arm).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload: the full W4A16 decode of the Qwen2.5-0.5B architecture at batch 1 — seeded
synthetic weights (real weights cannot be downloaded), a 512-token random prompt in an
fp16 KV slot, greedy decode of 256 tokens.  One *step* is one such 256-token decode.
``value`` is decode tokens/s with everything resident in HBM (tokens chained on the device
by CUDA-graph launches); ``e2e`` is the same metric through the per-token public call with
the token id travelling host -> device and the sampled id device -> host every token, as
the reference's own generation loop does.  With N > 1 (launched by torch.distributed.run)
every rank is an independent replica with its own weights and request (weak scaling, no
collective on the data path).

``--impl reference`` times the reference's Hugging Face eager fp32 path on the host cores
on a bounded sample of the same workload (oracle/hf_ref.py; the reference project has no
CPU implementation of its own kernels).
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402

PROMPT_LEN, GEN_TOKENS, BURST = 512, 256, 64
METRIC, UNIT = "decode_tokens_per_s_batch1_w4a16", "tokens/s"
CONFIG = {
    "workload": "full W4A16 decode, Qwen2.5-0.5B architecture, batch 1, 512-token prompt, 256 greedy tokens",
    "layers": 24, "vocab": 151936, "kv_cache": "fp16 slots", "weights": "int4 group 128 + fp16 lm_head",
    "l2_policy": "inputs larger than L2: each token streams 466 MB of weights and KV through a 126 MB L2",
}


def profile_shares() -> dict:
    """Figures taken from committed ncu summaries (not measured by this run): the time share of
    each layer kernel among the layer kernels and the DRAM traffic of one lm_head launch."""
    path = os.path.join(ROOT, "profiles", "decode_step_kernel_shares.json")
    with open(path) as handle:
        return json.load(handle)


def peaks() -> tuple[float, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as handle:
            return float(json.load(handle)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        clocks, reasons, max_mhz = [], set(), None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for row in self.rows:
            try:
                clocks.append(float(row[0]))
                max_mhz = float(row[1])
            except (ValueError, IndexError):
                continue
            for name, cell in zip(names, row[3:7]):
                if cell.lower().startswith("active"):
                    reasons.add(name)
        busy = sorted(clocks)[len(clocks) // 2:] if clocks else []
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max_mhz,
                "samples": len(clocks), "reasons": sorted(reasons)}


def build_model(device: str, layers: int = 24):
    entry.load_package()
    from quic_cu_b200 import model as qmodel
    from quic_cu_b200.checkpoint import qwen_config_dict, synthetic_checkpoint

    state = synthetic_checkpoint(n_layers=layers, vocab=151936, seed=0)
    net = qmodel.from_state_dict(state, qwen_config_dict(layers, 151936), device=device)
    return net, state


def cpu_baseline(state, threads: int | None = None, gen: int = 16, repeats: int = 1, warmup: int = 0):
    """The reference's HF eager fp32 path on the host cores: the 512-token prompt is prefilled
    untimed, then ``gen`` greedy decode forwards are timed (run.py:49-61's loop)."""
    from oracle import hf_ref
    from quic_cu_b200.checkpoint import qwen_config_dict

    if threads:
        torch.set_num_threads(threads)
    model = hf_ref.build_hf_model(state, qwen_config_dict(24, 151936), dtype=torch.float32, device="cpu")
    gen_ids = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, 151936, (1, PROMPT_LEN), generator=gen_ids)
    times = []
    with torch.inference_mode():
        for it in range(warmup + repeats):
            out = model(prompt, use_cache=True)
            cache, nxt = out.past_key_values, out.logits[:, -1:, :].argmax(-1)
            t0 = time.perf_counter()
            for _ in range(gen):
                out = model(nxt, past_key_values=cache, use_cache=True)
                nxt = out.logits[:, -1:, :].argmax(-1)
            if it >= warmup:
                times.append(time.perf_counter() - t0)
    per_step = sum(times) / len(times)
    return {"value": gen / per_step, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"HF Qwen2ForCausalLM eager fp32, same synthetic weights, 512-token prompt prefilled "
                      f"untimed, {gen} greedy decode forwards timed x{len(times)}"}, per_step


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    entry.load_package()
    from quic_cu_b200.checkpoint import synthetic_checkpoint

    state = synthetic_checkpoint(n_layers=24, vocab=151936, seed=0)
    gen = 16
    base, per_step = cpu_baseline(state, threads=os.cpu_count(), gen=gen, repeats=args.steps,
                                  warmup=min(args.warmup, 1))
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": CONFIG,
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def run_gpu(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the decode path has no CPU fallback")
    torch.cuda.set_device(local)
    device = f"cuda:{local}"
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device(device))

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    entry.load_package()
    from quic_cu_b200 import kernels as K

    if world > 1:
        # N replicas share the host: the small CPU tensor ops of the serving loop must not each
        # spin up (and then spin-wait in) an OpenMP team of every core
        torch.set_num_threads(max(1, (os.cpu_count() or 8) // (2 * world)))
    net, state = build_model(device, args.layers)
    cache = net.new_cache(n_slots=1, s_max=1024)
    gen_ids = torch.Generator().manual_seed(rank)  # every replica serves its own request
    prompt = torch.randint(0, 151936, (PROMPT_LEN,), generator=gen_ids)
    first, _ = net.prefill(cache, [0], [prompt])
    tok0, pos0 = cache.tok.clone(), cache.pos.clone()
    torch.cuda.synchronize()

    def reset():
        cache.tok.copy_(tok0)
        cache.pos.copy_(pos0)
        cache.host_len[0] = PROMPT_LEN

    def one_step():
        reset()
        for _ in range(GEN_TOKENS // BURST):
            net.decode_async(cache, [0], BURST)

    for _ in range(max(args.warmup, 3)):
        one_step()
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    start.record()
    for _ in range(args.steps):
        one_step()
    end.record()
    barrier()
    elapsed_ms = start.elapsed_time(end)
    clocks = sampler.stop()
    if dist is not None:
        t = torch.tensor([elapsed_ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    tokens = args.steps * GEN_TOKENS
    value = world * tokens / (elapsed_ms / 1e3)

    # ---- end to end: one public decode call per token, token id host <-> device every token
    pinned_t = torch.zeros(1, dtype=torch.int32).pin_memory()
    pinned = pinned_t.numpy()  # same page-locked memory, cheap element writes
    e2e_tokens = GEN_TOKENS
    reset()
    pinned[0] = int(first[0])
    for _ in range(8):
        pinned[0] = net.decode(cache, [0], 1, feed=pinned_t)[0][0]
    reset()
    pinned[0] = int(first[0])
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_tokens):
        # H2D: the token to feed (pinned host memory); D2H: the sampled token
        pinned[0] = net.decode(cache, [0], 1, feed=pinned_t)[0][0]
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    if dist is not None:
        t = torch.tensor([e2e_s], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e = {"value": world * e2e_tokens / e2e_s, "unit": UNIT, "h2d_bytes_per_step": 4 * GEN_TOKENS,
           "d2h_bytes_per_step": 4 * GEN_TOKENS,
           "note": "per 256-token step: 256 public decode calls, each with a 4-byte token id H2D from "
                   "pinned memory and a 4-byte sampled id D2H"}

    # ---- rooflines.  By time the step is its 120 layer kernels (87 %), by bytes the lm_head
    # (58 %): `roofline` names the group that dominates by time, `roofline_kernels` lists every
    # kernel type, `roofline_step` is the whole token.
    peak, peak_kind = peaks()
    prof = profile_shares()
    x = torch.randn(1, 896, device=device, dtype=torch.float16)
    for _ in range(3):
        K.lm_head_argmax(x, net.embed, net.final_norm, net.eps)
    reps = 50
    k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    k0.record()
    for _ in range(reps):
        K.lm_head_argmax(x, net.embed, net.final_norm, net.eps)
    k1.record()
    torch.cuda.synchronize()
    lm_us = k0.elapsed_time(k1) * 1e3 / reps
    lm_bytes = 151936 * 896 * 2 + 896 * 4
    mean_ctx = PROMPT_LEN + GEN_TOKENS / 2
    step_bytes = net.weight_bytes() + 12288 * (mean_ctx + 1)
    us_per_token = elapsed_ms * 1e3 / tokens
    step_gbs = step_bytes / (us_per_token * 1e-6) / 1e9
    layers_us = max(us_per_token - lm_us, 1e-3)           # all 5 x 24 layer kernels of a token
    layer_bytes = step_bytes - lm_bytes                     # W4 weights of 24 layers + K/V read and written
    per_layer = {"qkv_kernel<1>": 536256 + 2304 + 1792 + 512, "attn_decode_cta_kernel<true>": 512 * (mean_ctx + 1),
                 "oproj_kernel<1>": 417088, "gateup_kernel<1>": 4528384 + 1792, "down_kernel<1>": 2264192}
    kernels = []
    for name, share in prof["layer_kernel_share"].items():
        us = layers_us / net.n_layers * share
        kernels.append({"kernel": name, "launches_per_token": net.n_layers, "algorithmic_bytes": per_layer[name],
                        "us_per_launch": us, "achieved": per_layer[name] / us / 1e3, "unit": "GB/s",
                        "frac": per_layer[name] / us / 1e3 / peak, "share_of_step": us * net.n_layers / us_per_token,
                        "timing": "(token time - live lm_head time) / layers x the kernel's share of the layer "
                                  "kernels' time in the committed ncu launch list"})
    kernels.append({"kernel": "lm_head_kernel<1>", "launches_per_token": 1, "algorithmic_bytes": lm_bytes,
                    "us_per_launch": lm_us, "achieved": lm_bytes / lm_us / 1e3, "unit": "GB/s",
                    "frac": lm_bytes / lm_us / 1e3 / peak, "share_of_step": lm_us / us_per_token,
                    "traffic": prof["dram_traffic_bytes_per_launch"]["lm_head_kernel<1>"],
                    "traffic_source": "ncu capture summarised under profiles/ (not measured by this run)",
                    "timing": f"{reps} back-to-back launches between CUDA events on the launching stream; the "
                              "272 MB table exceeds L2"})
    roofline = {"bound": "hbm", "kernel": "the 120 layer kernels of a token (qkv, attention, o_proj, gate_up, down "
                                          "x 24: dominant by time)",
                "achieved": layer_bytes / layers_us / 1e3, "peak": peak, "unit": "GB/s",
                "frac": layer_bytes / layers_us / 1e3 / peak, "peak_kind": f"of {peak_kind}",
                "share_of_step": layers_us / us_per_token, "us_per_token": layers_us,
                "algorithmic_bytes": layer_bytes, "traffic": None,
                "timing": "token time (CUDA events over the timed region) minus the lm_head kernel's live time"}
    roofline_step = {"bound": "hbm", "scope": "whole decode step (121 kernels)", "achieved": step_gbs,
                     "peak": peak, "unit": "GB/s", "frac": step_gbs / peak, "us_per_token": us_per_token,
                     "algorithmic_bytes": step_bytes}

    # ---- batch 64 (the other batch size the metric names): 64 slots, same context, resident state
    batch64 = None
    if not args.skip_batch64:
        batch64 = measure_batch64(net, device, world, dist)
    extras = {}
    if world == 1 and not args.skip_extras and args.layers == 24:
        for name, fn in (("rows_sweep", lambda: measure_rows_sweep(net, device)),
                         ("prefill", lambda: measure_prefill(net, device))):
            try:
                extras[name] = fn()
            except Exception as exc:  # the headline line must not depend on the extra measurements
                extras[name] = {"error": f"{type(exc).__name__}: {exc}"}
    serving = None
    if args.serving_requests > 0:
        try:
            serving = measure_serving(net, device, args.serving_requests, world, dist, rank, args.serving_order)
        except Exception as exc:  # the headline line must not depend on the extra measurement
            serving = {"error": f"{type(exc).__name__}: {exc}"}

    if rank != 0:
        return
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int4 weights x fp16 activations, fp32 accumulate",
        "data": "synthetic", "config": CONFIG, "parallelism": f"{world} independent replica(s), no collective",
        "clocks": clocks, "e2e": e2e, "gpu_launches": world * args.steps * GEN_TOKENS * net.launches_per_step(cache, 1, PROMPT_LEN + GEN_TOKENS),
        "roofline": roofline, "roofline_kernels": kernels, "roofline_step": roofline_step, "batch64": batch64,
        "serving": serving,
    }
    line.update(extras)
    if args.layers != 24:
        line["invalid"] = "reduced layer count: profiling run, not a benchmark"
    if world == 1 and not args.skip_extras and args.layers == 24:
        del net, cache
        net = cache = None
        torch.cuda.empty_cache()
        try:
            line["dense_fp16"] = measure_dense(device)
        except Exception as exc:
            line["dense_fp16"] = {"error": f"{type(exc).__name__}: {exc}"}
    if world == 1 and not args.no_cpu_baseline and args.layers == 24:
        del net, cache
        base, _ = cpu_baseline(state, threads=os.cpu_count(), gen=16, repeats=1, warmup=0)
        line["cpu_baseline"] = base
    print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


def linear_sweep(device: str = "cuda:0", shapes=None, ms=(1, 4, 16, 64, 256, 8192), reps: int = 20) -> list[dict]:
    """The single W4A16 linear-op sweep of the benchmark configuration: the model's four
    (K, N) shapes at M in {1, 4, 16, 64, 256} (decode) and 8192 (prefill); int4 values and zero points uniform in 0..15,
    scales |N(0, 0.01)| + 1e-3, activations N(0, 1).  Each point is timed as a CUDA graph of
    ``reps`` launches (device time, no host overhead).  M = 1 runs the dequant GEMV, M >= 2
    the tcgen05 GEMM."""
    entry.load_package()
    from quic_cu_b200 import kernels as K
    from quic_cu_b200.checkpoint import synthetic_layer

    peak, kind = peaks()
    shapes = shapes or {"qkv": (896, 1152), "o_proj": (896, 896), "gate_up": (896, 9728), "down": (4864, 896)}
    out = []
    for name, (k, n) in shapes.items():
        layer = synthetic_layer(n, k, torch.Generator().manual_seed(0))
        w = K.W4Weight(n, k, device)
        w.put(layer["weight_packed"], layer["weight_scale"], layer["weight_zero_point"])
        for m in ms:
            x = torch.randn(m, k, generator=torch.Generator().manual_seed(m)).half().to(device)
            for _ in range(3):
                K.w4a16_linear(w, x)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for _ in range(reps):
                    K.w4a16_linear(w, x)
            graph.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(5):
                graph.replay()
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / (5 * reps)
            nbytes = w.weight_bytes + m * k * 2 + m * n * 2
            out.append({"layer": name, "k": k, "n": n, "m": m, "kernel": "tcgen05 gemm" if m >= 2 else "gemv",
                        "us": us, "GB/s": nbytes / us / 1e3, "hbm_frac": nbytes / us / 1e3 / peak,
                        "TFLOP/s": 2.0 * m * n * k / us / 1e6, "algorithmic_bytes": nbytes,
                        "note": "weights stay in L2 between the launches of a graph"})
    return out


def attention_sweep(device: str = "cuda:0", batches=(1, 16, 64, 256), contexts=(128, 1024, 8192, 32768)) -> list[dict]:
    """The split-K GQA decode-attention sweep of the benchmark configuration: 14 query / 2 KV
    heads, head_dim 64, fp16 N(0,1) Q/K/V, every row left-padded by a length uniform in
    [0, context/4].  Timed as a CUDA graph of launches through the reference-shaped op
    (flash_attn_decode().forward); bytes = K and V of the unpadded tokens + Q + O."""
    entry.load_package()
    from quic_cu_b200 import kernels as K

    peak, kind = peaks()
    out = []
    op = K.flash_attn_decode()
    for b in batches:
        for s in contexts:
            g = torch.Generator(device=device).manual_seed(b * 100003 + s)
            q = torch.randn((b, 14, 1, 64), device=device, generator=g).half()
            k = torch.randn((b, 2, s, 64), device=device, generator=g).half()
            v = torch.randn((b, 2, s, 64), device=device, generator=g).half()
            pads = torch.randint(0, s // 4 + 1, (b,), device=device, generator=g).int()
            for _ in range(3):
                op.forward(q, k, v, 0.125, pads)
            torch.cuda.synchronize()
            reps = 10 if b * s < (1 << 20) else 3
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for _ in range(reps):
                    op.forward(q, k, v, 0.125, pads)
            graph.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(3):
                graph.replay()
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / (3 * reps)
            tokens = int((s - pads.long()).sum().item())
            nbytes = tokens * 512 + b * 14 * 64 * 2 * 2
            out.append({"batch": b, "context": s, "splits": K.lib().quic_attn_pick_splits(b, s), "us": us,
                        "GB/s": nbytes / us / 1e3, "hbm_frac": nbytes / us / 1e3 / peak, "peak_kind": f"of {kind}",
                        "algorithmic_bytes": nbytes,
                        "note": "K/V larger than L2 from ~100 MB up; smaller cases are served from L2"})
            del q, k, v
    return out


def ttft_sweep(device: str = "cuda:0", grid=((1, 128), (1, 512), (4, 128), (4, 512), (16, 128), (16, 512)),
               gen_tokens: int = 32) -> list[dict]:
    """Time to first token and decode rate on the reference's own grid (benchmarks/collect.py:
    batch x context, CUDA events around the prefill, then around gen_tokens - 1 decode
    forwards; decode_tps = batch * (gen_tokens - 1) / decode seconds).  Prefill attention by
    the library's kernel; synthetic weights and random prompts."""
    net, _ = build_model(device, 24)
    net.prefill_backend = "quic"
    out = []
    for batch, ctx in grid:
        gen = torch.Generator().manual_seed(batch * 1000 + ctx)
        prompts = [torch.randint(0, 151936, (ctx,), generator=gen) for _ in range(batch)]
        slots = list(range(batch))
        cache = net.new_cache(n_slots=batch, s_max=max(1024, (ctx + gen_tokens + 63) // 64 * 64))
        for _ in range(2):
            net.prefill(cache, slots, prompts)
            net.decode_async(cache, slots, gen_tokens - 1)
        torch.cuda.synchronize()
        ttft, dec = [], []
        for _ in range(5):
            e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            e[0].record()
            net.prefill(cache, slots, prompts)
            e[1].record()
            net.decode_async(cache, slots, gen_tokens - 1)
            e[2].record()
            torch.cuda.synchronize()
            ttft.append(e[0].elapsed_time(e[1]))
            dec.append(e[1].elapsed_time(e[2]))
        out.append({"batch": batch, "context": ctx, "ttft_ms": sum(ttft) / len(ttft),
                    "decode_tps": batch * (gen_tokens - 1) / (sum(dec) / len(dec) / 1e3),
                    "peak_vram_mb": torch.cuda.max_memory_allocated() / 2 ** 20,
                    "note": "W4A16, prefill_backend quic; the reference's H100 figures for this grid: "
                            "TTFT 13.1 / 20.2 / 18.8 / 40.0 / 53.6 / 52.5 ms"})
    return out


def engine_batching(net, policy: str, max_batch_size: int = 4, num_requests: int = 8, max_tokens: int = 32,
                    prompt_len: int = 40) -> dict:
    """The reference's batching benchmark (benchmarks/collect.py:121-178): ``num_requests`` short
    prompts through ``Engine.run`` under one admission policy, wall clock around the run.  Prompts
    are seeded random token ids of the length its chat-templated sentences have."""
    from types import SimpleNamespace

    from quic_cu_b200.config import EngineConfig
    from quic_cu_b200.engine import Engine

    module = SimpleNamespace(load=lambda **options: (net, None))
    engine = Engine(config=EngineConfig(batching=policy, max_context=1024, prefill_backend="quic"),
                    max_batch_size=max_batch_size, model_module=module)
    engine.max_tokens = max_tokens
    gen = torch.Generator().manual_seed(8)
    for _ in range(num_requests):
        engine.add_request_ids(torch.randint(0, 151936, (prompt_len,), generator=gen))
    torch.cuda.reset_peak_memory_stats()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    outputs = engine.run()
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - t0
    total = sum(len(o) for o in outputs)
    return {"policy": policy, "max_batch_size": max_batch_size, "num_requests": len(outputs), "total_tokens": total,
            "elapsed_s": elapsed, "throughput_tps": total / elapsed if elapsed > 0 else 0.0,
            "peak_vram_mb": torch.cuda.max_memory_allocated() / 2 ** 20}


def collect(output_dir: str, device: str = "cuda:0") -> dict:
    """Writes ``benchmark_results.json`` and ``REPORT.md`` in the reference's schema
    (benchmarks/collect.py:181-247, benchmarks/report.py): the ``quic_quant`` path on the
    reference's default grid (batch 1, 4, 16 x context 128, 512, 1024, 2048, 32 generated
    tokens) and both admission policies of the engine."""
    entry.load_package()
    from quic_cu_b200 import report

    grid = tuple((b, c) for b in (1, 4, 16) for c in (128, 512, 1024, 2048))
    rows = ttft_sweep(device, grid)
    net, _ = build_model(device, 24)
    batching = {}
    for policy in ("static", "continuous"):
        engine_batching(net, policy)  # untimed pass: CUDA graph captures of a fresh engine
        batching[policy] = engine_batching(net, policy)
    data = report.collect_results({"quic_quant": rows}, batching)
    json_path = report.write_results(data, output_dir)
    report.generate_markdown_report(json_path, os.path.join(output_dir, "REPORT.md"))
    return data


def measure_batch64(net, device, world, dist):
    """Decode tokens/s with 64 rows in flight (64 KV slots, 512 cached tokens each, 128 greedy
    steps), state resident, CUDA events, max over ranks."""
    B, ctx, steps, burst = 64, PROMPT_LEN, 128, 32
    cache = net.new_cache(n_slots=B, s_max=1024)
    slots = list(range(B))
    gen = torch.Generator(device=device).manual_seed(1)
    # random K/V stand in for 512 prefilled tokens per slot (values do not change the work done)
    cache.kv.normal_(0, 1, generator=gen)
    cache.tok.copy_(torch.randint(0, 151936, (B,), generator=gen, device=device, dtype=torch.int32))

    def reset():
        cache.pos.fill_(ctx)
        for s in slots:
            cache.host_len[s] = ctx

    def run():
        reset()
        for _ in range(steps // burst):
            net.decode_async(cache, slots, burst)

    for _ in range(3):
        run()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 3
    e0.record()
    for _ in range(reps):
        run()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if dist is not None:
        t = torch.tensor([ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    us_step = ms * 1e3 / (reps * steps)
    peak, kind = peaks()
    step_bytes = net.weight_bytes() + B * 12288 * (ctx + steps / 2 + 1)
    return {"value": world * B / (us_step * 1e-6), "unit": UNIT, "batch": B, "context": ctx, "us_per_step": us_step,
            "kernels": "tcgen05 W4A16 GEMM + tcgen05 lm_head/argmax + attention streamed through a TMA ring",
            "hbm_frac": step_bytes / (us_step * 1e-6) / 1e9 / peak, "peak_kind": f"of {kind}",
            "algorithmic_bytes_per_step": step_bytes}


def _time_decode(net, device, rows: int, ctx: int = PROMPT_LEN, steps: int = 64, burst: int = 32, reps: int = 3) -> float:
    """us per decode step with ``rows`` rows in flight at ``ctx`` cached tokens (random K/V stand
    in for the prefilled tokens), state resident, CUDA events."""
    cache = net.new_cache(n_slots=max(rows, 1), s_max=1024)
    slots = list(range(rows))
    gen = torch.Generator(device=device).manual_seed(1)
    cache.kv.normal_(0, 1, generator=gen)
    cache.tok.copy_(torch.randint(0, 151936, (cache.n_slots,), generator=gen, device=device, dtype=torch.int32))

    def run():
        cache.pos.fill_(ctx)
        for s_ in slots:
            cache.host_len[s_] = ctx
        for _ in range(steps // burst):
            net.decode_async(cache, slots, burst)

    for _ in range(2):
        run()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        run()
    e1.record()
    torch.cuda.synchronize()
    cache.release_graphs()
    return e0.elapsed_time(e1) * 1e3 / (reps * steps)


def measure_rows_sweep(net, device) -> dict:
    """Decode step time against the number of rows: one row on the GEMV chain, two on its
    two-row form, 3..16 on the mma.sync chain, more on the tcgen05 step."""
    out = {}
    for rows in (1, 2, 3, 4, 8, 16, 32):
        us = _time_decode(net, device, rows)
        out[str(rows)] = {"us_per_step": us, "tokens_per_s": rows / (us * 1e-6)}
    one = out["1"]["us_per_step"]
    for v in out.values():
        v["vs_one_row"] = v["us_per_step"] / one
    return {"context": PROMPT_LEN, "rows": out}


def measure_prefill(net, device) -> dict:
    """Time to first token of 16 prompts of 2048 tokens through the public prefill call (ids on
    the host, first tokens read back), and the prefill attention kernel alone at 1 x 2048 and
    16 x 2048 on tcgen05 and on the mma.sync kernels it replaces."""
    from quic_cu_b200 import kernels as K

    n_seq, n = 16, 2048
    gen = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, 151936, (n,), generator=gen) for _ in range(n_seq)]
    cache = net.new_cache(n_slots=n_seq, s_max=n + 64)
    for _ in range(2):
        net.prefill(cache, list(range(n_seq)), prompts)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    reps = 3
    for _ in range(reps):
        first, _ = net.prefill(cache, list(range(n_seq)), prompts)
        first.cpu()
    ttft_ms = (time.perf_counter() - t0) / reps * 1e3
    del cache
    dev = dict(device=device, dtype=torch.int32)
    kernels = []
    for seqs in (1, 16):
        rows = seqs * n
        q = torch.randn((14, rows, 64), device=device).half()
        kc = torch.randn((seqs, 2, n, 64), device=device).half()
        vc = torch.randn_like(kc)
        starts = torch.tensor([i * n for i in range(seqs)], **dev)
        lens, slots = torch.tensor([n] * seqs, **dev), torch.arange(seqs, **dev)
        flops = seqs * 14 * n * (n + 1) / 2 * 64 * 4
        for mode, name in ((1, "tcgen05 + TMA"), (0, "mma.sync")):
            K.lib().quic_set_prefill_tensor_attention(mode)
            for _ in range(3):
                K.attn_prefill(q, kc, vc, starts, lens, slots, n, 0.125)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(10):
                K.attn_prefill(q, kc, vc, starts, lens, slots, n, 0.125)
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 100
            kernels.append({"sequences": seqs, "tokens": n, "kernel": name, "us": us, "tflops": flops / us / 1e6})
        K.lib().quic_set_prefill_tensor_attention(1)
    return {"ttft_ms": ttft_ms, "prompts": n_seq, "prompt_tokens": n, "attention": kernels,
            "note": "W4A16 linears on the tcgen05 GEMM at M = 32768, attention on tcgen05; causal flops counted"}


def measure_dense(device) -> dict:
    """The un-quantised fp16 model through the same step: one-row decode (GEMV chain over
    988 MB of weights per token) and 64 rows (tcgen05 fp16 GEMM)."""
    from quic_cu_b200 import model as qmodel
    from quic_cu_b200.checkpoint import qwen_config_dict, synthetic_dense_checkpoint

    cfg = qwen_config_dict(24, 151936)
    cfg.pop("quantization_config", None)
    net = qmodel.from_state_dict(synthetic_dense_checkpoint(n_layers=24, vocab=151936, seed=0), cfg, device=device)
    peak, kind = peaks()
    out = {}
    for rows in (1, 64):
        us = _time_decode(net, device, rows)
        step_bytes = net.weight_bytes() + rows * 12288 * (PROMPT_LEN + 33)
        out[str(rows)] = {"us_per_step": us, "tokens_per_s": rows / (us * 1e-6),
                          "hbm_frac": step_bytes / (us * 1e-6) / 1e9 / peak, "algorithmic_bytes_per_step": step_bytes}
    return {"dtype": "fp16 weights x fp16 activations, fp32 accumulate", "peak_kind": f"of {kind}", "rows": out}


def measure_serving(net, device, n_requests, world, dist, rank, order="longest"):
    """Continuous batching with 64 KV slots per GPU (benchmark configuration 4): prompt lengths
    uniform in 64..1024, output lengths uniform in 128..512 (forced through max_tokens; random
    weights never emit EOS), all requests queued at t = 0 (arrivals at saturation), greedy,
    prefill attention by the library's own kernel.  ``n_requests`` is the size of the WHOLE
    queue: the replicas pull chunks of 8 requests from one shared FIFO kept in the process
    group's store (quic_cu_b200.replicas.serve_pulled), so the work is fixed as N grows.
    ``order``: "fifo" queues the requests as generated; "longest" queues them by token budget
    (max_tokens, a field of every request), largest first -- the longest-processing-time rule: the
    batches that empty at the end of the run then hold the short requests, which matters as the
    share of a replica shrinks (512 requests: 3.08 s as generated, 2.65 s longest first).
    Wall clock on every rank from the common start to the moment the last chunk is done, max
    over ranks."""
    from types import SimpleNamespace

    import torch.distributed as tdist

    from quic_cu_b200.config import EngineConfig
    from quic_cu_b200.engine import Engine
    from quic_cu_b200.replicas import Request, StoreQueue, chunks_of, group_store, serve_pulled

    gen = torch.Generator().manual_seed(4)
    plens = torch.randint(64, 1025, (n_requests,), generator=gen).tolist()
    olens = torch.randint(128, 513, (n_requests,), generator=gen).tolist()
    reqs = [Request(i, tuple(torch.randint(0, 151936, (plens[i],), generator=gen).tolist()), olens[i])
            for i in range(n_requests)]
    if order == "longest":
        reqs.sort(key=lambda r: -r.max_tokens)
    chunk = 8
    n_chunks = len(chunks_of(reqs, chunk))
    store = group_store(dist) if dist is not None else tdist.HashStore()
    module = SimpleNamespace(load=lambda **options: (net, None))
    engine = Engine(config=EngineConfig(batching="continuous", max_context=2048, decode_burst=16,
                                        prefill_backend="quic"),
                    max_batch_size=64, model_module=module)
    # First pass: the engine captures one CUDA graph per (rows, context bound, burst) it meets
    # (a one-time cost of a long-lived server); second pass: the same queue on the warm engine.
    passes = []
    for p in range(2):
        queue = StoreQueue(store, n_chunks, rank, prefix=f"serving{p}", stale_s=60.0)
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        kept0, cpu0, t0 = engine.generated, time.process_time(), time.perf_counter()
        stats = serve_pulled(engine, reqs, queue, chunk=chunk)
        torch.cuda.synchronize()
        seconds = time.perf_counter() - t0
        mine = [seconds, float(engine.generated - kept0), stats["busy_s"], time.process_time() - cpu0,
                float(stats["requests"])]
        if dist is not None:
            everyone = [None] * world
            dist.all_gather_object(everyone, mine)
        else:
            everyone = [mine]
        passes.append(everyone)
    warm = passes[1]
    seconds = max(r[0] for r in warm)
    tokens = int(sum(r[1] for r in warm))
    cold_seconds = max(r[0] for r in passes[0])
    return {"value": tokens / seconds, "unit": "generated tokens/s (prefill included in the time)",
            "requests": n_requests, "generated_tokens": tokens, "prompt_tokens": sum(plens), "seconds": seconds,
            "first_pass_seconds": cold_seconds, "first_pass_value": int(sum(r[1] for r in passes[0])) / cold_seconds,
            "per_replica": [{"requests": int(r[4]), "generated_tokens": int(r[1]), "seconds": r[0],
                             "engine_busy_s": r[2], "host_cpu_share": r[3] / r[0] if r[0] > 0 else None} for r in warm],
            "queue_order": "longest token budget first" if order == "longest" else "as generated",
            "queue": "pull-based: chunks of 8 requests claimed from a FIFO in the process group's store; "
                     "the queue size is fixed as N grows (strong scaling)",
            "note": "value: second pass over the same queue on the same engine (decode graphs captured); "
                    "first_pass_*: fresh engine, captures included",
            "slots_per_gpu": 64, "decode_burst": 16, "replicas": world}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="quic_b200", choices=["quic_b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--skip-batch64", action="store_true", help="skip the extra batch-64 decode measurement")
    ap.add_argument("--skip-extras", action="store_true",
                    help="skip the rows sweep, the prefill and the dense fp16 measurements (N = 1 only)")
    ap.add_argument("--serving-requests", type=int, default=4096,
                    help="also serve a queue of this many synthetic requests with continuous batching (64 slots "
                         "per GPU, pulled by all replicas from one FIFO, two passes: about 35 s each on one GPU); "
                         "4096 is the benchmark configuration; 0 skips it")
    ap.add_argument("--batch64-only", action="store_true",
                    help="run only the 64-row decode measurement and print its block (profiler captures)")
    ap.add_argument("--serving-order", default="longest", choices=["longest", "fifo"],
                    help="order of the serving queue: by token budget, largest first (default), or as generated")
    ap.add_argument("--layers", type=int, default=24,
                    help="decoder layers of the synthetic model; values below 24 exist only to keep "
                         "profiler captures small and do not produce a valid benchmark line")
    ap.add_argument("--linear-sweep", action="store_true",
                    help="print the W4A16 linear-op sweep (one JSON line per point) and exit")
    ap.add_argument("--attention-sweep", action="store_true",
                    help="print the decode-attention sweep (one JSON line per point) and exit")
    ap.add_argument("--ttft-sweep", action="store_true",
                    help="print time-to-first-token and decode rate on the reference's batch x context grid and exit")
    ap.add_argument("--collect", default="", metavar="DIR",
                    help="write benchmark_results.json and REPORT.md in the reference collector's schema to DIR")
    ap.add_argument("--attention-point", default="",
                    help="with --attention-sweep: measure the single point 'batch,context' (profiler captures)")
    args = ap.parse_args()
    if args.attention_sweep:
        kw = {}
        if args.attention_point:
            b, s_ = (int(v) for v in args.attention_point.split(","))
            kw = {"batches": (b,), "contexts": (s_,)}
        for row in attention_sweep(**kw):
            print(json.dumps(row))
        return
    if args.collect:
        print(json.dumps(collect(args.collect)))
        return
    if args.ttft_sweep:
        for row in ttft_sweep():
            print(json.dumps(row))
        return
    if args.linear_sweep:
        for row in linear_sweep():
            print(json.dumps(row))
        return
    if args.batch64_only:
        net, _ = build_model("cuda:0", args.layers)
        print(json.dumps(measure_batch64(net, "cuda:0", 1, None)))
        return
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
