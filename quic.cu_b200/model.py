"""Qwen2.5-0.5B W4A16 model on the B200 kernels, behind the reference's model API.

Mirrors src/model.py of the reference: ``load(path, prefill_backend, use_marlin, use_machete,
tokenizer_path) -> (QUICForCausalLM, tokenizer)`` (src/model.py:306) and
``QUICForCausalLM.forward(input_ids, past_key_values, attention_mask, position_ids, use_cache)
-> CausalLMOutputWithPast`` (src/model.py:272).  Differences that callers can see:

* the cache object handed back is a ``SlotCache`` (slotted fp16 KV that stores real tokens
  only) instead of HF's ``DynamicCache``; it offers ``get_seq_length()`` and can be passed
  back in, which is all the reference's callers do with it (run.py:50-61,
  benchmarks/collect.py:61-92);
* a prefill returns logits of the last position only unless ``prefill_all_logits`` is set;
* decode (``seq_len == 1``) is ONE fused call: embedding, 24 layers, final norm, lm_head and
  argmax run as a chain of kernels with state on the device.  ``decode`` runs several
  consecutive greedy steps from a captured CUDA graph without a host round trip.
"""

from __future__ import annotations

import ctypes as C
import json
import numbers
import os
from dataclasses import dataclass

import torch

from . import kernels as K
from .checkpoint import LAYER_LINEARS, detect_group_size, packed_prefixes

DTYPE = torch.float16
# QUIC_PERSIST=1 (or model.use_persist = True) decodes batches of up to quic_persist_max_rows()
# rows in the persistent kernel: one launch per burst of tokens.  Off by default: measured at
# 587 us per token against 352 us for the kernel chain (24 layers, one row).
PERSIST = os.environ.get("QUIC_PERSIST", "0") == "1"
HIDDEN, HEADS, KV_HEADS, HEAD_DIM, INTER, QKV_N = K.HIDDEN, K.HEADS, K.KV_HEADS, K.HEAD_DIM, K.INTER, K.QKV_N


@dataclass
class CausalLMOutput:
    """Same two fields callers read from transformers' CausalLMOutputWithPast."""

    logits: torch.Tensor
    past_key_values: "SlotCache | None" = None


class SlotCache:
    """Slotted KV cache: fp16 [layers][K|V][slots][kv heads][s_max][64] plus the per-slot
    device state of the decode loop (next token, position) and the decode scratch arena.

    Replaces HF DynamicCache as used by the reference (src/model.py:160, src/engine.py:54):
    a slot stores only real tokens, so left padding never occupies memory and appending a
    token is a 512-byte write per layer instead of a torch.cat of the whole cache."""

    def __init__(self, n_layers: int, n_slots: int, s_max: int, vocab: int, device, ring: int = 64):
        self.n_layers, self.n_slots, self.s_max, self.vocab, self.ring = n_layers, n_slots, s_max, vocab, ring
        self.device = device
        self.kv = torch.zeros(n_layers, 2, n_slots, KV_HEADS, s_max, HEAD_DIM, dtype=DTYPE, device=device)
        self.tok = torch.zeros(n_slots, dtype=torch.int32, device=device)
        self.pos = torch.zeros(n_slots, dtype=torch.int32, device=device)
        self.out_tokens = torch.zeros(ring, n_slots, dtype=torch.int32, device=device)
        self.step_counter = torch.zeros(1, dtype=torch.int32, device=device)
        self.host_len = [0] * n_slots  # host mirror of pos (tokens cached per slot)
        self.batch_slots: list[int] = []  # slots of the batch rows, for the forward() API
        self._rows: dict[tuple, torch.Tensor] = {}      # row->slot maps by slot tuple (evictable)
        self._row_bufs: dict[int, torch.Tensor] = {}    # per batch size: the buffer captured graphs read
        self._scratch: dict[tuple, torch.Tensor] = {}
        self._graphs: dict[tuple, int] = {}
        self.max_graphs = 512                      # captured graphs kept; beyond that all are dropped and rebuilt
        self._plans: dict[tuple, tuple] = {}       # decode(): per (rows, steps) launch plan
        self._rows_loaded: dict[int, torch.Tensor] = {}  # row->slot map now on the device, per batch size
        self.host_steps = 0                        # host mirror of step_counter

    def check_slots(self, slots, count: int, what: str) -> None:
        """Every kernel indexes the KV planes and the per-slot state by slot: a slot outside
        the cache or one used twice in a batch is refused here, before any launch."""
        if len(slots) != count:
            raise ValueError(f"{what}: {len(slots)} slots for {count} rows")
        if any((not isinstance(s, numbers.Integral)) or s < 0 or s >= self.n_slots for s in slots):
            raise ValueError(f"{what}: slots must be integers in 0..{self.n_slots - 1}, got {list(slots)[:8]}")
        if len(set(slots)) != len(slots):
            raise ValueError(f"{what}: a slot appears twice in the batch")

    def get_seq_length(self, layer_idx: int = 0) -> int:
        return max((self.host_len[s] for s in self.batch_slots), default=0)

    def rows_tensor(self, slots: list[int]) -> torch.Tensor:
        key = tuple(slots)
        t = self._rows.get(key)
        if t is None:
            if len(self._rows) > 256:
                self._rows.clear()
            t = torch.tensor(slots, dtype=torch.int32, device=self.device)
            self._rows[key] = t
        return t

    def scratch(self, batch: int, splits: int) -> torch.Tensor:
        key = (batch, splits)
        t = self._scratch.get(key)
        if t is None:
            need = K.lib().quic_decode_scratch_bytes(batch, self.vocab, splits)
            t = torch.zeros(need, dtype=torch.uint8, device=self.device)
            self._scratch[key] = t
        return t

    def persist_sync(self) -> torch.Tensor:
        """Exchange area of the persistent decode kernel (zeroed once; its tags only grow)."""
        t = self.__dict__.get("_persist_sync")
        if t is None:
            t = torch.zeros(K.lib().quic_persist_sync_bytes(), dtype=torch.uint8, device=self.device)
            self._persist_sync = t
            self._persist_status = torch.zeros(1, dtype=torch.int32).pin_memory()
        return t

    def host_out(self) -> torch.Tensor:
        """Page-locked host mirror of ``out_tokens`` (filled by decode())."""
        t = self.__dict__.get("_host_out")
        if t is None:
            t = torch.zeros(self.ring, self.n_slots, dtype=torch.int32).pin_memory()
            self._host_out = t
        return t

    def release_graphs(self) -> None:
        """Destroys every captured graph with what only graphs refer to (launch plans, scratch
        arenas).  The caller makes sure that none of them is still running."""
        for g in self._graphs.values():
            K.lib().quic_graph_destroy(g)
        self._graphs.clear()
        self._plans.clear()
        self._scratch.clear()

    def __del__(self):
        try:
            self.release_graphs()
        except Exception:
            pass


def _ctx_bucket(n: int, batch: int = 1) -> int:
    """Context bound a captured graph is valid for: multiples of 128 up to 2048 (so the
    attention grid tracks the real context closely), powers of two beyond.  From 16 rows the
    step is 256: half as many graphs to capture, at most two more empty 64-token tiles per row."""
    step = 128 if batch < 16 else 256
    if n <= 2048:
        return max(step, (n + step - 1) // step * step)
    b = 4096
    while b < n:
        b *= 2
    return b


class QUICForCausalLM:
    """The model: W4A16 (or, for an un-quantised checkpoint, dense fp16) weights in device
    layout + the C structs the kernels read."""

    def __init__(self, config: dict, device="cuda"):
        self.config = config
        self.device = torch.device(device)
        self.n_layers = int(config["num_hidden_layers"])
        self.vocab = int(config["vocab_size"])
        self.eps = float(config.get("rms_norm_eps", 1e-6))
        rp = config.get("rope_parameters") or {}
        self.theta = float(rp.get("rope_theta", config.get("rope_theta", 1000000.0)))
        self.max_pos = int(config.get("max_position_embeddings", 32768))
        if (config["hidden_size"], config["intermediate_size"], config["num_attention_heads"],
                config["num_key_value_heads"]) != (HIDDEN, INTER, HEADS, KV_HEADS):
            raise RuntimeError("quic_b200 kernels are built for the Qwen2.5-0.5B layer shapes only")
        # kept for the reference's load(prefill_backend=...) signature; every value runs the
        # library's own prefill attention kernel
        self.prefill_backend = "quic"
        self.prefill_all_logits = False
        self.layers: list[dict] = []
        self.embed: torch.Tensor | None = None
        self.final_norm: torch.Tensor | None = None
        self._c_layers = None
        self._c_model = None
        self.default_slots = 8
        self.default_context = 4096
        self.use_persist = PERSIST
        self.dense = False  # True: un-quantised fp16 weights (F16Weight), the dense kernels
        self._wstream: torch.Tensor | None = None

    # ---- weights -------------------------------------------------------------
    def load_state(self, weights: dict) -> None:
        """Consumes a packed checkpoint state dict (names as in the reference's
        model.safetensors, src/model.py:332-356) and builds the device layout."""
        dev = self.device
        prefixes = packed_prefixes(weights)
        self.embed = weights["model.embed_tokens.weight"].to(dev, DTYPE).contiguous()
        self.final_norm = weights["model.norm.weight"].to(dev, DTYPE).contiguous()
        if self.embed.shape != (self.vocab, HIDDEN):
            raise RuntimeError("weight mismatch: embed_tokens shape")
        self.dense = not prefixes  # no packed tensor at all: the un-quantised fp16 model
        for i in range(self.n_layers):
            base = f"model.layers.{i}"
            for name, _, _, _ in LAYER_LINEARS:
                if not self.dense and f"{base}.{name}" not in prefixes:
                    raise RuntimeError(f"packed and dense layers cannot be mixed: '{base}.{name}' has no packed weight")

            def get(name, key):
                return weights[f"{base}.{name}.{key}"]

            if self.dense:
                self.layers.append(self._dense_layer(base, get, weights, dev))
                continue

            bias = torch.empty(QKV_N, dtype=DTYPE, device=dev)
            qkv = K.W4Weight(QKV_N, HIDDEN, dev, bias=bias)
            off = 0
            for name, n in (("self_attn.q_proj", 896), ("self_attn.k_proj", 128), ("self_attn.v_proj", 128)):
                qkv.put(get(name, "weight_packed"), get(name, "weight_scale"), get(name, "weight_zero_point"),
                        row_offset=off, row_order=K.ROWS_ROPE_PAIRS)
                b = get(name, "bias").to(dev, DTYPE)
                # same row order as the weights: (0,32,1,33,...) inside each head
                bias[off:off + n] = b.view(-1, 2, 32).transpose(1, 2).reshape(-1)
                off += n
            o = K.W4Weight(HIDDEN, HIDDEN, dev)
            o.put(get("self_attn.o_proj", "weight_packed"), get("self_attn.o_proj", "weight_scale"),
                  get("self_attn.o_proj", "weight_zero_point"))
            gu = K.W4Weight(2 * INTER, HIDDEN, dev)
            gu.put(get("mlp.gate_proj", "weight_packed"), get("mlp.gate_proj", "weight_scale"),
                   get("mlp.gate_proj", "weight_zero_point"), row_offset=0)
            gu.put(get("mlp.up_proj", "weight_packed"), get("mlp.up_proj", "weight_scale"),
                   get("mlp.up_proj", "weight_zero_point"), row_offset=INTER)
            down = K.W4Weight(HIDDEN, INTER, dev)
            down.put(get("mlp.down_proj", "weight_packed"), get("mlp.down_proj", "weight_scale"),
                     get("mlp.down_proj", "weight_zero_point"))
            self.layers.append({
                "qkv": qkv, "o": o, "gate_up": gu, "down": down,
                "ln1": weights[f"{base}.input_layernorm.weight"].to(dev, DTYPE).contiguous(),
                "ln2": weights[f"{base}.post_attention_layernorm.weight"].to(dev, DTYPE).contiguous(),
            })
        exponent = torch.arange(0, HEAD_DIM, 2, dtype=torch.float32) / HEAD_DIM
        inv_freq = (1.0 / (self.theta ** exponent)).to(dev).contiguous()  # src/model.py:82-84
        self.rope_cos, self.rope_sin = K.rope().init_table(inv_freq, self.max_pos)
        self._build_structs()
        torch.cuda.synchronize(dev)

    def _dense_layer(self, base: str, get, weights: dict, dev) -> dict:
        """The four fused matrices of a layer from un-quantised ``.weight`` tensors ([N, K])."""
        bias = torch.empty(QKV_N, dtype=DTYPE, device=dev)
        qkv = K.F16Weight(QKV_N, HIDDEN, dev, bias=bias)
        off = 0
        for name, n in (("self_attn.q_proj", 896), ("self_attn.k_proj", 128), ("self_attn.v_proj", 128)):
            qkv.put(get(name, "weight"), row_offset=off, row_order=K.ROWS_ROPE_PAIRS)
            bias[off:off + n] = get(name, "bias").to(dev, DTYPE).view(-1, 2, 32).transpose(1, 2).reshape(-1)
            off += n
        o = K.F16Weight(HIDDEN, HIDDEN, dev)
        o.put(get("self_attn.o_proj", "weight"))
        gu = K.F16Weight(2 * INTER, HIDDEN, dev)
        gu.put(get("mlp.gate_proj", "weight"), row_offset=0)
        gu.put(get("mlp.up_proj", "weight"), row_offset=INTER)
        down = K.F16Weight(HIDDEN, INTER, dev)
        down.put(get("mlp.down_proj", "weight"))
        return {"qkv": qkv, "o": o, "gate_up": gu, "down": down,
                "ln1": weights[f"{base}.input_layernorm.weight"].to(dev, DTYPE).contiguous(),
                "ln2": weights[f"{base}.post_attention_layernorm.weight"].to(dev, DTYPE).contiguous()}

    def _build_structs(self) -> None:
        arr = (K.Layer * self.n_layers)()
        for i, L in enumerate(self.layers):
            arr[i].qkv, arr[i].o = L["qkv"].struct(), L["o"].struct()
            arr[i].gate_up, arr[i].down = L["gate_up"].struct(), L["down"].struct()
            arr[i].ln1, arr[i].ln2 = K.ptr(L["ln1"]), K.ptr(L["ln2"])
        self._c_layers = arr
        self._c_model = K.Model(self.n_layers, self.vocab, self.eps, self.max_pos, arr, K.ptr(self.embed),
                                K.ptr(self.final_norm), K.ptr(self.rope_cos), K.ptr(self.rope_sin))

    def weight_bytes(self) -> int:
        """Algorithmic bytes one decode step reads from the weights (all layers + lm_head)."""
        per_layer = sum(L[k].weight_bytes for L in self.layers[:1] for k in ("qkv", "o", "gate_up", "down"))
        per_layer += QKV_N * 2 + 2 * HIDDEN * 2
        return per_layer * self.n_layers + self.vocab * HIDDEN * 2 + HIDDEN * 2

    def new_cache(self, n_slots: int | None = None, s_max: int | None = None) -> SlotCache:
        return SlotCache(self.n_layers, n_slots or self.default_slots, s_max or self.default_context,
                         self.vocab, self.device)

    def eval(self):
        return self

    def __call__(self, *args, **kwargs):
        return self.forward(*args, **kwargs)

    # ---- decode ----------------------------------------------------------------
    def _decode_struct(self, cache: SlotCache, batch: int, ctx: int, logits: torch.Tensor | None,
                       persist: bool = False):
        if persist:  # no scratch arena; the library picks the splits from ctx
            rows = cache._row_bufs.get(batch)
            if rows is None:
                rows = cache._row_bufs[batch] = torch.zeros(batch, dtype=torch.int32, device=self.device)
            d = K.Decode(K.ptr(cache.kv), cache.n_slots, cache.s_max, K.ptr(cache.tok), K.ptr(cache.pos),
                         K.ptr(rows), batch, K.ptr(cache.out_tokens), cache.ring, K.ptr(cache.step_counter),
                         K.ptr(logits), None, 0, ctx)
            return d, rows
        splits = K.lib().quic_decode_pick_splits(batch, ctx)
        # captured graphs keep this buffer's address: it lives as long as the cache
        rows = cache._row_bufs.get(batch)
        if rows is None:
            rows = cache._row_bufs[batch] = torch.zeros(batch, dtype=torch.int32, device=self.device)
        d = K.Decode(K.ptr(cache.kv), cache.n_slots, cache.s_max, K.ptr(cache.tok), K.ptr(cache.pos),
                     K.ptr(rows), batch, K.ptr(cache.out_tokens), cache.ring, K.ptr(cache.step_counter),
                     K.ptr(logits), K.ptr(cache.scratch(batch, splits)), splits, ctx)
        return d, rows

    def _graph(self, cache: SlotCache, batch: int, ctx: int, steps: int, logits: torch.Tensor | None):
        key = (batch, ctx, steps, K.ptr(logits))
        g = cache._graphs.get(key)
        if g is None and len(cache._graphs) >= cache.max_graphs:
            # a long-lived engine with ragged batches meets ever new (rows, context bound, steps):
            # start over rather than keep thousands of graphs and their scratch arenas
            torch.cuda.synchronize(self.device)
            cache.release_graphs()
        d, rows = self._decode_struct(cache, batch, ctx, logits)
        if g is None:
            if not hasattr(self, "_capture_stream"):
                # kernel nodes keep the priority of the stream they were captured on: decode steps go
                # ahead of a prefill that runs beside them on another stream
                self._capture_stream = torch.cuda.Stream(device=self.device, priority=-1)
            out = C.c_void_p()
            K.check(K.lib().quic_decode_graph_create(C.byref(self._c_model), C.byref(d), steps,
                                                     self._capture_stream.cuda_stream, C.byref(out)),
                    "decode_graph_create")
            g = out.value
            cache._graphs[key] = g
        return g, rows

    # ---- persistent decode kernel ------------------------------------------------------
    def persist_stream(self) -> torch.Tensor:
        """The per-CTA weight stream of the persistent kernel, packed on first use from the
        W4T matrices (a second copy of the layer weights, ~10 MB per layer)."""
        if self._wstream is None:
            need = K.lib().quic_persist_stream_bytes(self.n_layers)
            if need <= 0:
                raise RuntimeError("persistent decode: unsupported layer count")
            t = torch.empty(need, dtype=torch.uint8, device=self.device)
            K.check(K.lib().quic_persist_pack(C.byref(self._c_model), K.ptr(t), K.stream_ptr()), "persist_pack")
            self._wstream = t
        return self._wstream

    def persist_ok(self, batch: int, ctx: int) -> bool:
        """Whether ``batch`` rows with contexts up to ``ctx`` tokens run in the persistent kernel."""
        lib = K.lib()
        return (self.use_persist and not self.dense and batch <= lib.quic_persist_max_rows() and self.vocab >= 296
                and lib.quic_persist_stream_bytes(self.n_layers) > 0
                and lib.quic_persist_pick_splits(batch, ctx) <= 16)

    def launches_per_step(self, cache: SlotCache | None = None, batch: int = 1, ctx: int = 1024) -> int:
        """Kernels one decode step launches for ``batch`` rows at a context bound of ``ctx``
        (the persistent kernel is one launch per burst, counted as one per step here)."""
        if self.persist_ok(batch, ctx):
            return 1
        if cache is None:
            return 5 * self.n_layers + 1
        d, _ = self._decode_struct(cache, batch, ctx, None)
        return int(K.lib().quic_decode_launch_count(C.byref(self._c_model), C.byref(d)))

    def _prepare_decode(self, cache: SlotCache, slots: list[int], steps: int, logits):
        """Checks the request, loads the row->slot map and returns (handle, ring index of the
        first generated token row) after advancing the host mirrors.  ``handle`` is a captured
        graph (int) or, for the persistent kernel, the quic_decode_t of the launch."""
        if not slots:
            raise RuntimeError("decode: empty batch")
        cache.check_slots(slots, len(slots), "decode")
        if steps < 1 or steps > cache.ring:
            raise RuntimeError(f"decode: steps must be in 1..{cache.ring}")
        longest = max(cache.host_len[s] for s in slots)
        if longest + steps > cache.s_max or longest + steps > self.max_pos:
            raise RuntimeError("decode: context would exceed the KV slot length")
        ctx = min(_ctx_bucket(longest + steps, len(slots)), cache.s_max)
        if self.persist_ok(len(slots), ctx):
            g, rows = self._decode_struct(cache, len(slots), ctx, logits, persist=True)
        else:
            g, rows = self._graph(cache, len(slots), ctx, steps, logits)
        want = cache.rows_tensor(slots)
        if cache._rows_loaded.get(len(slots)) is not want:
            rows.copy_(want)
            cache._rows_loaded[len(slots)] = want
        first = cache.host_steps
        cache.host_steps = first + steps
        for s in slots:
            cache.host_len[s] += steps
        return g, first % cache.ring

    def decode_async(self, cache: SlotCache, slots: list[int], steps: int,
                     logits: torch.Tensor | None = None) -> int:
        """Enqueues ``steps`` greedy decode steps for the rows ``slots`` (no host sync).
        Returns the ring index of the first generated token row in ``cache.out_tokens``."""
        g, first = self._prepare_decode(cache, slots, steps, logits)
        self._launch(cache, g, steps)
        return first

    def _launch(self, cache: SlotCache, handle, steps: int) -> None:
        if isinstance(handle, K.Decode):
            K.check(K.lib().quic_decode_persist(C.byref(self._c_model), C.byref(handle), K.ptr(self.persist_stream()),
                                                K.ptr(cache.persist_sync()), steps, K.stream_ptr()), "decode_persist")
        else:
            K.check(K.lib().quic_graph_launch(handle, K.stream_ptr()), "graph_launch")

    def persist_status(self, cache: SlotCache) -> int:
        """Status word of the persistent kernel (0 = every wait was met); reading clears it
        and synchronises the stream."""
        out = C.c_int32(0)
        K.check(K.lib().quic_decode_persist_status(K.ptr(cache.persist_sync()), K.stream_ptr(), C.byref(out)),
                "decode_persist_status")
        return int(out.value)

    def decode(self, cache: SlotCache, slots: list[int], steps: int,
               feed: torch.Tensor | None = None) -> list[list[int]]:
        """``steps`` greedy tokens for every row: result[i][j] is token j of slots[i].

        The host-driven form of the reference's token loop (src/engine.py:82-104) in one
        library call: the optional ``feed`` (page-locked int32 [len(slots)], the token each
        row consumes first; ``slots`` must then be consecutive) travels host -> device, the
        captured steps run, the generated ids travel device -> host into a page-locked
        buffer, and the call returns when they have arrived."""
        n_in = 0
        if feed is not None:
            if feed.dtype != torch.int32 or feed.numel() != len(slots) or feed.is_cuda:
                raise ValueError("decode: feed must be a host int32 tensor with one token per row")
            n_in = len(slots)
        # A plan keeps everything that stays the same between calls for the same rows while
        # the context stays inside the captured graph's bound.
        key = (tuple(slots), steps)
        plan = cache._plans.get(key)
        first = cache.host_steps % cache.ring
        host_len = cache.host_len
        if (plan is not None and first + steps <= cache.ring
                and max(host_len[s] for s in slots) + steps <= plan[1]
                and cache._rows_loaded.get(len(slots)) is plan[2]):
            g = plan[0]
            cache.host_steps += steps
            for s in slots:
                host_len[s] += steps
        else:
            if n_in and any(b - a != 1 for a, b in zip(slots, slots[1:])):
                raise ValueError("decode: feed needs consecutive slots")
            g, first = self._prepare_decode(cache, slots, steps, None)
            longest = max(host_len[s] for s in slots)  # already advanced by `steps`
            bound = min(_ctx_bucket(longest, len(slots)), cache.s_max, self.max_pos)
            host = cache.host_out()
            plan = (g, bound, cache.rows_tensor(slots), cache.tok.data_ptr() + 4 * slots[0],
                    cache.out_tokens.data_ptr(), host.data_ptr(), host.numpy())
            if len(cache._plans) > 64:
                cache._plans.clear()
            cache._plans[key] = plan
            if first + steps > cache.ring:  # the block of rows wraps around the ring
                if n_in:
                    cache.tok[slots[0]: slots[0] + n_in].copy_(feed, non_blocking=True)
                self._launch(cache, g, steps)
                idx = (torch.arange(steps, device=self.device) + first) % cache.ring
                toks = cache.out_tokens.index_select(0, idx).index_select(1, cache.rows_tensor(slots).long())
                return toks.t().cpu().tolist()
        n = cache.n_slots
        offset = 4 * first * n
        if isinstance(g, K.Decode):
            sync = cache.persist_sync()
            rc = K.lib().quic_decode_persist_run_host(
                C.byref(self._c_model), C.byref(g), K.ptr(self.persist_stream()), K.ptr(sync), steps, K.stream_ptr(),
                feed.data_ptr() if n_in else None, plan[3], n_in, plan[4] + offset, plan[5] + offset, steps * n,
                cache._persist_status.data_ptr())
        else:
            rc = K.lib().quic_graph_run_host(g, K.stream_ptr(), feed.data_ptr() if n_in else None, plan[3], n_in,
                                             plan[4] + offset, plan[5] + offset, steps * n)
        if rc != 0:
            K.check(rc, "decode run_host")
        host_np = plan[6]
        if steps == 1 and len(slots) == 1:
            return [[int(host_np[first, slots[0]])]]
        return host_np[first: first + steps][:, slots].T.tolist()

    # ---- prefill -----------------------------------------------------------------
    @torch.inference_mode()
    def prefill(self, cache: SlotCache, slots: list[int], prompts: list[torch.Tensor],
                all_logits: bool = False, offsets: list[int] | None = None):
        """Runs the prompts (1-D int64 tensors) through the model, fills their KV slots and
        returns (first greedy token per prompt [n] int64, logits).  Linear layers run at
        M = total prompt tokens; attention is the library's causal prefill kernel, every
        sequence in one launch (the reference: src/model.py:164-199, prefill attention
        kernels/flash_attn_prefill_pytorch.py:10 / kernels/cuda/flash_attn_prefill.cu:87).

        ``offsets[i]`` > 0 makes ``prompts[i]`` the NEXT chunk of a prompt whose first
        offsets[i] tokens are already in slot slots[i] (chunked prefill): positions continue
        from there and attention sees the cached tokens as well."""
        dev = self.device
        cache.check_slots(slots, len(prompts), "prefill")
        lens = [int(p.numel()) for p in prompts]
        offs = [0] * len(lens) if offsets is None else [int(o) for o in offsets]
        if len(offs) != len(lens) or any(o < 0 for o in offs):
            raise ValueError("prefill: one non-negative offset per prompt")
        if any(o > 0 and cache.host_len[s] != o for s, o in zip(slots, offs)):
            raise ValueError("prefill: an offset must equal the tokens already cached in the slot")
        if any(n < 1 for n in lens):
            raise RuntimeError("prefill: empty prompt")
        if any(o + n > cache.s_max or o + n > self.max_pos for n, o in zip(lens, offs)):
            raise RuntimeError("prefill: prompt longer than the KV slot")
        bounds = [0]
        for n in lens:
            bounds.append(bounds[-1] + n)
        if not all_logits:
            return self._prefill_fused(cache, slots, prompts, lens, bounds, offs)
        ids = torch.cat([p.reshape(-1) for p in prompts]).to(dev, torch.long)
        # per token: its KV slot and its position (one small host -> device copy each)
        pos = torch.cat([torch.arange(o, o + n, dtype=torch.int32) for n, o in zip(lens, offs)]).to(dev, non_blocking=True)
        slot_of = torch.repeat_interleave(torch.tensor(slots, dtype=torch.int32),
                                          torch.tensor(lens)).to(dev, non_blocking=True)
        table = torch.tensor([bounds[:-1], lens, slots, offs], dtype=torch.int32).to(dev, non_blocking=True)
        seq_start, seq_len, seq_slot, seq_off = table[0], table[1], table[2], table[3]
        h = self.embed[ids]
        rms, lin = K.rmsnorm().forward, K.w4a16_linear
        xn = rms(h, self.layers[0]["ln1"], self.eps)
        for li, L in enumerate(self.layers):
            qkv = lin(L["qkv"], xn)
            # heads split, RoPE applied and K/V written into their slots by one kernel
            q = K.qkv_rope_append(qkv, slot_of, pos, self.rope_cos, self.rope_sin, cache.kv[li, 0], cache.kv[li, 1])
            attn = K.attn_prefill(q, cache.kv[li, 0], cache.kv[li, 1], seq_start, seq_len, seq_slot, max(lens),
                                  seq_off=seq_off)
            o = lin(L["o"], attn)
            xn, h = rms(o, L["ln2"], self.eps, residual=h)
            gu = lin(L["gate_up"], xn)
            act = K.swiglu_fused(gu)
            d = lin(L["down"], act)
            nxt = self.layers[li + 1]["ln1"] if li + 1 < self.n_layers else self.final_norm
            xn, h = rms(d, nxt, self.eps, residual=h)
        last = torch.tensor([b - 1 for b in bounds[1:]], device=dev)
        logits = K.gemm().forward(xn, self.embed)
        first = K.sampler().forward(logits[last].unsqueeze(1)).view(-1)
        st = torch.tensor(slots, device=dev, dtype=torch.long)
        cache.tok[st] = first.to(torch.int32)
        cache.pos[st] = torch.tensor([o + n for n, o in zip(lens, offs)], device=dev, dtype=torch.int32)
        for s, n, o in zip(slots, lens, offs):
            cache.host_len[s] = o + n
        return first, logits

    def _prefill_fused(self, cache: SlotCache, slots: list[int], prompts: list[torch.Tensor], lens: list[int],
                       bounds: list[int], offs: list[int]):
        """The whole prefill as ONE library call (quic_prefill): the host builds one int32 table
        (token ids, slot and position per row; start / length / slot / tokens already cached
        per sequence), copies it once, and reads nothing back."""
        dev = self.device
        rows, n_seq = bounds[-1], len(lens)
        table = torch.empty(3 * rows + 4 * n_seq, dtype=torch.int32)
        table[:rows] = torch.cat([p.reshape(-1) for p in prompts])
        table[rows:2 * rows] = torch.repeat_interleave(torch.tensor(slots, dtype=torch.int32), torch.tensor(lens))
        table[2 * rows:3 * rows] = torch.cat([torch.arange(o, o + n, dtype=torch.int32) for n, o in zip(lens, offs)])
        table[3 * rows:] = torch.tensor([bounds[:-1], lens, slots, offs], dtype=torch.int32).reshape(-1)
        t = table.to(dev, non_blocking=True)
        need = K.lib().quic_prefill_scratch_bytes(rows, n_seq, self.vocab)
        scratch = cache.__dict__.get("_prefill_scratch")
        if scratch is None or scratch.numel() < need:
            scratch = torch.zeros(int(need * 1.25), dtype=torch.uint8, device=dev)
            cache._prefill_scratch = scratch
        first = torch.empty(n_seq, dtype=torch.int64, device=dev)
        logits = torch.empty(n_seq, self.vocab, dtype=DTYPE, device=dev)
        base = t.data_ptr()
        p = K.Prefill(base, base + 4 * rows, base + 8 * rows, base + 12 * rows, base + 12 * rows + 4 * n_seq,
                      base + 12 * rows + 8 * n_seq, rows, n_seq, max(lens), K.ptr(cache.kv), cache.n_slots,
                      cache.s_max, K.ptr(cache.tok), K.ptr(cache.pos), K.ptr(first), K.ptr(logits), K.ptr(scratch),
                      base + 12 * rows + 12 * n_seq if any(offs) else None)
        K.check(K.lib().quic_prefill(C.byref(self._c_model), C.byref(p), K.stream_ptr()), "prefill")
        for s_, n, o in zip(slots, lens, offs):
            cache.host_len[s_] = o + n
        return first, logits

    # ---- reference-shaped forward ------------------------------------------------------
    @torch.inference_mode()
    def forward(self, input_ids: torch.Tensor, past_key_values: SlotCache | None = None,
                attention_mask: torch.Tensor | None = None, position_ids: torch.Tensor | None = None,
                use_cache: bool = True) -> CausalLMOutput:
        """Same contract as the reference's forward (src/model.py:272-303): ``input_ids``
        [B, T]; ``attention_mask`` [B, kv_len] with zeros on the LEFT padding; returns fp16
        logits and the cache.  ``position_ids`` are implied by the cache (#real tokens so
        far, exactly what the reference's engine passes, src/engine.py:93-95)."""
        if input_ids.dim() != 2:
            raise ValueError("input_ids must be [batch, seq_len]")
        batch, seq_len = input_ids.shape
        cache = past_key_values
        if cache is None:
            cache = self.new_cache(n_slots=max(batch, self.default_slots))
        if not cache.batch_slots:
            cache.batch_slots = list(range(batch))
        if len(cache.batch_slots) != batch:
            raise ValueError(f"cache holds {len(cache.batch_slots)} rows, input has {batch}")
        cache.check_slots(cache.batch_slots, batch, "forward")
        past_len = cache.get_seq_length()
        kv_len = past_len + seq_len
        input_ids = input_ids.to(self.device)
        if seq_len == 1:
            if any(cache.host_len[s] == 0 for s in cache.batch_slots) and attention_mask is None:
                pass  # a one-token prompt: handled by the decode kernels as position 0
            logits = cache.__dict__.setdefault("_logits", {}).get(batch)
            if logits is None:
                logits = torch.empty(batch, self.vocab, dtype=DTYPE, device=self.device)
                cache._logits[batch] = logits
            st = cache.rows_tensor(cache.batch_slots).long()
            cache.tok[st] = input_ids.view(-1).to(torch.int32)
            self.decode_async(cache, cache.batch_slots, 1, logits=logits)
            return CausalLMOutput(logits=logits.view(batch, 1, self.vocab),
                                  past_key_values=cache if use_cache else None)
        if past_len != 0:
            # the next chunk of every row's prompt (the reference's forward accepts a multi-token
            # input on a filled cache, src/model.py:280-291): no new padding can appear here
            if any(cache.host_len[s] == 0 for s in cache.batch_slots):
                raise RuntimeError("forward: a multi-token input continues rows that are already cached")
            if attention_mask is not None and not bool(attention_mask[:, -seq_len:].bool().all()):
                raise ValueError("forward: the tokens of a continuation cannot be padding")
            offs = [cache.host_len[s] for s in cache.batch_slots]
            want_all = self.prefill_all_logits
            _, logits = self.prefill(cache, cache.batch_slots, [input_ids[b] for b in range(batch)],
                                     all_logits=want_all, offsets=offs)
            logits = logits.view(batch, seq_len, self.vocab) if want_all else logits.view(batch, 1, self.vocab)
            return CausalLMOutput(logits=logits, past_key_values=cache if use_cache else None)
        if attention_mask is not None:
            if tuple(attention_mask.shape) != (batch, kv_len):
                raise ValueError(f"attention_mask {tuple(attention_mask.shape)} does not match "
                                 f"(batch={batch}, kv_len={kv_len})")
            lens = attention_mask.to(torch.long).sum(dim=1).tolist()
        else:
            lens = [seq_len] * batch
        prompts = [input_ids[b, seq_len - n:] for b, n in enumerate(lens)]
        want_all = self.prefill_all_logits
        _, logits = self.prefill(cache, cache.batch_slots, prompts, all_logits=want_all)
        if want_all:
            full = torch.zeros(batch, seq_len, self.vocab, dtype=DTYPE, device=self.device)
            a = 0
            for b, n in enumerate(lens):
                full[b, seq_len - n:] = logits[a:a + n]
                a += n
            logits = full
        else:
            logits = logits.view(batch, 1, self.vocab)
        return CausalLMOutput(logits=logits, past_key_values=cache if use_cache else None)


# ---- loading ---------------------------------------------------------------------------
def from_state_dict(weights: dict, config: dict, device="cuda") -> QUICForCausalLM:
    if not torch.cuda.is_available():
        raise RuntimeError("quic_b200 needs a CUDA device (no CPU path)")
    model = QUICForCausalLM(config, device=device)
    model.load_state(weights)
    return model


def load(path: str, prefill_backend: str = "pytorch", use_marlin: bool = False, use_machete: bool = False,
         tokenizer_path: str | None = None):
    """Same signature and return value as the reference's ``model.load`` (src/model.py:306).
    ``use_marlin`` / ``use_machete`` are accepted for compatibility; every packed layer runs
    the W4A16 kernels of this package.  The tokenizer is loaded when its files exist."""
    from safetensors.torch import load_file

    path = os.path.expanduser(path)
    with open(os.path.join(path, "config.json")) as handle:
        config = json.load(handle)
    weights = load_file(os.path.join(path, "model.safetensors"))
    if packed_prefixes(weights):  # (an un-quantised checkpoint runs the dense fp16 kernels)
        group = detect_group_size(config)
        if group != K.GROUP:
            raise RuntimeError(f"quic_b200 kernels are built for group size {K.GROUP}, checkpoint has {group}")
    model = from_state_dict(weights, config)
    if prefill_backend is not None:
        model.prefill_backend = prefill_backend
    tokenizer = None
    tok_dir = tokenizer_path or path
    if os.path.exists(os.path.join(tok_dir, "tokenizer.json")):
        from transformers import AutoTokenizer

        tokenizer = AutoTokenizer.from_pretrained(tok_dir)
    return model, tokenizer
