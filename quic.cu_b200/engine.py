"""Static / continuous batching engine over KV slots.

Keeps the reference's API (src/engine.py:26-168): ``Engine(registry, max_batch_size, config,
model_module)``, ``add_request(prompt)``, ``step()``, ``run() -> outputs sorted by request id``,
with the same request semantics:

* FIFO admission decided by the policies of ``scheduler`` before every iteration
  (src/engine.py:115-160);
* greedy sampling; the EOS token IS appended and ends the request, ``max_tokens`` caps it
  (src/engine.py:180-184, src/sequence.py:15-19);
* under static batching finished rows keep their slot until the whole batch has finished
  (src/scheduler.py:34-45).

What differs is where the state lives.  The reference keeps one left-padded batch whose
cache length only grows and rebuilds it with torch.cat on every admission
(src/engine.py:225-277).  Here every request owns a KV slot that stores real tokens only;
admission prefills into a free slot, release frees it, and an iteration is a burst of
``decode_burst`` greedy steps that run on the device from one CUDA graph launch, with one
device->host copy of the burst's tokens.  Tokens produced by a row after it finished are
discarded exactly as the reference discards them (src/engine.py:180-182).

With ``overlap_prefill`` (default) a request admitted while other rows are running is
prefilled on a second CUDA stream during those rows' next decode burst and joins the batch at
the following iteration: slots are disjoint, so the two never touch the same cache rows, and
the side stream is synchronised before any decode launch that includes the new rows.  The
outputs are the same (every request is an independent greedy decode); only the iteration at
which a request starts to decode moves by one.

``model_module.load(**options)`` must return ``(model, tokenizer)``; the model is driven
through three calls: ``new_cache(n_slots, s_max)``, ``prefill(cache, slots, prompts)`` and
``decode(cache, slots, steps)``.
"""

from __future__ import annotations

import itertools
from collections import deque

import torch

from .config import EngineConfig
from .metrics import MetricsRegistry, Span
from .scheduler import ContinuousAdmissionPolicy, StaticAdmissionPolicy
from .sequence import SequenceState

BATCHING_POLICIES = {
    "static": StaticAdmissionPolicy,
    "continuous": ContinuousAdmissionPolicy,
}


class Engine:
    def __init__(self, registry: MetricsRegistry | None = None, max_batch_size: int = 8,
                 config: EngineConfig | None = None, model_module=None) -> None:
        if config is None:
            config = EngineConfig()
        self.config = config
        self.max_batch_size = max_batch_size
        self.running: list[SequenceState] = []
        self.waiting: deque[SequenceState] = deque()

        load_options: dict[str, str | bool] = {}
        if config.model_path is not None:
            load_options["path"] = config.model_path
        if config.tokenizer_path is not None:
            load_options["tokenizer_path"] = config.tokenizer_path
        if config.use_machete:
            load_options["use_machete"] = True
        if getattr(config, "prefill_backend", None) is not None:
            load_options["prefill_backend"] = config.prefill_backend

        if model_module is None:
            from . import model as model_module  # the CUDA model; raises without the library
        self.model, self.tokenizer = model_module.load(**load_options)
        if getattr(config, "prefill_backend", None) is not None and hasattr(self.model, "prefill_backend"):
            self.model.prefill_backend = config.prefill_backend  # also for a model handed in ready-made
        self.max_tokens = 256
        self.registry = registry
        self.burst = max(1, int(config.decode_burst))
        self.overlap_prefill = bool(getattr(config, "overlap_prefill", True))
        self._prefill_stream = None
        self._decode_stream = None
        self.cache = self.model.new_cache(max_batch_size, config.max_context)
        self.free_slots: list[int] = list(range(max_batch_size))
        self._request_id_generator = itertools.count(1)
        self.batching_policy = BATCHING_POLICIES[config.batching]()
        self.eos_token_id = getattr(self.tokenizer, "eos_token_id", None)
        self.decode_steps = 0      # device decode iterations issued
        self.generated = 0         # tokens kept
        # Optional pull-based feed (request-sharded replicas): before every scheduling decision
        # ``request_source(room)`` is asked for up to ``room`` more requests (the slots that
        # are free or about to be), as (token ids, max_tokens, tag) triples; it returns []
        # when it has nothing (now).  ``on_finish``
        # is called with (tag, output) when a request that carries a tag is released.
        self.request_source = None
        self.on_finish = None
        self._tags: dict[int, object] = {}
        # chunked prefill: sequences whose prompt is only partly in their slot, and how much is
        self.prefill_chunk = getattr(config, "prefill_chunk", None)
        self.prefilling: list[SequenceState] = []
        self._prefilled: dict[int, int] = {}

    # ---- requests ------------------------------------------------------------------
    def add_request(self, prompt: str) -> int:
        """Chat-templated text request (src/engine.py:59-75)."""
        if self.tokenizer is None:
            raise RuntimeError("add_request(str) needs a tokenizer; use add_request_ids")
        encoding = self.tokenizer.apply_chat_template(
            [{"role": "user", "content": prompt}], add_generation_prompt=True,
            return_tensors="pt", return_dict=True)
        return self.add_request_ids(encoding["input_ids"])

    def add_request_ids(self, input_ids, max_tokens: int | None = None, tag=None) -> int:
        """Token-id request: ``input_ids`` is a list or a [1, T] / [T] tensor.  ``tag`` travels
        with the request and is handed to ``on_finish`` with its output."""
        ids = torch.as_tensor(input_ids, dtype=torch.long).reshape(1, -1).cpu()
        if ids.shape[1] < 1:
            raise ValueError("empty prompt")
        limit = self.max_tokens if max_tokens is None else max_tokens
        if ids.shape[1] + limit + self.burst > self.config.max_context:
            raise ValueError(f"prompt ({ids.shape[1]}) + max_tokens ({limit}) + burst does not fit a "
                             f"KV slot of {self.config.max_context} tokens")
        request_id = next(self._request_id_generator)
        seq = SequenceState(prompt_tokens=ids, request_id=request_id, max_tokens=limit)
        self._tags[request_id] = tag
        self.waiting.append(seq)
        return request_id

    # ---- one iteration ---------------------------------------------------------------
    def _update_sequence_with_token(self, sequence: SequenceState, token: int) -> None:
        if not sequence.is_finished:
            sequence.generated_tokens.append(token)
            self.generated += 1
            if self.eos_token_id is not None and token == self.eos_token_id:
                sequence.finished_at = len(sequence.generated_tokens) - 1

    @torch.inference_mode()
    def step(self, steps: int | None = None) -> None:
        """One decode iteration: ``steps`` greedy tokens for every unfinished row."""
        with Span("step", self.registry):
            with Span("prepare_decode", self.registry):
                live = [seq for seq in self.running if not seq.is_finished]
                if not live:
                    return
                if steps is None:
                    # a full burst whenever some row still needs one (keeps the set of captured
                    # graphs small); rows that finish inside the burst discard the overshoot
                    need = max(seq.max_tokens - len(seq.generated_tokens) for seq in live)
                    steps = self.burst if need >= self.burst else max(1, need)
                slots = [seq.slot for seq in live]
            with Span("forward_pass", self.registry):
                tokens = self.model.decode(self.cache, slots, steps)
                self.decode_steps += steps
            with Span("sample_and_update", self.registry):
                for seq, row in zip(live, tokens):
                    for token in row:
                        self._update_sequence_with_token(seq, int(token))

    @torch.inference_mode()
    def _prefill_begin(self, sequences: list[SequenceState], stream=None):
        """Assigns slots to new sequences and enqueues the prefill of every sequence's next
        chunk (the whole prompt without ``prefill_chunk``), on ``stream`` when given; nothing is
        read back yet.  Returns what ``_prefill_end`` needs."""
        for seq in sequences:
            if seq.slot is None:
                seq.slot = self.free_slots.pop(0)
        slots = [s.slot for s in sequences]
        offs = [self._prefilled.get(s.request_id, 0) for s in sequences]
        prompts, done = [], []
        for seq, off in zip(sequences, offs):
            ids = seq.prompt_tokens.view(-1)
            end = ids.numel() if not self.prefill_chunk else min(ids.numel(), off + int(self.prefill_chunk))
            prompts.append(ids[off:end])
            done.append(end)
        kwargs = {"offsets": offs} if any(offs) else {}
        if stream is None:
            first, _ = self.model.prefill(self.cache, slots, prompts, **kwargs)
        else:
            stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(stream):
                first, _ = self.model.prefill(self.cache, slots, prompts, **kwargs)
        return sequences, first, stream, done

    @torch.inference_mode()
    def _prefill_end(self, pending) -> list[SequenceState]:
        """Reads the first tokens back.  Sequences whose whole prompt is now cached get theirs
        and are returned (they join the running rows); the others stay in ``prefilling``."""
        sequences, first, stream, done = pending
        if stream is not None:
            stream.synchronize()  # the slots are complete before any later decode launch
        first = first.tolist() if hasattr(first, "tolist") else list(first)
        complete, self.prefilling = [], []
        for seq, token, end in zip(sequences, first, done):
            if end >= seq.prompt_tokens.numel():
                self._prefilled.pop(seq.request_id, None)
                self._update_sequence_with_token(seq, int(token))
                complete.append(seq)
            else:  # (the token predicted after a partial prompt is not used)
                self._prefilled[seq.request_id] = end
                self.prefilling.append(seq)
        return complete

    def _prefill_sequences(self, sequences: list[SequenceState]) -> list[SequenceState]:
        return self._prefill_end(self._prefill_begin(sequences))

    def _side_stream(self):
        """Second CUDA stream for overlapped prefills (None for a model that is not on a GPU)."""
        device = getattr(self.model, "device", None)
        if device is None or getattr(device, "type", "cpu") != "cuda":
            return None
        if self._prefill_stream is None:
            self._prefill_stream = torch.cuda.Stream(device=device)
        return self._prefill_stream

    def _main_stream(self):
        """With overlapped prefills the loop runs on a stream of high priority, so that the short
        kernels of a decode step get the next free SM ahead of a prefill's long ones (measured
        +4 % generated tokens/s on the 4096-request queue).  None: stay on the caller's stream."""
        device = getattr(self.model, "device", None)
        if not self.overlap_prefill or device is None or getattr(device, "type", "cpu") != "cuda":
            return None
        if self._decode_stream is None:
            self._decode_stream = torch.cuda.Stream(device=device, priority=-1)
        return self._decode_stream

    def _finish(self, seq: SequenceState):
        if self.tokenizer is not None:
            return self.tokenizer.decode(seq.generated_tokens, skip_special_tokens=True)
        return list(seq.generated_tokens)

    @torch.inference_mode()
    def run(self) -> list:
        """Serves the queue to completion; outputs ordered by request id (src/engine.py:168).
        Decoded strings with a tokenizer, token-id lists without one."""
        main = self._main_stream()
        if main is None:
            return self._run()
        caller = torch.cuda.current_stream(main.device)
        main.wait_stream(caller)
        with torch.cuda.stream(main):
            outputs = self._run()
        caller.wait_stream(main)
        return outputs

    def _run(self) -> list:
        outputs: dict[int, object] = {}
        with Span("request run", self.registry):
            while True:
                with Span("scheduling", self.registry):
                    if self.request_source is not None:
                        # ask only for what can be admitted now (slots that are free or about to
                        # be released): requests a replica hoards are requests another replica
                        # could be serving
                        done = sum(1 for seq in self.running if seq.is_finished)
                        room = len(self.free_slots) + done - len(self.waiting)
                        if room > 0:
                            for ids, limit, tag in self.request_source(room):
                                self.add_request_ids(ids, max_tokens=limit, tag=tag)
                    # (sequences still prefilling hold a slot: they count as running for admission)
                    decision = self.batching_policy.decide(self.running + self.prefilling, self.waiting,
                                                           self.max_batch_size)
                    released = {seq.request_id for seq in decision.release}
                    for seq in decision.release:
                        outputs[seq.request_id] = self._finish(seq)
                        tag = self._tags.pop(seq.request_id, None)
                        if self.on_finish is not None and tag is not None:
                            self.on_finish(tag, outputs[seq.request_id])
                        self.free_slots.append(seq.slot)
                        seq.slot = None
                    if released:
                        self.running = [s for s in self.running if s.request_id not in released]
                pending = None
                if decision.admit or self.prefilling:
                    with Span("prefill", self.registry):
                        admitted = self.prefilling + [self.waiting.popleft() for _ in decision.admit]
                        if self.overlap_prefill and any(not seq.is_finished for seq in self.running):
                            # the rows already running decode their burst while the admitted
                            # prompts (or their next chunks) prefill into their (disjoint) slots;
                            # they join afterwards
                            pending = self._prefill_begin(admitted, self._side_stream())
                        else:
                            self.running.extend(self._prefill_sequences(admitted))
                if not self.running and pending is None and not self.prefilling:
                    break
                self.step()
                if pending is not None:
                    with Span("prefill", self.registry):
                        self.running.extend(self._prefill_end(pending))
        return [outputs[request_id] for request_id in sorted(outputs)]
