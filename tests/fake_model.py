"""A CPU stand-in for the model behind the engine's three-call protocol
(new_cache / prefill / decode), injected through ``Engine(model_module=...)`` — the same
seam the reference's engine offers (src/engine.py:32,50-51)."""

from types import SimpleNamespace

EOS = 7


def next_token(prev: int, n_cached: int) -> int:
    return (prev * 31 + n_cached * 17 + 3) % 97


def expected_generation(prompt: list[int], max_tokens: int, eos=EOS) -> list[int]:
    out, n, tok = [], len(prompt), None
    prev = prompt[-1]
    while len(out) < max_tokens:
        tok = next_token(prev, n)
        out.append(tok)
        if eos is not None and tok == eos:
            break
        prev, n = tok, n + 1
    return out


class FakeSlotModel:
    def __init__(self):
        self.calls = []

    def new_cache(self, n_slots, s_max):
        return SimpleNamespace(n_slots=n_slots, s_max=s_max, last=[0] * n_slots, length=[0] * n_slots)

    def prefill(self, cache, slots, prompts, offsets=None):
        """``offsets``: tokens of each prompt already cached (chunked prefill)."""
        offsets = [0] * len(slots) if offsets is None else list(offsets)
        self.calls.append(("prefill", list(slots), [len(p) for p in prompts], offsets))
        first = []
        for slot, prompt, off in zip(slots, prompts, offsets):
            ids = [int(t) for t in prompt]
            assert off == 0 or cache.length[slot] == off, "a chunk continues what the slot holds"
            tok = next_token(ids[-1], off + len(ids))
            cache.last[slot], cache.length[slot] = tok, off + len(ids)
            first.append(tok)
        return first, None

    def decode(self, cache, slots, steps):
        self.calls.append(("decode", list(slots), steps))
        rows = []
        for slot in slots:
            row = []
            for _ in range(steps):
                assert cache.length[slot] + 1 <= cache.s_max
                tok = next_token(cache.last[slot], cache.length[slot] + 1)
                cache.length[slot] += 1
                cache.last[slot] = tok
                row.append(tok)
            rows.append(row)
        return rows


class FakeModule:
    """``load(**options) -> (model, tokenizer)`` like the reference's model module."""

    def __init__(self, tokenizer=None):
        self.model = FakeSlotModel()
        self.tokenizer = tokenizer
        self.options = None

    def load(self, **options):
        self.options = options
        return self.model, self.tokenizer
