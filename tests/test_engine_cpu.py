"""Engine semantics on the CPU with an injected fake model (no CUDA involved)."""

import pytest
import torch

from quic_cu_b200.config import EngineConfig
from quic_cu_b200.engine import Engine
from tests.fake_model import EOS, FakeModule, expected_generation


def _engine(batching, max_batch=4, burst=3, tokenizer=None, **kw):
    module = FakeModule(tokenizer)
    cfg = EngineConfig(batching=batching, decode_burst=burst, max_context=256, **kw)
    return Engine(config=cfg, max_batch_size=max_batch, model_module=module), module


def test_empty_run_returns_empty_list():  # reference tests/test_engine.py:12
    engine, _ = _engine("continuous")
    assert engine.run() == []


@pytest.mark.parametrize("batching", ["static", "continuous"])
@pytest.mark.parametrize("burst", [1, 3, 8])
@pytest.mark.parametrize("overlap", [True, False])
def test_outputs_equal_independent_greedy_generation(batching, burst, overlap):
    engine, module = _engine(batching, max_batch=3, burst=burst, overlap_prefill=overlap)
    engine.max_tokens = 16
    prompts = [[5, 6, 7], [1], [9, 9, 9, 9], [2, 3], [11] * 10, [4, 5], [8]]
    limits = [16, 3, 16, 1, 9, 16, 2]
    for p, lim in zip(prompts, limits):
        engine.add_request_ids(p, max_tokens=lim)
    outputs = engine.run()
    assert len(outputs) == len(prompts)
    for out, p, lim in zip(outputs, prompts, limits):  # ordered by request id
        assert out == expected_generation(p, lim, eos=None)
    assert sorted(engine.free_slots) == [0, 1, 2]
    assert not engine.running and not engine.waiting
    if batching == "static":
        # a new batch is admitted only once every row of the previous one has finished
        prefills = [c[1] for c in module.model.calls if c[0] == "prefill"]
        assert [len(p) for p in prefills] == [3, 3, 1]


def test_eos_is_appended_and_ends_the_request():  # src/engine.py:180-184
    class Tok:
        eos_token_id = EOS

        def decode(self, tokens, skip_special_tokens=True):
            return " ".join(str(t) for t in tokens)

    engine, _ = _engine("continuous", tokenizer=Tok())
    found = None
    for start in range(1, 60):
        gen = expected_generation([start], 40)
        if gen[-1] == EOS and 1 < len(gen) < 40:
            found = (start, gen)
            break
    assert found, "no prompt of the fake model reaches EOS"
    engine.add_request_ids([found[0]], max_tokens=40)
    out = engine.run()
    assert out == [" ".join(str(t) for t in found[1])]


def test_load_options_follow_the_reference_engine():  # src/engine.py:40-51
    engine, module = _engine("continuous", model_path="/m", tokenizer_path="/t")
    assert module.options == {"path": "/m", "tokenizer_path": "/t", "prefill_backend": "quic"}
    engine2, module2 = _engine("static")
    assert module2.options == {"prefill_backend": "quic"}


def test_request_that_cannot_fit_a_slot_is_rejected():
    engine, _ = _engine("continuous")
    with pytest.raises(ValueError):
        engine.add_request_ids(list(range(250)), max_tokens=16)
    with pytest.raises(ValueError):
        engine.add_request_ids([])
    with pytest.raises(RuntimeError):
        engine.add_request("text needs a tokenizer")


def test_continuous_refills_vacant_slots_while_others_run():
    engine, module = _engine("continuous", max_batch=2, burst=2)
    engine.add_request_ids([1], max_tokens=2)
    engine.add_request_ids([2], max_tokens=12)
    engine.add_request_ids([3], max_tokens=2)
    engine.run()
    calls = module.model.calls
    # request 3 is prefilled into the slot request 1 vacated while request 2 is still decoding
    second_prefill = [i for i, c in enumerate(calls) if c[0] == "prefill"][1]
    assert calls[second_prefill][1] == [0]
    assert any(c[0] == "decode" and len(c[1]) == 2 for c in calls[second_prefill:])


def test_overlapped_admission_prefills_before_the_running_rows_decode():
    """With overlap_prefill a request admitted while another is running is prefilled first (on
    the GPU: on a second stream), the running row decodes alone, and the new row joins the next
    burst; without it the new row decodes in the same iteration."""
    def order(overlap):
        engine, module = _engine("continuous", max_batch=2, burst=2, overlap_prefill=overlap)
        engine.add_request_ids([1], max_tokens=2)
        engine.add_request_ids([2], max_tokens=12)
        engine.add_request_ids([3], max_tokens=4)
        out = engine.run()
        calls = module.model.calls
        second = [i for i, c in enumerate(calls) if c[0] == "prefill"][1]
        return out, [(c[0], len(c[1])) for c in calls[second:second + 3]]

    out_a, seq_a = order(True)
    out_b, seq_b = order(False)
    assert out_a == out_b
    assert seq_a == [("prefill", 1), ("decode", 1), ("decode", 2)]
    assert seq_b == [("prefill", 1), ("decode", 2), ("decode", 2)]


@pytest.mark.parametrize("overlap", [False, True])
def test_chunked_prefill_gives_the_same_outputs_and_interleaves_with_decode(overlap):
    """With prefill_chunk = 4 a 10-token prompt enters its slot in three calls (4, 4, 2 tokens,
    each continuing at the tokens already cached), the rows that are running decode a burst
    between the chunks, and every output equals independent greedy generation."""
    module = FakeModule()
    engine = Engine(max_batch_size=2, model_module=module,
                    config=EngineConfig(batching="continuous", decode_burst=2, overlap_prefill=overlap,
                                        max_context=64, prefill_chunk=4))
    engine.max_tokens = 9
    engine.eos_token_id = None
    prompts = [[3, 4], list(range(20, 30)), [5, 6, 7]]
    for p in prompts:
        engine.add_request_ids(p)
    outputs = engine.run()
    assert outputs == [expected_generation(p, 9, eos=None) for p in prompts]
    calls = module.model.calls
    long_chunks = [(n, o) for c in calls if c[0] == "prefill"
                   for slot, n, o in zip(c[1], c[2], c[3]) if (n, o) in ((4, 0), (4, 4), (2, 8))]
    assert long_chunks == [(4, 0), (4, 4), (2, 8)]
    first = next(i for i, c in enumerate(calls) if c[0] == "prefill" and 4 in c[3])   # second chunk
    last = next(i for i, c in enumerate(calls) if c[0] == "prefill" and 8 in c[3])    # third chunk
    assert any(c[0] == "decode" for c in calls[first:last])  # the short request decodes in between
