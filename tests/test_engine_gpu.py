"""Engine on the GPU: per-request outputs equal the oracle's independent greedy decode."""

from types import SimpleNamespace

import pytest
import torch

from quic_cu_b200.config import EngineConfig
from quic_cu_b200.engine import Engine

pytestmark = pytest.mark.gpu


def _prefix_ok(got, ref_tokens, ref_logits, near_tie=2e-2):
    for i, (g, r) in enumerate(zip(got, ref_tokens)):
        if g != r:
            top = torch.topk(ref_logits[i].float(), 2)
            assert (top.values[0] - top.values[1]).item() < near_tie and g in top.indices.tolist(), (i, g, r)
            return
    assert len(got) == len(ref_tokens)


@pytest.mark.parametrize("batching,prefill_backend", [("static", "pytorch"), ("continuous", "pytorch"),
                                                      ("continuous", "quic")])
def test_engine_multirequest_generation(tiny_model, batching, prefill_backend):  # reference tests/test_engine.py:20
    net, ref, _, _ = tiny_model
    module = SimpleNamespace(load=lambda **options: (net, None))
    engine = Engine(config=EngineConfig(batching=batching, max_context=128, decode_burst=4,
                                        prefill_backend=prefill_backend),
                    max_batch_size=4, model_module=module)
    engine.max_tokens = 10
    gen = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 2048, (n,), generator=gen).tolist() for n in (5, 17, 1, 9, 30, 2, 12)]
    limits = [10, 10, 3, 7, 10, 1, 10]
    for p, lim in zip(prompts, limits):
        engine.add_request_ids(p, max_tokens=lim)
    outputs = engine.run()
    assert len(outputs) == len(prompts)
    for out, p, lim in zip(outputs, prompts, limits):
        ref_tokens, ref_logits = ref.greedy(p, lim)
        assert len(out) == lim
        _prefix_ok(out, ref_tokens, ref_logits)
    assert engine.run() == []
    net.prefill_backend = "pytorch"  # the fixture is shared


@pytest.mark.parametrize("overlap", [True, False])
def test_overlapped_prefill_is_repeatable_and_follows_the_oracle(tiny_model, overlap):
    """More requests than slots, so most admissions happen while other rows decode: with
    overlap_prefill they are prefilled on a second stream during the running rows' burst.  Every
    output follows the oracle, and a second run of the same queue on the same engine returns
    the same tokens (a race between the two streams would show as a difference)."""
    net, ref, _, _ = tiny_model
    module = SimpleNamespace(load=lambda **options: (net, None))
    engine = Engine(config=EngineConfig(batching="continuous", max_context=256, decode_burst=4,
                                        prefill_backend="quic", overlap_prefill=overlap),
                    max_batch_size=3, model_module=module)
    gen = torch.Generator().manual_seed(11)
    lens = [23, 150, 7, 64, 1, 99, 31, 12, 180, 5, 47, 3]
    limits = [9, 14, 30, 5, 22, 11, 1, 17, 8, 26, 13, 6]
    prompts = [torch.randint(0, 2048, (n,), generator=gen).tolist() for n in lens]
    runs = []
    for _ in range(2):
        for p, lim in zip(prompts, limits):
            engine.add_request_ids(p, max_tokens=lim)
        runs.append(engine.run())
    assert runs[0] == runs[1]
    for out, p, lim in zip(runs[0], prompts, limits):
        ref_tokens, ref_logits = ref.greedy(p, lim)
        assert len(out) == lim
        _prefix_ok(out, ref_tokens, ref_logits)
    net.prefill_backend = "pytorch"  # the fixture is shared


def test_load_from_checkpoint_directory(tmp_path, tiny_model):
    """model.load(path) reads config.json + model.safetensors like src/model.py:306-365."""
    from quic_cu_b200 import model as qmodel
    from quic_cu_b200.checkpoint import write_checkpoint_dir

    net, _, state, config = tiny_model
    write_checkpoint_dir(str(tmp_path), state, config)
    loaded, tokenizer = qmodel.load(str(tmp_path), use_marlin=True)
    assert tokenizer is None and len(loaded.layers) == 2
    prompt = torch.tensor([[4, 8, 15, 16, 23, 42]])
    a = net(prompt).logits
    b = loaded(prompt).logits
    assert torch.equal(a, b)
    bad = dict(config, hidden_size=1024)
    with pytest.raises(RuntimeError):
        qmodel.QUICForCausalLM(bad)


def test_forward_rejects_what_the_reference_rejects(tiny_model):
    net, _, _, _ = tiny_model
    with pytest.raises(ValueError):  # src/model.py:286-287
        net(torch.tensor([[1, 2, 3]]), attention_mask=torch.ones(1, 5))
    cache = net.new_cache(n_slots=2, s_max=16)
    cache.batch_slots = [0]
    with pytest.raises(RuntimeError):
        net(torch.arange(20)[None], past_key_values=cache)  # longer than the slot


def test_left_padded_batch_prefill_matches_unpadded(tiny_model):
    """The reference batches by left padding (src/engine.py:187-222); padded rows must give
    the same logits as the same prompts alone."""
    net, _, _, _ = tiny_model
    rows = [[7, 8, 9, 10, 11], [3, 4]]
    ids = torch.tensor([[7, 8, 9, 10, 11], [0, 0, 0, 3, 4]])
    mask = torch.tensor([[1, 1, 1, 1, 1], [0, 0, 0, 1, 1]])
    out = net(ids, attention_mask=mask)
    assert out.logits.shape == (2, 1, 2048)
    for b, row in enumerate(rows):
        alone = net(torch.tensor([row])).logits
        assert torch.allclose(out.logits[b].float(), alone[0].float(), atol=2e-3)
    # one more decode step on the padded batch, mask extended as the reference engine does
    nxt = out.logits[:, -1:, :].argmax(-1)
    mask2 = torch.cat([mask, torch.ones(2, 1, dtype=mask.dtype)], dim=1)
    step = net(nxt, past_key_values=out.past_key_values, attention_mask=mask2)
    assert step.logits.shape == (2, 1, 2048) and torch.isfinite(step.logits).all()
