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


def _write_stub_tokenizer(path, vocab):
    """WordLevel tokenizer ("t<i>" <-> i, <unk> = 0, <eos> = 1) with a chat template, in the
    files AutoTokenizer reads (tokenizer.json + tokenizer_config.json)."""
    import json
    import os

    from tokenizers import Tokenizer, models, pre_tokenizers

    words = {f"t{i}": i for i in range(2, vocab)}
    words["<unk>"], words["<eos>"] = 0, 1
    tok = Tokenizer(models.WordLevel(words, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.WhitespaceSplit()
    tok.save(os.path.join(path, "tokenizer.json"))
    template = ("{% for m in messages %}t5 {{ m['content'] }} t6{% endfor %}"
                "{% if add_generation_prompt %} t7{% endif %}")
    with open(os.path.join(path, "tokenizer_config.json"), "w") as handle:
        json.dump({"tokenizer_class": "PreTrainedTokenizerFast", "unk_token": "<unk>", "eos_token": "<eos>",
                   "chat_template": template}, handle)


@pytest.mark.parametrize("spelling", ["top_level", "config_groups"])
def test_checkpoint_dir_with_tokenizer_runs_text_requests(tmp_path, tiny_model, spelling):
    """The on-disk form the reference ingests (src/model.py:332-363, src/quant/checkpoint.py:5-20,
    src/engine.py:59-75): a compressed-tensors style directory whose safetensors carry
    ``.weight_shape`` beside the packed tensors, whose quantization_config spells the group
    size at the top level or under config_groups, and whose tokenizer files hold a chat
    template.  Engine(model_path=...) loads it, add_request(str) applies the template, run()
    returns decoded strings; the tokens must be the oracle's."""
    from safetensors import safe_open

    from quic_cu_b200.checkpoint import write_checkpoint_dir
    from quic_cu_b200.config import EngineConfig
    from quic_cu_b200.engine import Engine

    _, ref, state, config = tiny_model
    config = {k: v for k, v in config.items() if k != "quantization_config"}
    if spelling == "top_level":
        config["quantization_config"] = {"quant_method": "compressed-tensors", "group_size": 128, "bits": 4}
    else:
        config["quantization_config"] = {"quant_method": "compressed-tensors", "config_groups": {
            "group_0": {"targets": ["Linear"], "weights": {"num_bits": 4, "group_size": 128, "symmetric": False}}}}
    write_checkpoint_dir(str(tmp_path), state, config)
    _write_stub_tokenizer(str(tmp_path), 2048)
    with safe_open(str(tmp_path / "model.safetensors"), "pt") as handle:
        shapes = [k for k in handle.keys() if k.endswith(".weight_shape")]
        assert len(shapes) == 2 * 7
        assert handle.get_tensor("model.layers.0.mlp.down_proj.weight_shape").tolist() == [896, 4864]

    engine = Engine(max_batch_size=4, config=EngineConfig(model_path=str(tmp_path), max_context=256,
                                                         batching="continuous", prefill_backend="quic"))
    assert engine.tokenizer is not None and engine.eos_token_id == 1
    engine.max_tokens = 12
    texts = ["t10 t11 t12", "t900 t3", "t77 t78 t79 t80 t81 t82"]
    for text in texts:
        engine.add_request(text)
    outputs = engine.run()
    assert len(outputs) == 3 and all(isinstance(o, str) for o in outputs)
    for text, out in zip(texts, outputs):
        ids = [5] + [int(w[1:]) for w in text.split()] + [6, 7]        # the template, by hand
        want_tokens, want_logits = ref.greedy(ids, 12)
        if 1 in want_tokens:                                            # generation stops at <eos>
            want_tokens = want_tokens[: want_tokens.index(1) + 1]
        got = [1 if w == "<eos>" else int(w[1:]) for w in out.split()]
        kept = [t for t in want_tokens if t not in (0, 1)]              # special tokens are skipped on decode
        n = min(len(got), len(kept))
        assert n >= 1
        for i in range(n):
            if got[i] != kept[i]:
                top = torch.topk(want_logits[i].float(), 2)
                assert (top.values[0] - top.values[1]).item() < 2e-2, (text, i, got[i], kept[i])
                break

    bad = dict(config, quantization_config={"quant_method": "compressed-tensors", "group_size": 32})
    write_checkpoint_dir(str(tmp_path), state, bad)
    with pytest.raises(RuntimeError, match="group size"):
        Engine(max_batch_size=2, config=EngineConfig(model_path=str(tmp_path), max_context=64))


def test_engine_with_chunked_prefill_matches_unchunked(tiny_model):
    """prefill_chunk = 16: long prompts enter their slots a chunk per iteration while the
    running rows decode; the outputs are those of the unchunked engine."""
    from quic_cu_b200.config import EngineConfig
    from quic_cu_b200.engine import Engine
    from tests.fake_model import FakeModule

    net = tiny_model[0]
    gen = torch.Generator().manual_seed(31)
    prompts = [torch.randint(0, 2048, (int(n),), generator=gen).tolist() for n in (5, 70, 33, 16, 49, 2)]

    def serve(chunk):
        module = FakeModule()
        module.model = net
        engine = Engine(max_batch_size=3, model_module=module,
                        config=EngineConfig(batching="continuous", max_context=256, decode_burst=4,
                                            prefill_chunk=chunk))
        engine.max_tokens = 10
        for p in prompts:
            engine.add_request_ids(p)
        return engine.run()

    assert serve(16) == serve(None)
