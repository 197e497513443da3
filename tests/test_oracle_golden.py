"""Pins the CPU oracle to outputs of the reference's own Python (tests/golden/)."""

import json
import os
from collections import deque

import numpy as np
import torch

from oracle import hf_ref, quic_ref
from quic_cu_b200.checkpoint import (detect_group_size, pack_layer, packed_prefixes, qwen_config_dict,
                                     synthetic_checkpoint)
from quic_cu_b200.scheduler import ContinuousAdmissionPolicy, StaticAdmissionPolicy
from quic_cu_b200.sequence import SequenceState

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def test_dequantize_matches_reference_bit_for_bit():
    for tag in ("a", "b"):
        g = np.load(os.path.join(GOLDEN, f"dequant_{tag}.npz"))
        got = quic_ref.dequantize(g["weight_packed"], g["weight_scale"], g["weight_zero_point"])
        assert got.dtype == np.float32
        assert np.array_equal(got.view(np.uint32), g["reference"].view(np.uint32))


def test_pack_layer_round_trips_through_the_oracle_unpack():
    gen = torch.Generator().manual_seed(0)
    q = torch.randint(0, 16, (64, 256), generator=gen)
    zp = torch.randint(0, 16, (64, 2), generator=gen)
    packed, zpacked = pack_layer(q, zp)
    assert packed.dtype == torch.int32 and packed.shape == (64, 32) and zpacked.shape == (8, 2)
    assert np.array_equal(quic_ref.unpack_q(packed.numpy()), q.numpy().astype(np.uint8))
    assert np.array_equal(quic_ref.unpack_zp(zpacked.numpy(), 64), zp.numpy().astype(np.uint8))
    # extreme nibbles exercise the sign bit of the int32 words
    q15 = torch.full((8, 8), 15)
    packed15, _ = pack_layer(q15, torch.zeros(8, 1, dtype=torch.long))
    assert (packed15 == -1).all()
    assert np.array_equal(quic_ref.unpack_q(packed15.numpy()), np.full((8, 8), 15, np.uint8))


def test_scheduler_matches_reference_decisions():
    with open(os.path.join(GOLDEN, "scheduler.json")) as handle:
        cases = json.load(handle)
    assert len(cases) == 40
    for case in cases:
        for name, policy in (("static", StaticAdmissionPolicy()), ("continuous", ContinuousAdmissionPolicy())):
            running = []
            for d in case["running"]:
                s = SequenceState(prompt_tokens=torch.tensor([[1]]), request_id=d["id"], max_tokens=d["max_tokens"])
                s.generated_tokens = [9] * d["generated"]
                if d["eos"] and d["generated"] > 0:
                    s.finished_at = d["generated"] - 1
                running.append(s)
            waiting = deque(SequenceState(prompt_tokens=torch.tensor([[2]]), request_id=w, max_tokens=4)
                            for w in case["waiting"])
            dec = policy.decide(running, waiting, case["max_batch"])
            assert [s.request_id for s in dec.release] == case[name]["release"], (name, case)
            assert [s.request_id for s in dec.admit] == case[name]["admit"], (name, case)


def test_oracle_paths_match_reference_hf_quant_logits():
    """Both restatements — the op-by-op pipeline and the HF wrapper — reproduce the logits the
    reference's model_hf.load produced for the seeded 2-layer checkpoint."""
    g = np.load(os.path.join(GOLDEN, "hf_quant_logits.npz"))
    spec = json.loads(str(g["model"]))
    state = synthetic_checkpoint(**spec)
    prompt, tokens = g["prompt"].tolist(), g["tokens"].tolist()
    want = torch.from_numpy(g["logits"]).float()

    ref_tokens, ref_logits = quic_ref.RefModel(state, spec["n_layers"]).greedy(prompt, len(tokens))
    assert ref_tokens == tokens
    assert torch.allclose(ref_logits.float(), want, rtol=2e-2, atol=5e-2)
    assert (ref_logits.float() - want).abs().max() < 2e-2

    hf = hf_ref.build_hf_model(state, qwen_config_dict(spec["n_layers"], spec["vocab"]), dtype=torch.float32)
    hf_tokens, hf_logits = hf_ref.greedy_with_logits(hf, torch.tensor([prompt]), len(tokens))
    assert hf_tokens == tokens
    assert (hf_logits - want).abs().max() < 2e-2
    forced = hf_ref.teacher_forced_logits(hf, torch.tensor([prompt]), tokens)
    assert torch.allclose(forced, hf_logits, atol=1e-4)


def test_oracle_float_ops_follow_the_reference_test_recipes():
    torch.manual_seed(0)
    x = torch.randn(8, 896).half()
    w = torch.ones(896).half()
    variance = x.float().pow(2).mean(-1, keepdim=True)  # reference tests/test_kernels.py:19-20
    assert torch.equal(quic_ref.rmsnorm(x, w), (x.float() * torch.rsqrt(variance + 1e-6) * w.float()).half())
    gate, up = torch.randn(4, 4864).half(), torch.randn(4, 4864).half()
    want = (torch.nn.functional.silu(gate.float()) * up.float()).half()  # tests/test_kernels.py:33
    assert torch.allclose(quic_ref.swiglu(gate, up).float(), want.float(), atol=1e-2)
    # decode attention recipe, tests/test_attention.py:70-78
    q, k, v = torch.randn(4, 14, 64).half(), torch.randn(4, 2, 16, 64).half(), torch.randn(4, 2, 16, 64).half()
    pads = torch.tensor([0, 2, 4, 15])
    pos = torch.arange(16)
    mask = (pos[None, :] >= pads[:, None])[:, None, None, :].expand(4, 14, 1, 16)
    want = torch.nn.functional.scaled_dot_product_attention(
        q[:, :, None].float(), k.repeat_interleave(7, 1).float(), v.repeat_interleave(7, 1).float(),
        attn_mask=mask, scale=0.125)[:, :, 0]
    got = quic_ref.attn_decode(q, k, v, 0.125, start=pads)
    assert torch.allclose(got.float(), want, atol=1e-2)
    assert torch.count_nonzero(quic_ref.attn_decode(q, k, v, 0.125, start=torch.full((4,), 16))) == 0
    assert quic_ref.argmax_lowest(torch.tensor([[1.0, 3.0, 3.0, 2.0]])).tolist() == [1]


def test_checkpoint_helpers():
    state = synthetic_checkpoint(n_layers=1, vocab=64, seed=0)
    assert len(packed_prefixes(state)) == 7
    assert detect_group_size(qwen_config_dict(1, 64)) == 128
    assert detect_group_size({"quantization_config": {"group_size": 64}}) == 64
    assert detect_group_size({}) == 32
    again = synthetic_checkpoint(n_layers=1, vocab=64, seed=0)
    assert all(torch.equal(state[k], again[k]) for k in state)
