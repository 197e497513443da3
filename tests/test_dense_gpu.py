"""The un-quantised fp16 model through the same fused step (the reference's second execution
path: a linear without a packed weight runs kernels/cuda/gemm.cu:36, src/model.py:35-41):
the dense GEMV chain (one or two rows), the tcgen05 fp16 GEMM (more rows, prefill) and loading an
unpacked checkpoint, against torch, the same-rounding oracle and HF fp16 (the recipe of the
reference's tests/test_parity.py:29-30,73-77: mean |dlogit| < 0.05, argmax equal)."""

import pytest
import torch

pytestmark = pytest.mark.gpu
RTOL, ATOL = 2e-2, 5e-2


@pytest.fixture(scope="module")
def dense_model():
    """2-layer, vocab-2048 dense model on the GPU, its same-rounding CPU oracle and its state."""
    from oracle.quic_ref import RefModel
    from quic_cu_b200 import model as qmodel
    from quic_cu_b200.checkpoint import qwen_config_dict, synthetic_dense_checkpoint

    state = synthetic_dense_checkpoint(n_layers=2, vocab=2048, seed=4321)
    config = qwen_config_dict(2, 2048)
    config.pop("quantization_config", None)
    net = qmodel.from_state_dict(state, config)
    assert net.dense
    torch.cuda.synchronize()
    return net, RefModel(state, 2), state, config


def _near_tie_ok(got, ref_tokens, ref_logits, near_tie=2e-2):
    for i, (g, r) in enumerate(zip(got, ref_tokens)):
        if g == r:
            continue
        top = torch.topk(ref_logits[i].float(), 2)
        assert (top.values[0] - top.values[1]).item() < near_tie and g in top.indices.tolist(), (i, g, r)
        return i
    return len(ref_tokens)


@pytest.mark.parametrize("n,k", [(1152, 896), (896, 896), (9728, 896), (896, 4864)])
@pytest.mark.parametrize("m", [1, 3, 16, 40, 200, 1500])
def test_dense_linear_matches_torch(m, n, k):
    """GEMV (one row), tcgen05 GEMM (more): fp32 accumulation, fp16 output, bias added in fp16."""
    from quic_cu_b200 import kernels as K

    g = torch.Generator(device="cuda").manual_seed(m * 31 + n + k)
    w = K.F16Weight(n, k, "cuda", bias=(torch.randn(n, device="cuda", generator=g) * 0.1).half() if n == 1152 else None)
    w.put((torch.randn(n, k, device="cuda", generator=g) * 0.02).half())
    x = torch.randn(m, k, device="cuda", generator=g).half()
    y = K.w4a16_linear(w, x)
    want = (x.float() @ w.w.float().t()).half().float()
    if w.bias is not None:
        want = (want + w.bias.float()).half().float()
    assert torch.allclose(y.float(), want, rtol=4e-3, atol=4e-3), (y.float() - want).abs().max()
    assert K.lib().quic_w4a16_tensor_status() == 0


@pytest.mark.parametrize("rows", [1, 2, 3, 4, 6, 20, 24])
def test_dense_decode_matches_oracle(dense_model, rows):
    """Prefill + greedy bursts: the chain of decode_layers_f16.cu up to 2 rows, the GEMM step
    beyond; tokens against the oracle row by row (up to a near-tie)."""
    net, ref, _, _ = dense_model
    gen = torch.Generator().manual_seed(rows)
    prompts = [torch.randint(0, 2048, (int(n),), generator=gen) for n in torch.randint(1, 40, (rows,), generator=gen)]
    cache = net.new_cache(n_slots=max(rows, 4), s_max=128)
    slots = list(range(rows))
    first, _ = net.prefill(cache, slots, prompts)
    rest = net.decode(cache, slots, 6)
    for i in range(rows):
        ref_tokens, ref_logits = ref.greedy(prompts[i].tolist(), 7)
        _near_tie_ok([int(first[i])] + rest[i], ref_tokens, ref_logits)


def test_dense_logits_token_by_token(dense_model):
    """forward() one token at a time (every step is the dense chain with logits kept)."""
    net, ref, _, _ = dense_model
    prompt = [3, 1500, 77, 9, 2047, 12]
    ref_tokens, ref_logits = ref.greedy(prompt, 5)
    cache = net.new_cache(n_slots=2, s_max=64)
    cache.batch_slots = [1]
    logits = None
    for t in prompt:
        logits = net(torch.tensor([[t]]), past_key_values=cache).logits
    got_tokens, got_logits = [], []
    for _ in range(5):
        got_logits.append(logits[0, 0].clone())
        nxt = logits[:, -1:, :].argmax(dim=-1)
        got_tokens.append(int(nxt))
        logits = net(nxt, past_key_values=cache).logits
    n = _near_tie_ok(got_tokens, ref_tokens, ref_logits)
    got, want = torch.stack(got_logits)[: n + 1].float().cpu(), ref_logits[: n + 1].float()
    assert torch.allclose(got, want, rtol=RTOL, atol=ATOL), (got - want).abs().max()


def test_dense_parity_with_hf_fp16(tmp_path):
    """A 4-layer un-quantised checkpoint written to disk in the reference's tensor names,
    loaded through model.load(), against HF fp16 (eager) on the CPU: mean |dlogit| < 0.05 on
    teacher-forced positions and equal greedy tokens over 100 steps (up to a near-tie)."""
    from oracle import hf_ref
    from quic_cu_b200 import model as qmodel
    from quic_cu_b200.checkpoint import qwen_config_dict, synthetic_dense_checkpoint, write_checkpoint_dir

    state = synthetic_dense_checkpoint(n_layers=4, vocab=2048, seed=99)
    config = qwen_config_dict(4, 2048)
    config.pop("quantization_config", None)
    write_checkpoint_dir(str(tmp_path), state, config)
    net, _ = qmodel.load(str(tmp_path), prefill_backend="quic")
    assert net.dense
    hf = hf_ref.build_hf_model(state, config, dtype=torch.float16)
    prompt = torch.randint(0, 2048, (1, 24), generator=torch.Generator().manual_seed(7))
    cache = net.new_cache(n_slots=2, s_max=256)
    first, _ = net.prefill(cache, [0], [prompt[0]])
    got = [int(first[0])] + net.decode(cache, [0], 64)[0] + net.decode(cache, [0], 35)[0]
    want_logits = hf_ref.teacher_forced_logits(hf, prompt, got)
    assert len(got) == 100
    want_tokens = want_logits.argmax(-1).tolist()
    for i, (g, w) in enumerate(zip(got, want_tokens)):  # teacher-forced: every position stands alone
        if g != w:
            top = torch.topk(want_logits[i].float(), 2)
            assert (top.values[0] - top.values[1]).item() < 5e-2 and g in top.indices.tolist(), (i, g, w)
    assert sum(g == w for g, w in zip(got, want_tokens)) >= 97

    cache = net.new_cache(n_slots=2, s_max=256)
    cache.batch_slots = [0]
    out = net(prompt, past_key_values=cache)
    ours = [out.logits[0, -1].float().cpu()]
    for t in got[:15]:
        ours.append(net(torch.tensor([[t]]), past_key_values=cache).logits[0, 0].float().cpu())
    delta = (torch.stack(ours) - want_logits[:16].float()).abs()
    assert delta.mean().item() < 0.05, delta.mean().item()
