"""The tcgen05 paths: W4A16 GEMM (2 rows and more), tensor lm_head and the batched decode step."""

import pytest
import torch

from oracle import quic_ref

pytestmark = pytest.mark.gpu
SHAPES = {"qkv": (896, 1152), "o_proj": (896, 896), "gate_up": (896, 9728), "down": (4864, 896)}  # K x N


def _near_tie_ok(got, ref_tokens, ref_logits, near_tie=2e-2):
    for i, (g, r) in enumerate(zip(got, ref_tokens)):
        if g != r:
            top = torch.topk(ref_logits[i].float(), 2)
            assert (top.values[0] - top.values[1]).item() < near_tie and g in top.indices.tolist(), (i, g, r)
            return


@pytest.mark.parametrize("name", list(SHAPES))
def test_tensor_gemm_matches_gemv_and_oracle(name):
    from quic_cu_b200 import kernels as K
    from quic_cu_b200.checkpoint import synthetic_layer

    k, n = SHAPES[name]
    layer = synthetic_layer(n, k, torch.Generator().manual_seed(21))
    w = K.W4Weight(n, k, "cuda")
    w.put(layer["weight_packed"], layer["weight_scale"], layer["weight_zero_point"])
    w.bias = (torch.randn(n, generator=torch.Generator().manual_seed(1)) * 0.02).half().cuda()
    w16 = torch.from_numpy(quic_ref.dequantize_f16(layer["weight_packed"].numpy(), layer["weight_scale"].numpy(),
                                                   layer["weight_zero_point"].numpy()))
    # (from 2049 / 2689 rows every shape gives a CTA two row tiles; 2600 and 3000 end in a CTA
    # with one partly filled tile and with a full and a partly filled one)
    for m in (2, 3, 4, 5, 16, 17, 64, 100, 256, 300, 1000, 2500, 2600, 3000):
        x = torch.randn(m, k, generator=torch.Generator().manual_seed(m)).half()
        y_tc = K.w4a16_linear(w, x.cuda(), use_tensor=True)
        y_gemv = K.w4a16_linear(w, x.cuda(), use_tensor=False)
        want = quic_ref.w4a16_linear(x, w16, w.bias.cpu())
        assert torch.allclose(y_tc.cpu().float(), want.float(), rtol=2e-3, atol=2e-2)
        # same fp16 weights, fp32 accumulation in both kernels: at most one fp16 ulp apart
        assert torch.allclose(y_tc.float(), y_gemv.float(), rtol=2e-3, atol=2e-2)
    torch.cuda.synchronize()
    assert K.lib().quic_w4a16_tensor_status() == 0


@pytest.mark.parametrize("batch", [2, 4, 9, 12, 16, 17, 40])
def test_batched_decode_step_matches_oracle(tiny_model, batch):
    """2..15 rows run the layer chain on mma.sync (rows on the M side), 16 and more the tcgen05
    step; every row must still give what the oracle gives for that request alone."""
    from quic_cu_b200 import kernels as K

    net, ref, _, _ = tiny_model
    gen = torch.Generator().manual_seed(batch)
    lens = torch.randint(1, 40, (batch,), generator=gen).tolist()
    prompts = [torch.randint(0, 2048, (n,), generator=gen) for n in lens]
    cache = net.new_cache(n_slots=64, s_max=128)
    slots = list(range(batch, 0, -1))  # rows need not sit in slot order
    first, _ = net.prefill(cache, slots, prompts)
    rest = net.decode(cache, slots, 4)
    for i in range(0, batch, max(1, batch // 6)):
        ref_tokens, ref_logits = ref.greedy(prompts[i].tolist(), 5)
        _near_tie_ok([int(first[i])] + rest[i], ref_tokens, ref_logits)
    assert K.lib().quic_w4a16_tensor_status() == 0


@pytest.mark.parametrize("batch", [2, 3, 4, 5, 8, 11, 16])
def test_the_three_decode_steps_agree_with_oracle(tiny_model, batch):
    """The same rows through the five-kernel layer chain on mma.sync (forced from 2 rows), through
    the GEMV chain (where it takes the batch: up to 4 rows) and through the tcgen05 step (forced
    from 2 rows): each must match the oracle row by row."""
    from quic_cu_b200 import kernels as K

    net, ref, _, _ = tiny_model
    gen = torch.Generator().manual_seed(100 + batch)
    prompts = [torch.randint(0, 2048, (int(n),), generator=gen) for n in torch.randint(1, 30, (batch,), generator=gen)]
    want = [ref.greedy(p.tolist(), 5) for p in prompts]
    paths = [(17, 2), (2, 17)] + ([(17, 17)] if batch <= 4 else [])  # (tensor from, mma.sync chain from)
    try:
        for tensor_from, mma_from in paths:
            K.lib().quic_set_tensor_min_batch(tensor_from)
            K.lib().quic_set_mma_chain_min_batch(mma_from)
            cache = net.new_cache(n_slots=16, s_max=128)  # new cache: graphs are captured per setting
            slots = list(range(batch))
            first, _ = net.prefill(cache, slots, prompts)
            rest = net.decode(cache, slots, 4)
            for i in range(batch):
                _near_tie_ok([int(first[i])] + rest[i], want[i][0], want[i][1])
    finally:
        K.lib().quic_set_tensor_min_batch(16)
        K.lib().quic_set_mma_chain_min_batch(3)
    assert K.lib().quic_w4a16_tensor_status() == 0


@pytest.mark.parametrize("threshold", [17, 2])
def test_batched_forward_logits_match_oracle(tiny_model, threshold):
    """Logits of a 12-row decode step (tensor lm_head; layers on the mma.sync chain or, forced,
    on the tcgen05 step) against the oracle's per-row logits."""
    from quic_cu_b200 import kernels as K

    net, ref, _, _ = tiny_model
    K.lib().quic_set_tensor_min_batch(threshold)
    gen = torch.Generator().manual_seed(77)
    prompts = [torch.randint(0, 2048, (int(n),), generator=gen).tolist() for n in range(3, 15)]
    width = max(len(p) for p in prompts)
    ids = torch.zeros(len(prompts), width, dtype=torch.long)
    mask = torch.zeros(len(prompts), width, dtype=torch.long)
    for i, p in enumerate(prompts):
        ids[i, width - len(p):] = torch.tensor(p)
        mask[i, width - len(p):] = 1
    out = net(ids, attention_mask=mask)
    nxt = out.logits[:, -1:, :].argmax(-1)
    step = net(nxt, past_key_values=out.past_key_values)
    assert step.logits.shape == (12, 1, 2048)
    for i in (0, 5, 11):
        ref_tokens, ref_logits = ref.greedy(prompts[i], 2)
        if int(nxt[i]) != ref_tokens[0]:
            continue  # near tie on the first token: the second step saw another input
        got = step.logits[i, 0].float().cpu()
        try:
            assert torch.allclose(got, ref_logits[1].float(), rtol=2e-2, atol=5e-2), (got - ref_logits[1].float()).abs().max()
        finally:
            K.lib().quic_set_tensor_min_batch(16)


def test_a_gemm_wait_that_runs_out_is_reported_and_the_next_call_works(tiny_model):
    """The bounded waits of the tcgen05 GEMM: with the probe limit lowered and one packed weight
    tile never requested (the library's test hook), the consumer warps' wait for that tile runs
    out, the MMA warp's and the epilogue's waits follow, every role leaves its loop, the CTA
    releases its tensor memory and returns; the status word names the wait.  Nothing faults.
    Then, with the hook cleared: the same call is correct, and a decode burst whose graph was
    captured under the hook raises from decode() and a fresh one works."""
    from quic_cu_b200 import kernels as K

    net, ref, _, _ = tiny_model
    lib = K.lib()
    L = net.layers[0]
    x = torch.randn(64, 896, device="cuda", dtype=torch.float16, generator=torch.Generator(device="cuda").manual_seed(1))
    want = K.w4a16_linear(L["qkv"], x, use_tensor=1).clone()
    assert lib.quic_w4a16_tensor_status() == 0
    try:
        lib.quic_w4a16_tensor_test_hook(20000, 0)
        K.w4a16_linear(L["qkv"], x, use_tensor=1)
        code = lib.quic_w4a16_tensor_status()
        assert code != 0 and (code >> 16) in (1, 2, 3), hex(code)
        assert lib.quic_w4a16_tensor_status() == 0          # the word was taken
        lib.quic_w4a16_tensor_test_hook(0, -1)
        assert torch.equal(K.w4a16_linear(L["qkv"], x, use_tensor=1), want)
        assert lib.quic_w4a16_tensor_status() == 0

        # decode(): the graph of a 20-row burst captured under the hook carries it
        gen = torch.Generator().manual_seed(5)
        prompts = [torch.randint(0, 2048, (6,), generator=gen) for _ in range(20)]
        slots = list(range(20))
        cache = net.new_cache(n_slots=20, s_max=64)
        net.prefill(cache, slots, prompts)
        lib.quic_w4a16_tensor_test_hook(20000, 0)
        try:
            with pytest.raises(RuntimeError, match="bounded wait"):
                net.decode(cache, slots, 2)
        finally:
            lib.quic_w4a16_tensor_test_hook(0, -1)
        assert lib.quic_w4a16_tensor_status() == 0          # decode() took the word
        cache = net.new_cache(n_slots=20, s_max=64)
        first, _ = net.prefill(cache, slots, prompts)
        rest = net.decode(cache, slots, 3)
        for i in (0, 7, 19):
            ref_tokens, ref_logits = ref.greedy(prompts[i].tolist(), 4)
            _near_tie_ok([int(first[i])] + rest[i], ref_tokens, ref_logits)
    finally:
        lib.quic_w4a16_tensor_test_hook(0, -1)
    assert lib.quic_w4a16_tensor_status() == 0


def test_a_streamed_attention_wait_that_runs_out_is_reported_and_the_next_call_works(tiny_model):
    """The bounded waits of the streamed decode attention: under the library's test hook the first
    tile of every row is never requested and the waits probe 20000 times at most; the consumer
    warp's wait runs out, the producer's wait for that stage follows, the CTA reports and returns.
    decode() raises; with the hook cleared a fresh cache decodes what the oracle gives."""
    from quic_cu_b200 import kernels as K

    net, ref, _, _ = tiny_model
    lib = K.lib()
    gen = torch.Generator().manual_seed(6)
    prompts = [torch.randint(0, 2048, (70 + i,), generator=gen) for i in range(24)]
    slots = list(range(24))
    assert lib.quic_w4a16_tensor_status() == 0
    cache = net.new_cache(n_slots=24, s_max=128)
    net.prefill(cache, slots, prompts)
    lib.quic_attn_stream_test_hook(2)
    try:
        with pytest.raises(RuntimeError, match="bounded wait"):
            net.decode(cache, slots, 2)
    finally:
        lib.quic_attn_stream_test_hook(0)
    assert lib.quic_w4a16_tensor_status() == 0          # decode() took the word
    cache = net.new_cache(n_slots=24, s_max=128)
    first, _ = net.prefill(cache, slots, prompts)
    rest = net.decode(cache, slots, 3)
    for i in (0, 11, 23):
        ref_tokens, ref_logits = ref.greedy(prompts[i].tolist(), 4)
        _near_tie_ok([int(first[i])] + rest[i], ref_tokens, ref_logits)
    assert lib.quic_w4a16_tensor_status() == 0


@pytest.mark.parametrize("rows", [1, 3, 8, 16, 20, 40])
def test_decode_gives_the_same_bits_every_run(tiny_model, rows):
    """Cross-CTA hand-offs (arrival counters, cluster merges, split-K planes) must not make the
    result depend on timing: the same prompts decoded from scratch five times leave bit-identical
    tokens and bit-identical KV slots, on every form of the step."""
    net = tiny_model[0]
    gen = torch.Generator().manual_seed(500 + rows)
    prompts = [torch.randint(0, 2048, (int(n),), generator=gen) for n in torch.randint(1, 700, (rows,), generator=gen)]
    slots = list(range(rows))
    want_tokens = want_kv = None
    for _ in range(5):
        cache = net.new_cache(n_slots=rows, s_max=768)
        first, _ = net.prefill(cache, slots, prompts)
        tokens = (first.tolist(), net.decode(cache, slots, 12))
        torch.cuda.synchronize()
        if want_tokens is None:
            want_tokens, want_kv = tokens, cache.kv.clone()
        else:
            assert tokens == want_tokens
            assert torch.equal(cache.kv, want_kv)
