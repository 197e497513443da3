"""GPU parity of the fused decode step against the CPU oracle and the reference's
dequantised-weight Hugging Face path."""

import json
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
# tolerance of the acceptance gate: logits within rtol 2e-2 / atol 5e-2 per step
RTOL, ATOL = 2e-2, 5e-2


def _close(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return bool(((a - b).abs() <= ATOL + RTOL * b.abs()).all()), (a - b).abs().max().item()


def _assert_greedy_matches(got_tokens, ref_tokens, ref_logits, near_tie=2e-2):
    """Greedy sequences must agree up to the first position where the oracle's own top-2
    margin is below ``near_tie`` (numerical noise may then pick the runner-up, after which
    the two sequences legitimately differ)."""
    for i, (g, r) in enumerate(zip(got_tokens, ref_tokens)):
        if g == r:
            continue
        top = torch.topk(ref_logits[i].float(), 2)
        gap = (top.values[0] - top.values[1]).item()
        assert gap < near_tie and g in top.indices.tolist(), (i, g, r, gap)
        return i
    return len(ref_tokens)


def test_token_by_token_matches_oracle(tiny_model):
    """Prompt and generation both through the fused decode step (positions 0..n)."""
    net, ref, _, _ = tiny_model
    prompt = [11, 7, 1999, 42, 0, 512, 77, 1023]
    ref_tokens, ref_logits = ref.greedy(prompt, 6)
    cache = net.new_cache(n_slots=4, s_max=256)
    cache.batch_slots = [2]
    logits = None
    for t in prompt:
        logits = net(torch.tensor([[t]]), past_key_values=cache).logits
    got_tokens, got_logits = [], []
    for _ in range(6):
        got_logits.append(logits[0, 0].clone())
        nxt = logits[:, -1:, :].argmax(dim=-1)
        got_tokens.append(int(nxt))
        logits = net(nxt, past_key_values=cache).logits
    n = _assert_greedy_matches(got_tokens, ref_tokens, ref_logits)
    ok, err = _close(torch.stack(got_logits)[: n + 1], ref_logits[: n + 1])
    assert ok, err


def test_prefill_then_graph_decode_matches_oracle(tiny_model):
    net, ref, _, _ = tiny_model
    prompt = [3, 1, 4, 1, 5, 9, 2, 6, 5, 3, 5, 8, 9, 7, 9]
    ref_tokens, ref_logits = ref.greedy(prompt, 9)
    cache = net.new_cache(n_slots=4, s_max=256)
    first, logits = net.prefill(cache, [3], [torch.tensor(prompt)])
    ok, err = _close(logits[0], ref_logits[0])
    assert ok, err
    tokens = [int(first[0])] + net.decode(cache, [3], 8)[0]
    _assert_greedy_matches(tokens, ref_tokens, ref_logits)
    # the same decode as eight single-step launches gives the same tokens bit for bit
    cache2 = net.new_cache(n_slots=4, s_max=256)
    first2, _ = net.prefill(cache2, [1], [torch.tensor(prompt)])
    again = [int(first2[0])] + [net.decode(cache2, [1], 1)[0][0] for _ in range(8)]
    assert again == tokens


def test_prefill_with_the_library_attention_kernel_matches_oracle(tiny_model):
    """Heads split + RoPE + KV write and causal attention by the library's kernels for three
    ragged prompts at once; last-position logits and the greedy continuation must follow the
    oracle."""
    net, ref, _, _ = tiny_model
    gen = torch.Generator().manual_seed(21)
    prompts = [torch.randint(0, 2048, (n,), generator=gen) for n in (70, 1, 33)]
    want = [ref.greedy(p.tolist(), 5) for p in prompts]
    cache = net.new_cache(n_slots=4, s_max=128)
    first, logits = net.prefill(cache, [2, 0, 3], prompts)
    for i in range(3):
        ok, err = _close(logits[i], want[i][1][0])
        assert ok, (i, err)
    rest = net.decode(cache, [2, 0, 3], 4)
    for i in range(3):
        _assert_greedy_matches([int(first[i])] + rest[i], want[i][0], want[i][1])


def test_prefill_of_several_hundred_rows_matches_oracle(tiny_model):
    """415 rows in one prefill: from 129 rows on the gate|up GEMM gives a CTA two row tiles and puts
    its SwiGLU output together in shared memory (here: one full CTA and one whose second tile is
    partly filled); the logits of every prompt's last position must follow the oracle."""
    net, ref, _, _ = tiny_model
    gen = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, 2048, (n,), generator=gen) for n in (260, 150, 5)]
    want = [ref.greedy(p.tolist(), 1) for p in prompts]
    cache = net.new_cache(n_slots=4, s_max=320)
    first, logits = net.prefill(cache, [1, 3, 0], prompts)
    for i in range(3):
        ok, err = _close(logits[i], want[i][1][0])
        assert ok, (i, err)
        _assert_greedy_matches([int(first[i])], want[i][0], want[i][1])


def test_the_graph_cache_is_bounded_and_rebuilds(tiny_model):
    """A cache keeps at most ``max_graphs`` captured graphs; when another one is needed all are
    destroyed (with their launch plans and scratch arenas) and decoding goes on, same tokens."""
    net, _, _, _ = tiny_model
    prompt = torch.tensor([5, 6, 7, 8, 9, 10, 11])
    want_cache = net.new_cache(n_slots=2, s_max=128)
    first, _ = net.prefill(want_cache, [0], [prompt])
    want = [int(first[0])] + net.decode(want_cache, [0], 12)[0]

    cache = net.new_cache(n_slots=2, s_max=128)
    cache.max_graphs = 2
    first, _ = net.prefill(cache, [0], [prompt])
    got = [int(first[0])]
    for steps in (1, 2, 3, 1, 2, 3):  # three graph shapes through two places, twice
        got += net.decode(cache, [0], steps)[0]
        assert len(cache._graphs) <= 2
    assert got == want


def test_prefill_beyond_8192_rows_goes_out_in_one_launch_per_linear(tiny_model):
    """Five prompts of 2000 tokens are 10000 rows: beyond 8192 rows a packed linear covers all rows in
    one launch (no K split at that size, so no workspace).  The same prompts prefilled as 6000 and
    4000 rows must leave the same first tokens, the same logits and the same cache."""
    net, _, _, _ = tiny_model
    gen = torch.Generator().manual_seed(81)
    prompts = [torch.randint(0, 2048, (2000,), generator=gen) for _ in range(5)]
    whole = net.new_cache(n_slots=5, s_max=2048)
    first, logits = net.prefill(whole, [0, 1, 2, 3, 4], prompts)
    parts = net.new_cache(n_slots=5, s_max=2048)
    first_a, logits_a = net.prefill(parts, [0, 1, 2], prompts[:3])
    first_b, logits_b = net.prefill(parts, [3, 4], prompts[3:])
    assert first.tolist() == first_a.tolist() + first_b.tolist()
    assert torch.equal(logits, torch.cat([logits_a, logits_b]))
    assert torch.equal(whole.kv[:, :, :, :, :2000], parts.kv[:, :, :, :, :2000])


def test_bursts_single_steps_and_host_fed_steps_agree(tiny_model):
    """150 tokens three ways: graph bursts of 64 steps (the ring of generated tokens wraps),
    single-step calls, and single-step calls that feed the previous token back from pinned
    host memory.  Bit-identical tokens: the kernels read cache rows written one step earlier
    ahead of their dependency wait, and with a two-layer model consecutive steps sit only a
    few kernels apart."""
    net, _, _, _ = tiny_model
    prompt = torch.tensor([17, 4, 256, 1000, 31, 8, 8, 1203, 77])
    n = 150

    cache = net.new_cache(n_slots=2, s_max=256)
    first, _ = net.prefill(cache, [1], [prompt])
    bursts, left = [int(first[0])], n
    while left:
        k = min(64, left)
        bursts += net.decode(cache, [1], k)[0]
        left -= k

    cache = net.new_cache(n_slots=2, s_max=256)
    first, _ = net.prefill(cache, [0], [prompt])
    singles = [int(first[0])] + [net.decode(cache, [0], 1)[0][0] for _ in range(n)]

    cache = net.new_cache(n_slots=2, s_max=256)
    first, _ = net.prefill(cache, [1], [prompt])
    pinned = torch.zeros(1, dtype=torch.int32).pin_memory()
    fed = [int(first[0])]
    for _ in range(n):
        pinned[0] = fed[-1]
        fed.append(net.decode(cache, [1], 1, feed=pinned)[0][0])

    assert singles == bursts
    assert fed == bursts
    with pytest.raises(ValueError):
        net.decode(cache, [1], 1, feed=torch.zeros(2, dtype=torch.int32))


def test_many_distinct_row_orders_keep_graphs_valid(tiny_model):
    """300 decode calls, each with a different ordered triple of slots (more row->slot maps
    than the cache keeps), all replaying the one graph captured for three rows.  The buffer
    that graph reads must survive the eviction of cached maps, and every slot's tokens must
    still follow the oracle (up to the first near-tie, where sequences may part)."""
    import itertools

    net, ref, _, _ = tiny_model
    gen = torch.Generator().manual_seed(9)
    prompts = [torch.randint(0, 2048, (int(n),), generator=gen) for n in range(3, 11)]
    cache = net.new_cache(n_slots=8, s_max=256)
    first, _ = net.prefill(cache, list(range(8)), prompts)
    got = [[int(first[i])] for i in range(8)]
    address = None
    for triple in itertools.islice(itertools.permutations(range(8), 3), 300):
        out = net.decode(cache, list(triple), 1)
        if address is None:
            address = cache._row_bufs[3].data_ptr()
        for slot, toks in zip(triple, out):
            got[slot] += toks
    assert cache._row_bufs[3].data_ptr() == address
    assert len(cache._rows) <= 257
    agreed = 0
    for slot in range(8):
        ref_tokens, ref_logits = ref.greedy(prompts[slot].tolist(), len(got[slot]))
        agreed += _assert_greedy_matches(got[slot], ref_tokens, ref_logits)
    assert agreed > 4 * 100  # most rows follow the oracle through the whole schedule


def test_batched_rows_are_independent(tiny_model):
    """Rows of different lengths in one batch give what each gives alone (left-padding
    semantics of the reference's batch: padded keys never contribute)."""
    net, ref, _, _ = tiny_model
    prompts = [[5, 6, 7], [100, 200, 300, 400, 500, 600, 700], [9], [1, 2], [42] * 12]
    want = [ref.greedy(p, 5) for p in prompts]
    cache = net.new_cache(n_slots=8, s_max=128)
    slots = [6, 0, 3, 7, 1]
    first, _ = net.prefill(cache, slots, [torch.tensor(p) for p in prompts])
    rest = net.decode(cache, slots, 4)
    for i in range(len(prompts)):
        _assert_greedy_matches([int(first[i])] + rest[i], want[i][0], want[i][1])


@pytest.mark.parametrize("prompt_len,steps", [(1100, 5), (2043, 9)])
def test_single_row_decode_beyond_1024_tokens(tiny_model, prompt_len, steps):
    """One row at 1025..2048 tokens of context runs the single-warp attention kernel with 17..32
    splits, which the o_proj kernel merges in two passes of loads; the second case also crosses
    2048 tokens, where the throughput kernel takes over."""
    net, ref, _, _ = tiny_model
    prompt = torch.randint(0, 2048, (prompt_len,), generator=torch.Generator().manual_seed(prompt_len)).tolist()
    ref_tokens, ref_logits = ref.greedy(prompt, steps)
    cache = net.new_cache(n_slots=2, s_max=2304)
    cache.batch_slots = [1]
    out = net(torch.tensor([prompt]), past_key_values=cache)
    tokens, kept = [], []
    for _ in range(steps):
        kept.append(out.logits[0, -1].clone())
        nxt = kept[-1].argmax().view(1, 1)
        tokens.append(int(nxt))
        out = net(nxt, past_key_values=cache)
    n = _assert_greedy_matches(tokens, ref_tokens, ref_logits)
    ok, err = _close(torch.stack(kept)[: n + 1], ref_logits[: n + 1])
    assert ok, err
    # the same tokens from one graph of several steps
    cache2 = net.new_cache(n_slots=2, s_max=2304)
    first, _ = net.prefill(cache2, [0], [torch.tensor(prompt)])
    again = [int(first[0])] + net.decode(cache2, [0], steps - 1)[0]
    assert again == tokens


def test_single_row_long_context_matches_the_batched_step(tiny_model):
    """Beyond 2048 tokens one row runs the throughput attention kernel with up to 64 splits that
    the o_proj kernel merges in passes of 16; four rows run the tensor-core step, whose splits
    the last CTA merges.  Same prompt, same fed tokens: the logits of the two must agree."""
    net, _, _, _ = tiny_model
    gen = torch.Generator().manual_seed(77)
    prompt = torch.randint(0, 2048, (4300,), generator=gen)
    others = [torch.randint(0, 2048, (n,), generator=gen) for n in (40, 700, 3000)]
    steps = 5

    one = net.new_cache(n_slots=1, s_max=8192)
    first, _ = net.prefill(one, [0], [prompt])
    one.batch_slots = [0]
    fed, single = [int(first[0])], []
    for _ in range(steps):
        logits = net(torch.tensor([[fed[-1]]]), past_key_values=one).logits[0, 0].clone()
        single.append(logits)
        fed.append(int(logits.argmax()))

    four = net.new_cache(n_slots=4, s_max=8192)
    firsts, _ = net.prefill(four, [2, 0, 1, 3], [prompt] + others)
    assert int(firsts[0]) == fed[0]
    four.batch_slots = [2, 0, 1, 3]
    nxt = firsts.view(4, 1).clone()
    for i in range(steps):
        nxt[0, 0] = fed[i]
        logits = net(nxt, past_key_values=four).logits[:, 0]
        ok, err = _close(logits[0], single[i])
        assert ok, (i, err)
        nxt = logits.argmax(dim=-1, keepdim=True)


@pytest.mark.parametrize("repeat_early_requests", [False, True])
def test_many_ragged_rows_streamed_attention_matches_the_small_batch_chain(tiny_model, repeat_early_requests):
    """24 rows of 5..1900 tokens in one tensor-core step: from 21 rows on, up to 2048 tokens of
    context, a CTA per (row, KV head) streams the row's cache through an eight-stage ring (rows
    beyond 512 tokens wrap it, the longest four times) and four warps keep running softmaxes.
    The same rows as two batches of 12 run the mma.sync chain with the cluster attention; fed the
    same tokens, the logits of the two must agree.  Second form: the kernel repeats the tile requests
    it made before the dependency wait (its path for a step counter that moved meanwhile)."""
    from quic_cu_b200 import kernels as K

    net, _, _, _ = tiny_model
    gen = torch.Generator().manual_seed(79)
    lens = [5, 63, 64, 65, 127, 128, 129, 300, 511, 512, 513, 700, 1023, 1024, 1025, 1300, 1536, 1700, 1900, 1, 2,
            450, 900, 33]
    prompts = [torch.randint(0, 2048, (n,), generator=gen) for n in lens]
    steps = 3

    halves = net.new_cache(n_slots=24, s_max=2048)
    firsts, _ = net.prefill(halves, list(range(24)), prompts)
    fed, chain = [firsts.view(24, 1).clone()], []
    for _ in range(steps):
        rows = []
        for lo in (0, 12):
            halves.batch_slots = list(range(lo, lo + 12))
            rows.append(net(fed[-1][lo:lo + 12], past_key_values=halves).logits[:, 0].clone())
        chain.append(torch.cat(rows))
        fed.append(chain[-1].argmax(dim=-1, keepdim=True))

    whole = net.new_cache(n_slots=24, s_max=2048)
    firsts24, _ = net.prefill(whole, list(range(24)), prompts)
    assert firsts24.tolist() == firsts.tolist()
    whole.batch_slots = list(range(24))
    K.lib().quic_attn_stream_test_hook(int(repeat_early_requests))
    try:
        for i in range(steps):
            logits = net(fed[i], past_key_values=whole).logits[:, 0]
            ok, err = _close(logits, chain[i])
            assert ok, (i, err)
        torch.cuda.synchronize()
    finally:
        K.lib().quic_attn_stream_test_hook(0)
    assert K.lib().quic_w4a16_tensor_status() == 0


def test_many_rows_beyond_2048_tokens_streamed_attention_matches_the_split_kernel(tiny_model):
    """22 rows, one of 4300 tokens: the streamed attention walks 68 tiles of that row through its
    twelve-stage ring.  The same rows as two batches of 11 run the mma.sync chain, whose attention
    beyond 4096 tokens is the split kernel; fed the same tokens, the logits must agree."""
    net, _, _, _ = tiny_model
    gen = torch.Generator().manual_seed(80)
    lens = [4300, 2049, 2048, 3000] + [17 * (i + 1) for i in range(18)]
    prompts = [torch.randint(0, 2048, (n,), generator=gen) for n in lens]
    halves = net.new_cache(n_slots=22, s_max=4608)
    firsts, _ = net.prefill(halves, list(range(22)), prompts)
    fed, chain = [firsts.view(22, 1).clone()], []
    for _ in range(2):
        rows = []
        for lo in (0, 11):
            halves.batch_slots = list(range(lo, lo + 11))
            rows.append(net(fed[-1][lo:lo + 11], past_key_values=halves).logits[:, 0].clone())
        chain.append(torch.cat(rows))
        fed.append(chain[-1].argmax(dim=-1, keepdim=True))
    whole = net.new_cache(n_slots=22, s_max=4608)
    firsts22, _ = net.prefill(whole, list(range(22)), prompts)
    assert firsts22.tolist() == firsts.tolist()
    whole.batch_slots = list(range(22))
    for i in range(2):
        logits = net(fed[i], past_key_values=whole).logits[:, 0]
        ok, err = _close(logits, chain[i])
        assert ok, (i, err)


def test_three_ragged_rows_long_context_match_the_batched_step(tiny_model):
    """Three rows of 4300 / 40 / 2500 tokens on the GEMV chain (3-row kernels, throughput
    attention kernel, splits without tokens for the short rows, o_proj merging 64 splits)
    against the same rows inside a 4-row tensor-core step, fed the same tokens."""
    net, _, _, _ = tiny_model
    gen = torch.Generator().manual_seed(78)
    prompts = [torch.randint(0, 2048, (n,), generator=gen) for n in (4300, 40, 2500, 900)]
    steps = 4

    three = net.new_cache(n_slots=4, s_max=8192)
    firsts, _ = net.prefill(three, [3, 1, 0], prompts[:3])
    three.batch_slots = [3, 1, 0]
    nxt = firsts.view(3, 1).clone()
    fed, chain = [nxt.clone()], []
    for _ in range(steps):
        logits = net(nxt, past_key_values=three).logits[:, 0].clone()
        chain.append(logits)
        nxt = logits.argmax(dim=-1, keepdim=True)
        fed.append(nxt.clone())

    four = net.new_cache(n_slots=4, s_max=8192)
    firsts4, _ = net.prefill(four, [0, 1, 2, 3], prompts)
    assert firsts4[:3].tolist() == firsts.tolist()
    four.batch_slots = [0, 1, 2, 3]
    nxt4 = firsts4.view(4, 1).clone()
    for i in range(steps):
        nxt4[:3] = fed[i]
        logits = net(nxt4, past_key_values=four).logits[:, 0]
        ok, err = _close(logits[:3], chain[i])
        assert ok, (i, err)
        nxt4 = logits.argmax(dim=-1, keepdim=True)


def test_golden_hf_quant_logits(tiny_model):
    """Against logits the reference's own model_hf.load produced (tests/golden/make_golden.py)."""
    net, _, _, _ = tiny_model
    g = np.load(os.path.join(GOLDEN, "hf_quant_logits.npz"))
    assert json.loads(str(g["model"])) == {"n_layers": 2, "vocab": 2048, "seed": 1234}
    prompt, tokens = g["prompt"].tolist(), g["tokens"].tolist()
    cache = net.new_cache(n_slots=2, s_max=128)
    cache.batch_slots = [0]
    out = net(torch.tensor([prompt]), past_key_values=cache)
    got = [out.logits[0, -1].clone()]
    for t in tokens[:-1]:  # teacher-forced with the reference's tokens
        out = net(torch.tensor([[t]]), past_key_values=cache)
        got.append(out.logits[0, -1].clone())
    got = torch.stack(got)
    ok, err = _close(got, torch.from_numpy(g["logits"]))
    assert ok, err
    assert got.argmax(-1).tolist() == tokens


def test_slots_are_checked_before_any_launch(tiny_model):
    """Slots outside the cache, repeated slots and a slot count that does not match the rows
    are refused on the host by prefill(), decode() and forward()."""
    net = tiny_model[0]
    cache = net.new_cache(n_slots=2, s_max=64)
    p = torch.tensor([5, 6, 7])
    for bad in ([2], [-1], [0, 0], [0, 1, 1]):
        with pytest.raises(ValueError):
            net.prefill(cache, bad, [p] * len(bad))
    with pytest.raises(ValueError):
        net.prefill(cache, [0, 1], [p])
    net.prefill(cache, [1], [p])
    for bad in ([2], [1, 1], [-3]):
        with pytest.raises(ValueError):
            net.decode(cache, bad, 1)
    small = net.new_cache(n_slots=2, s_max=64)
    with pytest.raises(ValueError):  # three rows, two slots
        net(torch.tensor([[1, 2], [3, 4], [5, 6]]), past_key_values=small)
    assert net.decode(cache, [1], 2)[0]  # the cache is still usable


@pytest.mark.parametrize("all_logits", [False, True])
def test_chunked_prefill_equals_whole_prompt_prefill(tiny_model, all_logits):
    """A prompt prefilled in chunks (prefill(..., offsets=...): 17 + 40 + 3 tokens and, in the
    same calls, a second sequence in one piece) must leave the slot and the following decode
    exactly as the whole prompt does, in the fused library call and in the per-op path."""
    net = tiny_model[0]
    gen = torch.Generator().manual_seed(21)
    long_p, short_p = torch.randint(0, 2048, (60,), generator=gen), torch.randint(0, 2048, (9,), generator=gen)
    whole = net.new_cache(n_slots=4, s_max=128)
    first_w, _ = net.prefill(whole, [2, 0], [long_p, short_p], all_logits=all_logits)
    tokens_w = net.decode(whole, [2, 0], 8)

    cache = net.new_cache(n_slots=4, s_max=128)
    net.prefill(cache, [2, 0], [long_p[:17], short_p], all_logits=all_logits)
    net.prefill(cache, [2], [long_p[17:57]], all_logits=all_logits, offsets=[17])
    first_c, _ = net.prefill(cache, [2], [long_p[57:]], all_logits=all_logits, offsets=[57])
    assert cache.host_len[2] == 60 and int(cache.pos[2]) == 60
    assert int(first_c[0]) == int(first_w[0])
    assert torch.equal(cache.kv[:, :, 2, :, :60], whole.kv[:, :, 2, :, :60])
    assert net.decode(cache, [2, 0], 8) == tokens_w
    with pytest.raises(ValueError):
        net.prefill(cache, [2], [long_p[:4]], offsets=[5])  # does not continue what the slot holds


def test_forward_accepts_a_multi_token_input_on_a_filled_cache(tiny_model):
    """The reference's forward takes seq_len > 1 with past_key_values (src/model.py:280-291):
    here that is the next chunk of every row's prompt."""
    net, ref, _, _ = tiny_model
    prompt = [11, 7, 1999, 42, 0, 512, 77, 1023, 5, 6, 900]
    ref_tokens, ref_logits = ref.greedy(prompt, 1)
    cache = net.new_cache(n_slots=2, s_max=64)
    cache.batch_slots = [1]
    net(torch.tensor([prompt[:4]]), past_key_values=cache)
    out = net(torch.tensor([prompt[4:]]), past_key_values=cache)
    assert out.logits.shape == (1, 1, 2048) and cache.get_seq_length() == len(prompt)
    got = out.logits[0, 0].float().cpu()
    assert torch.allclose(got, ref_logits[0].float(), rtol=2e-2, atol=5e-2), (got - ref_logits[0].float()).abs().max()
