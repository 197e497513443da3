"""The persistent decode kernel (one launch per burst of tokens, 1..4 rows) against the CPU
oracle and against the kernel chain it replaces, through the C ABI."""

import pytest
import torch

pytestmark = pytest.mark.gpu
RTOL, ATOL = 2e-2, 5e-2


def _close(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return bool(((a - b).abs() <= ATOL + RTOL * b.abs()).all()), (a - b).abs().max().item()


def _greedy_agrees(got, ref_tokens, ref_logits, near_tie=2e-2):
    """Index of the first position where the sequences part (only allowed at a near-tie of the
    oracle's top two logits), or len(ref_tokens)."""
    for i, (g, r) in enumerate(zip(got, ref_tokens)):
        if g == r:
            continue
        top = torch.topk(ref_logits[i].float(), 2)
        gap = (top.values[0] - top.values[1]).item()
        assert gap < near_tie and g in top.indices.tolist(), (i, g, r, gap)
        return i
    return len(ref_tokens)


@pytest.fixture()
def persist_net(tiny_model):
    net = tiny_model[0]
    old = net.use_persist
    net.use_persist = True
    yield net
    net.use_persist = old


def test_single_row_logits_and_tokens_match_oracle(persist_net, tiny_model):
    """Prompt and generation token by token through forward(): every step is one launch of the
    persistent kernel with logits kept (positions 0..n, so the first launch sees an empty slot)."""
    net, ref = persist_net, tiny_model[1]
    prompt = [11, 7, 1999, 42, 0, 512, 77, 1023]
    ref_tokens, ref_logits = ref.greedy(prompt, 6)
    cache = net.new_cache(n_slots=4, s_max=256)
    cache.batch_slots = [2]
    assert net.persist_ok(1, 256)
    logits = None
    for t in prompt:
        logits = net(torch.tensor([[t]]), past_key_values=cache).logits
    got_tokens, got_logits = [], []
    for _ in range(6):
        got_logits.append(logits[0, 0].clone())
        nxt = logits[:, -1:, :].argmax(dim=-1)
        got_tokens.append(int(nxt))
        logits = net(nxt, past_key_values=cache).logits
    assert net.persist_status(cache) == 0
    n = _greedy_agrees(got_tokens, ref_tokens, ref_logits)
    ok, err = _close(torch.stack(got_logits)[: n + 1], ref_logits[: n + 1])
    assert ok, err


@pytest.mark.parametrize("rows", [1, 2, 3, 4])
def test_bursts_match_the_kernel_chain_and_the_oracle(persist_net, tiny_model, rows):
    """Ragged rows, a 40-token burst in one launch: the persistent kernel must give the oracle's
    tokens (up to a near-tie) and the logits of the kernel chain on the same fed tokens."""
    net, ref = persist_net, tiny_model[1]
    gen = torch.Generator().manual_seed(100 + rows)
    lens = [70, 9, 300, 33][:rows]
    prompts = [torch.randint(0, 2048, (n,), generator=gen) for n in lens]
    slots = [5, 0, 3, 6][:rows]
    steps = 40

    cache = net.new_cache(n_slots=8, s_max=512)
    first, _ = net.prefill(cache, slots, prompts)
    burst = net.decode(cache, slots, steps)
    assert net.persist_status(cache) == 0
    for i in range(rows):
        want_tokens, want_logits = ref.greedy(prompts[i].tolist(), 12)
        _greedy_agrees([int(first[i])] + burst[i][:11], want_tokens, want_logits)

    # the same burst as single steps gives the same tokens bit for bit
    cache1 = net.new_cache(n_slots=8, s_max=512)
    net.prefill(cache1, slots, prompts)
    singles = [[] for _ in range(rows)]
    for _ in range(steps):
        out = net.decode(cache1, slots, 1)
        for i in range(rows):
            singles[i] += out[i]
    assert singles == burst

    # logits of one more step, persistent kernel vs kernel chain, same cache contents
    cache.batch_slots = slots
    cache1.batch_slots = slots
    nxt = torch.tensor([[b[-1]] for b in burst])
    a = net(nxt, past_key_values=cache).logits[:, 0].clone()
    net.use_persist = False
    try:
        b = net(nxt, past_key_values=cache1).logits[:, 0].clone()
    finally:
        net.use_persist = True
    ok, err = _close(a, b)
    assert ok, err
    assert a.argmax(-1).tolist() == b.argmax(-1).tolist() or err < 2e-2


@pytest.mark.parametrize("prompt_len", [383, 384, 1100, 3900])
def test_split_boundaries_and_long_contexts(persist_net, tiny_model, prompt_len):
    """Contexts around a split boundary (splits of 192 tokens below 512: the row being decoded
    is the last of a split at 383 and the first of the next at 384) and up to the kernel's
    longest context, sixteen splits of 256 tokens merged by the o_proj CTAs in rounds of four:
    logits against the oracle's teacher-forced pass."""
    from oracle.quic_ref import RefModel

    net = persist_net
    ref = RefModel(tiny_model[2], 2, max_pos=4096)
    prompt = torch.randint(0, 2048, (prompt_len,), generator=torch.Generator().manual_seed(prompt_len))
    steps = 5
    cache = net.new_cache(n_slots=2, s_max=4096)
    assert net.persist_ok(1, min(4096, prompt_len + 128))
    first, _ = net.prefill(cache, [1], [prompt])
    cache.batch_slots = [1]
    fed, kept = [int(first[0])], []
    for _ in range(steps):
        logits = net(torch.tensor([[fed[-1]]]), past_key_values=cache).logits[0, 0].clone()
        kept.append(logits)
        fed.append(int(logits.argmax()))
    assert net.persist_status(cache) == 0
    want = ref.teacher_forced(prompt.tolist(), fed)[1:]  # logits after feeding fed[0..steps-1]
    ok, err = _close(torch.stack(kept), want[:steps])
    assert ok, err


def test_host_fed_single_steps_agree_with_a_burst(persist_net):
    """The host-driven form (token in from pinned memory, id and status word out, stream
    synchronised) must reproduce the tokens of one 24-step launch."""
    net = persist_net
    prompt = torch.tensor([17, 4, 256, 1000, 31, 8, 8, 1203, 77])
    cache = net.new_cache(n_slots=2, s_max=256)
    first, _ = net.prefill(cache, [1], [prompt])
    burst = [int(first[0])] + net.decode(cache, [1], 24)[0]
    cache = net.new_cache(n_slots=2, s_max=256)
    first, _ = net.prefill(cache, [1], [prompt])
    pinned = torch.zeros(1, dtype=torch.int32).pin_memory()
    fed = [int(first[0])]
    for _ in range(24):
        pinned[0] = fed[-1]
        fed.append(net.decode(cache, [1], 1, feed=pinned)[0][0])
    assert fed == burst


def test_a_wait_that_runs_out_is_reported_and_the_next_launch_works(persist_net):
    """Bounded waits: with the probe limit lowered to 4096 and CTA 0 withholding its o_proj
    result of layer 0 (both through the header words of the exchange area), the polls that
    need that result give up, the kernel returns, the status word names the wait, nothing
    was generated; after clearing the hook the same area serves a normal launch whose
    tokens match an undisturbed run."""
    net = persist_net
    prompt = torch.tensor([5, 900, 13, 2000, 7])
    want_cache = net.new_cache(n_slots=2, s_max=256)
    first, _ = net.prefill(want_cache, [0], [prompt])
    want = net.decode(want_cache, [0], 6)[0]

    cache = net.new_cache(n_slots=2, s_max=256)
    net.prefill(cache, [0], [prompt])
    hdr = cache.persist_sync()[:16].view(torch.int32)
    hdr[2] = 4096
    hdr[3] = 1
    pos_before = int(cache.pos[0])
    with pytest.raises(RuntimeError, match="bounded wait"):
        net.decode(cache, [0], 1)
    torch.cuda.synchronize()
    assert int(cache.pos[0]) == pos_before      # no token was produced
    assert int(hdr[1]) == 0                     # the failing call cleared the word
    hdr[2] = 0
    hdr[3] = 0
    cache.host_steps -= 1                       # undo the host mirrors of the abandoned step
    cache.host_len[0] -= 1
    assert net.decode(cache, [0], 6)[0] == want
    assert net.persist_status(cache) == 0

    # the asynchronous form leaves the code in the status word: 0x100 | (layer * 8 + phase)
    hdr[2] = 4096
    hdr[3] = 2
    net.decode_async(cache, [0], 1)
    assert net.persist_status(cache) == (0x100 | (1 * 8 + 3))
    hdr[2] = 0
    hdr[3] = 0
    cache.host_steps -= 1
    cache.host_len[0] -= 1
    more = net.decode(cache, [0], 3)[0]
    assert more == net.decode(want_cache, [0], 3)[0]
