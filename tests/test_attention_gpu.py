"""Split-K GQA decode attention against SDPA (the reference's recipe,
tests/test_attention.py:57-82: same shapes, pads, seed rule and tolerance) and the oracle."""

import pytest
import torch
import torch.nn.functional as F

from oracle import quic_ref

pytestmark = pytest.mark.gpu
BATCH, HEADS, HEAD_DIM = 4, 14, 64
SCALE = HEAD_DIM ** -0.5
ATOL = 1e-2


def _sdpa(q, k, v, pad_lens):
    kv_len = k.shape[2]
    pos = torch.arange(kv_len, device=q.device)
    not_pad = pos[None, :] >= pad_lens[:, None]
    mask = not_pad[:, None, None, :].expand(q.shape[0], HEADS, 1, kv_len)
    return F.scaled_dot_product_attention(q.float(), k.repeat_interleave(7, dim=1).float(),
                                          v.repeat_interleave(7, dim=1).float(), attn_mask=mask,
                                          scale=SCALE).to(q.dtype)


@pytest.mark.parametrize("kv_len", [16, 64, 256])
def test_decode_matches_sdpa_with_left_padding(kv_len):
    from quic_cu_b200 import kernels as K

    generator = torch.Generator(device="cuda").manual_seed(kv_len)
    q = torch.randn((BATCH, HEADS, 1, HEAD_DIM), device="cuda", generator=generator).half()
    k = torch.randn((BATCH, 2, kv_len, HEAD_DIM), device="cuda", generator=generator).half()
    v = torch.randn((BATCH, 2, kv_len, HEAD_DIM), device="cuda", generator=generator).half()
    pad_lens = torch.tensor([0, 2, kv_len // 4, kv_len - 1], device="cuda", dtype=torch.int32)
    out = K.flash_attn_decode().forward(q, k, v, SCALE, pad_lens)
    expected = _sdpa(q, k, v, pad_lens)
    assert out.shape == (BATCH, HEADS, 1, HEAD_DIM)
    assert torch.isfinite(out).all()
    assert torch.allclose(out.float(), expected.float(), atol=ATOL)


@pytest.mark.parametrize("batch,kv_len,splits", [(1, 1, 0), (1, 33, 1), (2, 300, 3), (3, 1000, 0),
                                                  (1, 8192, 0), (5, 2049, 7), (16, 1024, 0)])
def test_decode_split_merge_and_ragged(batch, kv_len, splits):
    """Every split count gives the same answer; pads uniform in [0, S/4]; second call re-uses
    the scratch (arrival counters must have been re-armed)."""
    from quic_cu_b200 import kernels as K

    g = torch.Generator(device="cuda").manual_seed(batch * 100003 + kv_len)
    q = torch.randn((batch, HEADS, 1, HEAD_DIM), device="cuda", generator=g).half()
    k = torch.randn((batch, 2, kv_len, HEAD_DIM), device="cuda", generator=g).half()
    v = torch.randn((batch, 2, kv_len, HEAD_DIM), device="cuda", generator=g).half()
    pads = torch.randint(0, kv_len // 4 + 1, (batch,), device="cuda", generator=g).int()
    expected = _sdpa(q, k, v, pads)
    for _ in range(2):
        out = K.flash_attn_decode().forward(q, k, v, SCALE, pads, splits=splits)
        assert torch.allclose(out.float(), expected.float(), atol=ATOL)
    out_nopad = K.flash_attn_decode().forward(q, k, v)  # default scale, no pads
    assert torch.allclose(out_nopad.float(), _sdpa(q, k, v, torch.zeros_like(pads)).float(), atol=ATOL)


@pytest.mark.parametrize("batch,kv_len", [(1, 1), (1, 64), (1, 65), (2, 300), (3, 1000), (1, 1024), (4, 1537)])
def test_decode_latency_variant(batch, kv_len):
    """One split per 64 tokens selects the single-warp tensor-core variant the decode chain
    uses at small batch: left pads (one row fully padded where there are several rows), keys
    beyond the last split masked, the splits merged by the last CTA to arrive; twice, so the
    arrival counters must have been re-armed."""
    from quic_cu_b200 import kernels as K

    g = torch.Generator(device="cuda").manual_seed(batch * 7919 + kv_len)
    q = torch.randn((batch, HEADS, 1, HEAD_DIM), device="cuda", generator=g).half()
    k = torch.randn((batch, 2, kv_len, HEAD_DIM), device="cuda", generator=g).half()
    v = torch.randn((batch, 2, kv_len, HEAD_DIM), device="cuda", generator=g).half()
    pads = torch.randint(0, kv_len // 2 + 1, (batch,), device="cuda", generator=g).int()
    if batch > 2:
        pads[1] = kv_len
    want = quic_ref.attn_decode(q[:, :, 0].cpu(), k.cpu(), v.cpu(), SCALE, start=pads.cpu())
    splits = (kv_len + 63) // 64
    for _ in range(2):
        out = K.flash_attn_decode().forward(q, k, v, SCALE, pads, splits=splits)
        assert torch.isfinite(out).all()
        assert torch.allclose(out[:, :, 0].cpu().float(), want.float(), atol=ATOL)


def test_all_masked_row_gives_zeros_and_oracle_agrees():
    """flash_attn_decode.cu:118-121: a row whose every key is padding yields 0."""
    from quic_cu_b200 import kernels as K

    g = torch.Generator(device="cuda").manual_seed(5)
    q = torch.randn((3, HEADS, 1, HEAD_DIM), device="cuda", generator=g).half()
    k = torch.randn((3, 2, 700, HEAD_DIM), device="cuda", generator=g).half()
    v = torch.randn((3, 2, 700, HEAD_DIM), device="cuda", generator=g).half()
    pads = torch.tensor([700, 0, 699], device="cuda", dtype=torch.int32)
    for splits in (1, 4):
        out = K.flash_attn_decode().forward(q, k, v, SCALE, pads, splits=splits)
        assert torch.count_nonzero(out[0]) == 0
        want = quic_ref.attn_decode(q[:, :, 0].cpu(), k.cpu(), v.cpu(), SCALE, start=pads.cpu())
        assert torch.allclose(out[:, :, 0].cpu().float(), want.float(), atol=2e-3)


@pytest.mark.parametrize("batch,kv_len", [(4, 32768), (256, 1024), (64, 8192), (64, 32768), (256, 8192)])
def test_decode_sweep_corners(batch, kv_len):
    """Corners of the benchmark's attention sweep (maximum context, maximum batch, and the two
    largest problems, which are the ones that run at the memory roofline: 2.1 GB of K and V
    each): against SDPA on the first rows, and split-count invariance on all rows."""
    from quic_cu_b200 import kernels as K

    g = torch.Generator(device="cuda").manual_seed(batch + kv_len)
    q = torch.randn((batch, HEADS, 1, HEAD_DIM), device="cuda", generator=g).half()
    k = torch.randn((batch, 2, kv_len, HEAD_DIM), device="cuda", generator=g).half()
    v = torch.randn((batch, 2, kv_len, HEAD_DIM), device="cuda", generator=g).half()
    pads = torch.randint(0, kv_len // 4 + 1, (batch,), device="cuda", generator=g).int()
    out = K.flash_attn_decode().forward(q, k, v, SCALE, pads)
    rows = slice(0, min(batch, 4))
    expected = _sdpa(q[rows], k[rows], v[rows], pads[rows])
    assert torch.allclose(out[rows].float(), expected.float(), atol=ATOL)
    other = K.flash_attn_decode().forward(q, k, v, SCALE, pads, splits=1 if kv_len <= 8192 else 7)
    assert torch.allclose(out.float(), other.float(), atol=2e-3)
    assert torch.isfinite(out).all()


@pytest.mark.parametrize("lens", [[1], [16], [17, 64], [65, 3, 130], [560], [1024, 300], [1500, 700, 33]])
def test_prefill_attention_matches_causal_sdpa(lens):
    """quic_attn_prefill against causal torch SDPA per sequence (the reference's default
    prefill attention, kernels/flash_attn_prefill_pytorch.py:10): sequences of ragged
    lengths in one launch, keys and values read from scattered KV slots."""
    from quic_cu_b200 import kernels as K

    g = torch.Generator(device="cuda").manual_seed(sum(lens))
    rows, n_slots, s_max = sum(lens), 5, 1536  # one sequence or up to 1024 rows: warps split the keys; beyond: rows
    slots = [4, 0, 2][: len(lens)]
    q = torch.randn((HEADS, rows, HEAD_DIM), device="cuda", generator=g).half()
    kc = torch.randn((n_slots, 2, s_max, HEAD_DIM), device="cuda", generator=g).half()
    vc = torch.randn((n_slots, 2, s_max, HEAD_DIM), device="cuda", generator=g).half()
    starts = [sum(lens[:i]) for i in range(len(lens))]
    dev = dict(device="cuda", dtype=torch.int32)
    out = K.attn_prefill(q, kc, vc, torch.tensor(starts, **dev), torch.tensor(lens, **dev),
                         torch.tensor(slots, **dev), max(lens), SCALE)
    assert out.shape == (rows, HEADS * HEAD_DIM) and torch.isfinite(out).all()
    for a, n, s in zip(starts, lens, slots):
        want = torch.nn.functional.scaled_dot_product_attention(
            q[None, :, a:a + n].float(), kc[None, s, :, :n].float(), vc[None, s, :, :n].float(),
            is_causal=True, scale=SCALE, enable_gqa=True)[0]  # [14, n, 64]
        got = out[a:a + n].view(n, HEADS, HEAD_DIM).transpose(0, 1).float()
        assert torch.allclose(got, want, atol=ATOL), (n, (got - want).abs().max().item())


@pytest.mark.parametrize("batch,kv_len", [(1, 1), (2, 63), (1, 512), (3, 513), (2, 1000), (16, 777), (4, 2048),
                                          (2, 3585), (5, 4096)])
def test_decode_cta_merge_variant(batch, kv_len):
    """The scratch-free form (CTAs of 512 tokens; beyond 512 tokens a cluster of CTAs merged
    through the first CTA's shared memory) against the oracle: ragged left pads, one row fully
    padded, lengths on both sides of a CTA and of a warp boundary, the longest cache it takes."""
    from quic_cu_b200 import kernels as K

    g = torch.Generator(device="cuda").manual_seed(batch * 104729 + kv_len)
    q = torch.randn((batch, HEADS, 1, HEAD_DIM), device="cuda", generator=g).half()
    k = torch.randn((batch, 2, kv_len, HEAD_DIM), device="cuda", generator=g).half()
    v = torch.randn((batch, 2, kv_len, HEAD_DIM), device="cuda", generator=g).half()
    pads = torch.randint(0, kv_len // 2 + 1, (batch,), device="cuda", generator=g).int()
    if batch > 2:
        pads[1] = kv_len
    want = quic_ref.attn_decode(q[:, :, 0].cpu(), k.cpu(), v.cpu(), SCALE, start=pads.cpu())
    for _ in range(2):
        out = K.flash_attn_decode().forward(q, k, v, SCALE, pads, cta_merge=True)
        assert torch.isfinite(out).all()
        assert torch.allclose(out[:, :, 0].float().cpu(), want.float(), atol=ATOL)


def test_decode_cta_merge_refuses_longer_caches():
    from quic_cu_b200 import kernels as K

    q = torch.zeros((1, HEADS, 1, HEAD_DIM), device="cuda").half()
    k = torch.zeros((1, 2, 4097, HEAD_DIM), device="cuda").half()
    with pytest.raises(RuntimeError, match="4096"):
        K.flash_attn_decode().forward(q, k, k, SCALE, None, cta_merge=True)


def test_prefill_attention_of_a_later_chunk_sees_the_cached_tokens():
    """quic_attn_prefill with seq_off: the rows of a call are tokens off .. off + len - 1 of their
    sequence, keys and values 0 .. off + len - 1 come from the slot; against causal SDPA over
    the whole sequence.  Offsets on both sides of the 16-row and 32-key tile edges, one
    sequence without an offset, one whose slot index is not its row."""
    from quic_cu_b200 import kernels as K

    g = torch.Generator(device="cuda").manual_seed(11)
    offs, lens, slots = [37, 0, 16, 511], [50, 21, 1, 33], [2, 0, 3, 1]
    s_max = 600
    kc = torch.zeros(4, 2, s_max, 64, device="cuda", dtype=torch.float16)
    vc = torch.zeros_like(kc)
    rows = sum(lens)
    q = torch.randn(HEADS, rows, 64, device="cuda", generator=g).half()
    starts, want = [], torch.empty(rows, HEADS * 64)
    a = 0
    for off, n, slot in zip(offs, lens, slots):
        starts.append(a)
        kc[slot, :, : off + n] = torch.randn(2, off + n, 64, device="cuda", generator=g).half()
        vc[slot, :, : off + n] = torch.randn(2, off + n, 64, device="cuda", generator=g).half()
        keys = kc[slot, :, : off + n].repeat_interleave(7, dim=0).float()
        vals = vc[slot, :, : off + n].repeat_interleave(7, dim=0).float()
        qs = q[:, a:a + n].float()                                           # [14, n, 64]
        causal = torch.arange(off + n, device="cuda")[None, :] <= (off + torch.arange(n, device="cuda"))[:, None]
        o = F.scaled_dot_product_attention(qs[None], keys[None], vals[None], attn_mask=causal[None, None], scale=SCALE)
        want[a:a + n] = o[0].transpose(0, 1).reshape(n, -1).cpu()
        a += n
    dev = dict(device="cuda", dtype=torch.int32)
    out = K.attn_prefill(q, kc, vc, torch.tensor(starts, **dev), torch.tensor(lens, **dev), torch.tensor(slots, **dev),
                         max(lens), seq_off=torch.tensor(offs, **dev))
    assert torch.allclose(out.float().cpu(), want, atol=ATOL), (out.float().cpu() - want).abs().max()


@pytest.mark.parametrize("kv_repeated", [True, False])
def test_flash_attn_prefill_getter_matches_the_reference_recipe(kv_repeated):
    """flash_attn_prefill().forward on a left-padded batch, the reference's call shape
    (src/model.py:176-183), against its PyTorch backend's mask recipe
    (kernels/flash_attn_prefill_pytorch.py:21-32) on the rows that are real tokens."""
    from quic_cu_b200 import kernels as K

    g = torch.Generator(device="cuda").manual_seed(3)
    b, n = 3, 70
    q = torch.randn(b, HEADS, n, 64, device="cuda", generator=g).half()
    k = torch.randn(b, 2, n, 64, device="cuda", generator=g).half()
    v = torch.randn(b, 2, n, 64, device="cuda", generator=g).half()
    pads = torch.tensor([0, 13, 69], device="cuda", dtype=torch.int32)
    kr, vr = k.repeat_interleave(7, dim=1), v.repeat_interleave(7, dim=1)
    out = K.flash_attn_prefill().forward(q, kr if kv_repeated else k, vr if kv_repeated else v, True, SCALE, pads)
    pos = torch.arange(n, device="cuda")
    mask = ((pos[None, :] <= pos[:, None])[None, None] & (pos[None, :] >= pads[:, None])[:, None, None, :]) | \
        torch.eye(n, dtype=torch.bool, device="cuda")
    want = F.scaled_dot_product_attention(q.float(), kr.float(), vr.float(), attn_mask=mask, scale=SCALE)
    real = (pos[None, :] >= pads[:, None])[:, None, :, None].expand_as(out)
    assert torch.allclose(out.float()[real], want[real], atol=ATOL)
    assert torch.count_nonzero(out[~real]) == 0


@pytest.mark.parametrize("lens,offs", [([128], None), ([300, 129], None), ([2048], None), ([640, 1, 200], None),
                                       ([256, 130], [100, 513]), ([129], [1407])])
def test_prefill_attention_tensor_and_mma_kernels_agree_with_sdpa(lens, offs):
    """Prompts of 128 tokens and more run on tcgen05 (128-row query tiles, 64-key tiles through
    TMA, S and O in tensor memory); the mma.sync kernels are kept for shorter ones and as the
    comparison here.  Both against causal SDPA over each whole sequence: ragged lengths, rows
    that end inside a tile, later chunks of a prompt (offsets on both sides of tile edges)."""
    from quic_cu_b200 import kernels as K

    g = torch.Generator(device="cuda").manual_seed(sum(lens) + 7)
    offs = offs or [0] * len(lens)
    rows, n_slots, s_max = sum(lens), 4, 2048
    slots = [3, 0, 2][: len(lens)]
    q = torch.randn((HEADS, rows, HEAD_DIM), device="cuda", generator=g).half()
    kc = torch.randn((n_slots, 2, s_max, HEAD_DIM), device="cuda", generator=g).half()
    vc = torch.randn((n_slots, 2, s_max, HEAD_DIM), device="cuda", generator=g).half()
    starts = [sum(lens[:i]) for i in range(len(lens))]
    dev = dict(device="cuda", dtype=torch.int32)
    args = (q, kc, vc, torch.tensor(starts, **dev), torch.tensor(lens, **dev), torch.tensor(slots, **dev), max(lens), SCALE)
    off_t = torch.tensor(offs, **dev) if any(offs) else None
    out = K.attn_prefill(*args, seq_off=off_t)
    assert K.lib().quic_w4a16_tensor_status() == 0
    try:
        K.lib().quic_set_prefill_tensor_attention(0)
        other = K.attn_prefill(*args, seq_off=off_t)
    finally:
        K.lib().quic_set_prefill_tensor_attention(1)
    assert torch.isfinite(out).all()
    for a, n, s, o in zip(starts, lens, slots, offs):
        keys = kc[s, :, : o + n].repeat_interleave(7, dim=0).float()
        vals = vc[s, :, : o + n].repeat_interleave(7, dim=0).float()
        causal = torch.arange(o + n, device="cuda")[None, :] <= (o + torch.arange(n, device="cuda"))[:, None]
        want = F.scaled_dot_product_attention(q[None, :, a:a + n].float(), keys[None], vals[None],
                                              attn_mask=causal[None, None], scale=SCALE)[0]
        got = out[a:a + n].view(n, HEADS, HEAD_DIM).transpose(0, 1).float()
        assert torch.allclose(got, want, atol=ATOL), (n, o, (got - want).abs().max().item())
        ref = other[a:a + n].view(n, HEADS, HEAD_DIM).transpose(0, 1).float()
        assert torch.allclose(got, ref, atol=4e-3), (n, o, (got - ref).abs().max().item())


def test_prefill_attention_gives_the_same_bits_every_run():
    """The tcgen05 kernel's roles hand tiles to each other through mbarriers; a hand-off that lets
    one pair of softmax warps run ahead of another shows up as a few rows that differ between
    runs (it did, once: arrivals for tile i + 1 counted for tile i).  Thirty runs of a ragged
    batch with a 4300-token sequence must be bit-identical, and so must the decode attention
    with a cluster merge."""
    from quic_cu_b200 import kernels as K

    g = torch.Generator(device="cuda").manual_seed(99)
    lens = [4300, 40, 700, 3000]
    rows, s_max = sum(lens), 4352
    q = torch.randn((HEADS, rows, HEAD_DIM), device="cuda", generator=g).half()
    kc = torch.randn((4, 2, s_max, HEAD_DIM), device="cuda", generator=g).half()
    vc = torch.randn((4, 2, s_max, HEAD_DIM), device="cuda", generator=g).half()
    dev = dict(device="cuda", dtype=torch.int32)
    starts = torch.tensor([sum(lens[:i]) for i in range(4)], **dev)
    args = (q, kc, vc, starts, torch.tensor(lens, **dev), torch.arange(4, **dev), max(lens), SCALE)
    first = K.attn_prefill(*args).clone()
    for _ in range(30):
        assert torch.equal(K.attn_prefill(*args), first)

    qd = torch.randn((3, HEADS, 1, HEAD_DIM), device="cuda", generator=g).half()
    pads = torch.tensor([0, 100, 4000], **dev)
    kd, vd = kc[:3, :, :4096].contiguous(), vc[:3, :, :4096].contiguous()  # the longest cache that kernel takes
    first = K.flash_attn_decode().forward(qd, kd, vd, SCALE, pads, cta_merge=True).clone()
    for _ in range(30):
        assert torch.equal(K.flash_attn_decode().forward(qd, kd, vd, SCALE, pads, cta_merge=True), first)
    assert K.lib().quic_w4a16_tensor_status() == 0
