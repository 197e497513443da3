"""Stand-alone ops against the reference's own test recipes (tests/test_kernels.py of the
reference: same shapes and tolerances) and against the CPU oracle."""

import pytest
import torch
import torch.nn.functional as F

from oracle import quic_ref

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from quic_cu_b200 import kernels

    return kernels


def test_rmsnorm(K):  # reference tests/test_kernels.py:11
    torch.manual_seed(0)
    x = torch.randn(8, 896, device="cuda", dtype=torch.float16)
    w = torch.ones(896, device="cuda", dtype=torch.float16)
    out = K.rmsnorm().forward(x, w, 1e-6)
    variance = x.float().pow(2).mean(-1, keepdim=True)
    expected = (x.float() * torch.rsqrt(variance + 1e-6) * w.float()).half()
    assert torch.allclose(out, expected, atol=1e-2)


@pytest.mark.parametrize("rows", [0, 1, 7, 8, 9, 1000])
def test_rmsnorm_residual_vs_oracle(K, rows):
    torch.manual_seed(rows)
    x = torch.randn(rows, 896, device="cuda", dtype=torch.float16)
    r = torch.randn(rows, 896, device="cuda", dtype=torch.float16) * 3
    w = (torch.randn(896, device="cuda") * 0.5 + 1).half()
    y, total = K.rmsnorm().forward(x, w, 1e-6, residual=r)
    want_total = quic_ref.residual_add(x.cpu(), r.cpu())
    assert torch.equal(total.cpu(), want_total)  # one fp16 rounding of an fp32 sum: exact
    want = quic_ref.rmsnorm(want_total, w.cpu(), 1e-6)
    assert torch.allclose(y.cpu().float(), want.float(), atol=2e-3, rtol=2e-3)


def test_swiglu(K):  # reference tests/test_kernels.py:26
    torch.manual_seed(0)
    gate = torch.randn(16, 4864, device="cuda", dtype=torch.float16)
    up = torch.randn(16, 4864, device="cuda", dtype=torch.float16)
    out = K.swiglu().forward(gate, up)
    expected = (F.silu(gate.float()) * up.float()).half()
    assert torch.allclose(out, expected, atol=1e-2)
    # the same on the fused gate|up layout: bit-identical to the two-tensor form
    fused = K.swiglu_fused(torch.cat([gate, up], dim=1))
    assert torch.equal(fused, out)
    assert K.swiglu_fused(torch.empty(0, 9728, device="cuda", dtype=torch.float16)).shape == (0, 4864)


def test_gemm(K):  # reference tests/test_kernels.py:38
    torch.manual_seed(0)
    m, k, n = 8, 896, 4864
    x = torch.randn(m, k, device="cuda", dtype=torch.float16) * 0.1
    w = torch.randn(n, k, device="cuda", dtype=torch.float16) * 0.1
    b = torch.randn(n, device="cuda", dtype=torch.float16) * 0.1
    out = K.gemm().forward(x, w, b)
    expected = F.linear(x.float(), w.float(), b.float())
    assert torch.allclose(out.float(), expected, rtol=1e-2, atol=2e-2)
    out1 = K.gemm().forward(x[:1], w, None)
    assert torch.allclose(out1.float(), F.linear(x[:1].float(), w.float()), rtol=1e-2, atol=2e-2)


def test_sampler(K):  # reference tests/test_kernels.py:51
    torch.manual_seed(0)
    logits = torch.randn(4, 1, 151936, device="cuda", dtype=torch.float16)
    out = K.sampler().forward(logits)
    assert torch.equal(out.view(-1), torch.argmax(logits, dim=-1).view(-1))


def test_sampler_ties_pick_lowest_index(K):  # kernels/cuda/sampler.cu:38-40
    logits = torch.zeros(3, 1, 5000, device="cuda", dtype=torch.float16)
    logits[0, 0, [4999, 17, 2500]] = 3.0
    logits[1, 0, :] = -1.0
    logits[2, 0, [4098, 4097]] = 0.5
    assert K.sampler().forward(logits).view(-1).tolist() == [17, 0, 4097]


def test_lm_head_argmax_matches_gemm_and_sampler(K):
    torch.manual_seed(1)
    for b, vocab in ((1, 151936), (3, 4096), (8, 2050), (11, 1024)):
        x = torch.randn(b, 896, device="cuda", dtype=torch.float16)
        w = (torch.randn(896, device="cuda") * 0.3 + 1).half()
        table = (torch.randn(vocab, 896, device="cuda") * 0.02).half()
        tokens, logits = K.lm_head_argmax(x, table, w, 1e-6, want_logits=True)
        xn = quic_ref.rmsnorm(x.cpu(), w.cpu(), 1e-6).cuda()
        want = F.linear(xn.float(), table.float())
        assert torch.allclose(logits.float(), want, atol=2e-3, rtol=2e-3)
        # argmax is exact given the kernel's own fp16 logits
        assert torch.equal(tokens, K.sampler().forward(logits.unsqueeze(1)).view(-1))
        tokens2, _ = K.lm_head_argmax(xn, table)  # pre-normalised input, second call re-uses scratch
        assert torch.equal(tokens2, tokens)


def test_rope_table_and_rotation(K):
    exponent = torch.arange(0, 64, 2, dtype=torch.float32) / 64
    inv_freq = (1.0 / (1e6 ** exponent)).cuda()
    cos, sin = K.rope().init_table(inv_freq, 32768)
    rc, rs = quic_ref.rope_tables(32768)
    # accurate sincos on both sides: at most one fp16 ulp apart
    assert (cos.cpu().float() - rc.float()).abs().max() <= 1e-3
    assert (sin.cpu().float() - rs.float()).abs().max() <= 1e-3
    torch.manual_seed(0)
    x = torch.randn(2, 5, 7, 64, device="cuda", dtype=torch.float16)
    y = K.rope().forward(x, cos[:7].contiguous(), sin[:7].contiguous())
    want = quic_ref.rope(x.cpu(), cos[:7].cpu()[None, None], sin[:7].cpu()[None, None])
    assert torch.allclose(y.cpu().float(), want.float(), atol=2e-3)
    pos = torch.tensor([[3, 9, 100, 5, 6, 7, 30000], [0, 1, 2, 3, 4, 5, 6]], device="cuda")
    y2 = K.rope().forward(x, cos[pos].contiguous(), sin[pos].contiguous())
    want2 = quic_ref.rope(x.cpu(), cos[pos].cpu()[:, None], sin[pos].cpu()[:, None])
    assert torch.allclose(y2.cpu().float(), want2.float(), atol=2e-3)


def test_qkv_rope_append_matches_split_rope_and_cache_update(K):
    """Prefill form: one kernel instead of the reference's _heads + rope.forward x2 +
    DynamicCache.update (src/model.py:138-160).  Stored columns hold rotation pairs side by
    side inside every head; tokens of two sequences go to different slots."""
    torch.manual_seed(3)
    exponent = torch.arange(0, 64, 2, dtype=torch.float32) / 64
    cos, sin = K.rope().init_table((1.0 / (1e6 ** exponent)).cuda(), 4096)
    lens, slots = [37, 5], [3, 0]
    rows = sum(lens)
    qkv = torch.randn(rows, 1152, device="cuda", dtype=torch.float16)
    pos = torch.cat([torch.arange(n, dtype=torch.int32) for n in lens]).cuda()
    slot_of = torch.repeat_interleave(torch.tensor(slots, dtype=torch.int32), torch.tensor(lens)).cuda()
    kc = torch.zeros(4, 2, 64, 64, device="cuda", dtype=torch.float16)
    vc = torch.zeros_like(kc)
    q = K.qkv_rope_append(qkv, slot_of, pos, cos, sin, kc, vc)
    assert q.shape == (14, rows, 64)
    natural = qkv.cpu().view(rows, 18, 32, 2).transpose(2, 3).reshape(rows, 18, 64)
    c, s_ = cos.cpu()[pos.cpu().long()][:, None], sin.cpu()[pos.cpu().long()][:, None]
    rotated = quic_ref.rope(natural[:, :16], c, s_)  # [rows, 16, 64]
    # fp32 rotation with or without a fused multiply-add: at most one fp16 ulp apart
    assert torch.allclose(q.cpu().float(), rotated[:, :14].transpose(0, 1).float(), atol=2e-3, rtol=1e-3)
    start = 0
    for n, slot in zip(lens, slots):
        assert torch.allclose(kc[slot, :, :n].cpu().float(), rotated[start:start + n, 14:16].transpose(0, 1).float(),
                              atol=2e-3, rtol=1e-3)
        assert torch.equal(vc[slot, :, :n].cpu(), natural[start:start + n, 16:18].transpose(0, 1))
        assert torch.count_nonzero(kc[slot, :, n:]) == 0
        start += n
    assert torch.count_nonzero(kc[1]) == 0 and torch.count_nonzero(vc[2]) == 0


def test_rows_with_slots_outside_the_cache_append_nothing(K):
    """A row whose slot is not one of the cache's (or whose position is negative) still gets
    its query written, but nothing is appended for it and the rows of a sequence in such a slot
    are skipped by the prefill attention; the valid rows are unaffected."""
    torch.manual_seed(4)
    exponent = torch.arange(0, 64, 2, dtype=torch.float32) / 64
    cos, sin = K.rope().init_table((1.0 / (1e6 ** exponent)).cuda(), 4096)
    n_slots, rows = 3, 6
    qkv = torch.randn(rows, 1152, device="cuda", dtype=torch.float16)
    slot_of = torch.tensor([1, 1, 3, -1, 1000, 2], dtype=torch.int32, device="cuda")
    pos = torch.tensor([0, 1, 0, 0, 0, -1], dtype=torch.int32, device="cuda")
    # the planes sit inside a larger zeroed block, so a stray write would land where it is seen
    block = torch.zeros(n_slots + 4, 2, 16, 64, device="cuda", dtype=torch.float16)
    vblock = torch.zeros_like(block)
    kc, vc = block[:n_slots], vblock[:n_slots]
    q = K.qkv_rope_append(qkv, slot_of, pos, cos, sin, kc, vc)
    good = torch.zeros_like(kc)
    q_ref = K.qkv_rope_append(qkv[:2].contiguous(), slot_of[:2].contiguous(), pos[:2].contiguous(), cos, sin, good,
                              torch.zeros_like(vc))
    assert torch.equal(q[:, :2], q_ref) and torch.isfinite(q).all()
    assert torch.equal(kc, good)
    assert torch.count_nonzero(block[n_slots:]) == 0 and torch.count_nonzero(vblock[n_slots:]) == 0
    assert torch.count_nonzero(kc[0]) == 0 and torch.count_nonzero(kc[2]) == 0

    dev = dict(device="cuda", dtype=torch.int32)
    out = K.attn_prefill(q[:, :4].contiguous(), kc, vc, torch.tensor([0, 2], **dev), torch.tensor([2, 2], **dev),
                         torch.tensor([1, 7], **dev), 2)
    want = K.attn_prefill(q[:, :2].contiguous(), kc, vc, torch.tensor([0], **dev), torch.tensor([2], **dev),
                          torch.tensor([1], **dev), 2)
    assert torch.equal(out[:2], want)


def test_errors_are_runtime_errors(K):
    with pytest.raises(RuntimeError):
        K.rmsnorm().forward(torch.zeros(2, 896, dtype=torch.float16), torch.ones(896, dtype=torch.float16), 1e-6)
    with pytest.raises(RuntimeError):
        K.swiglu().forward(torch.zeros(2, 100, device="cuda", dtype=torch.float16),
                           torch.zeros(2, 100, device="cuda", dtype=torch.float16))
    with pytest.raises(RuntimeError):
        K.sampler().forward(torch.zeros(2, 2, 10, device="cuda", dtype=torch.float16))
