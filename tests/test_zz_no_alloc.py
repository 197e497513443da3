"""The allocation-free attention entry point (quic_attn_decode_noalloc).

Some users of the library call it from places where they cannot allocate device memory —
inside a latency-critical serving loop that must never trigger cudaMalloc's device-wide
synchronisation, or as a plug-in of a host runtime that hands out no allocator.  For them
the split-K partials live in an array built into the library instead of a scratch tensor.
This file checks, through the C ABI, that the variant returns what the ordinary entry
point returns, twice in a row (the array is shared and keeps old contents), and that
oversized requests are refused.  It sorts last so a fail-fast run has already covered
everything else.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu
ATOL = 1e-2  # tolerance of the attention tests


def _call_noalloc(K, q, k, v, pads, splits):
    b, s = q.shape[0], k.shape[2]
    out = torch.empty_like(q)
    rc = K.lib().quic_attn_decode_noalloc(K.ptr(q), K.ptr(k), K.ptr(v), 2 * s * 64, s * 64, K.ptr(pads), None,
                                          s, 0.125, K.ptr(out), b, splits, K.stream_ptr())
    return rc, out


def test_noalloc_matches_the_scratch_variant_twice_in_a_row():
    from quic_cu_b200 import kernels as K

    for case, (b, s, splits) in enumerate([(3, 1500, 5), (2, 4096, 0), (16, 700, 2)]):
        g = torch.Generator(device="cuda").manual_seed(100 + case)
        q = torch.randn((b, 14, 1, 64), device="cuda", generator=g).half()
        k = torch.randn((b, 2, s, 64), device="cuda", generator=g).half()
        v = torch.randn((b, 2, s, 64), device="cuda", generator=g).half()
        pads = torch.randint(0, s // 4 + 1, (b,), device="cuda", generator=g).int()
        want = K.flash_attn_decode().forward(q, k, v, 0.125, pads, splits=splits)
        for _ in range(2):
            rc, got = _call_noalloc(K, q, k, v, pads, splits)
            assert rc == 0, K.lib().quic_last_error()
            torch.cuda.synchronize()
            assert torch.allclose(got.float(), want.float(), atol=ATOL)
        # a different problem in between must not leak into the next call
        rc, _ = _call_noalloc(K, q[:1], k[:1, :, :300].contiguous(), v[:1, :, :300].contiguous(), pads[:1] * 0, 2)
        assert rc == 0
        rc, got = _call_noalloc(K, q, k, v, pads, splits)
        torch.cuda.synchronize()
        assert rc == 0 and torch.allclose(got.float(), want.float(), atol=ATOL)


def test_noalloc_refuses_requests_beyond_the_built_in_array():
    from quic_cu_b200 import kernels as K

    lib = K.lib()
    limit = lib.quic_attn_decode_noalloc_max_bytes()
    assert limit == 8 << 20
    b, s, splits = 64, 8192, 64
    assert lib.quic_attn_scratch_bytes(b, splits) > limit
    q = torch.zeros((b, 14, 1, 64), device="cuda", dtype=torch.float16)
    k = torch.zeros((b, 2, s, 64), device="cuda", dtype=torch.float16)
    rc, _ = _call_noalloc(K, q, k, k, torch.zeros(b, device="cuda", dtype=torch.int32), splits)
    assert rc == -4 and b"8 MiB" in lib.quic_last_error()
    rc, out = _call_noalloc(K, q, k, k, torch.zeros(b, device="cuda", dtype=torch.int32), 16)
    torch.cuda.synchronize()
    assert rc == 0 and torch.count_nonzero(out) == 0
