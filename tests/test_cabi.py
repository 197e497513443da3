"""The C-ABI library loads and exports every function include/quic_b200.h declares
(no compute calls: this runs without a GPU)."""

import ctypes
import os
import re

from quic_cu_b200 import kernels as K

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "quic_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(quic_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    names = _declared()
    assert len(names) >= 20
    handle = ctypes.CDLL(K.LIB_PATH)
    for name in names:
        assert hasattr(handle, name), f"{name} declared in the header but not exported"
        assert name in K.SIGNATURES, f"{name} has no ctypes signature"
    assert sorted(K.SIGNATURES) == names


def test_host_only_queries():
    lib = K.lib()
    assert lib.quic_abi_version() == 1
    assert lib.quic_attn_pick_splits(1, 128) == 2
    assert lib.quic_attn_pick_splits(1, 64) == 1
    assert lib.quic_attn_pick_splits(1, 32768) == 64
    assert lib.quic_attn_pick_splits(256, 32768) == 3
    assert lib.quic_attn_pick_splits(4096, 32768) == 1
    assert lib.quic_attn_scratch_bytes(4, 8) > 4 * 14 * 8 * 64 * 4
    assert lib.quic_decode_scratch_bytes(1, 151936, 4) > 0
    assert lib.quic_w4a16_workspace_bytes(1, 896, 4864) >= 896 * 4
    # fused prefill arena: grows with the rows, holds at least the gate|up activations
    small, big = lib.quic_prefill_scratch_bytes(128, 1, 151936), lib.quic_prefill_scratch_bytes(4096, 8, 151936)
    assert 128 * 9728 * 2 < small < big and big > 4096 * 9728 * 2
    assert lib.quic_prefill_scratch_bytes(0, 1, 151936) == 0
    # decode split policy: one warp per 64 tokens on the small-batch chain and on the tensor step up to 2048 tokens
    assert lib.quic_decode_pick_splits(1, 640) == 10
    assert lib.quic_decode_pick_splits(64, 768) == 12
    assert 1 <= lib.quic_decode_pick_splits(64, 8192) <= 64


def test_struct_sizes_match_the_header():
    assert ctypes.sizeof(K.W4) == 48  # four pointers, two ints, the dense-weight pointer
    assert ctypes.sizeof(K.Layer) == 4 * 48 + 16
    assert ctypes.sizeof(K.Model) == 56
    assert ctypes.sizeof(K.Decode) == 96
    assert ctypes.sizeof(K.Prefill) == 128


def test_argument_errors_are_reported_without_a_gpu():
    import pytest

    lib = K.lib()
    rc = lib.quic_rmsnorm(None, None, None, 1e-6, None, None, 4, None)
    assert rc == -1 and b"null" in lib.quic_last_error()
    with pytest.raises(RuntimeError):
        K.check(rc, "rmsnorm")
    assert lib.quic_gemm_f16(8, 8, None, 8, 1, 16, 7, None) == -2  # K not a multiple of 8
