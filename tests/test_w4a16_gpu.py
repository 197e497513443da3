"""W4A16: bit-exact unpack/dequant and the linear op at the model's four shapes."""

import os

import numpy as np
import pytest
import torch

from oracle import quic_ref

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
SHAPES = {"qkv": (896, 1152), "o_proj": (896, 896), "gate_up": (896, 9728), "down": (4864, 896)}  # K x N


def _layer(k, n, seed):
    from quic_cu_b200 import kernels as K
    from quic_cu_b200.checkpoint import synthetic_layer

    layer = synthetic_layer(n, k, torch.Generator().manual_seed(seed))
    w = K.W4Weight(n, k, "cuda")
    w.put(layer["weight_packed"], layer["weight_scale"], layer["weight_zero_point"])
    w16 = quic_ref.dequantize_f16(layer["weight_packed"].numpy(), layer["weight_scale"].numpy(),
                                  layer["weight_zero_point"].numpy())
    return w, torch.from_numpy(w16)


@pytest.mark.parametrize("tag", ["a", "b"])
def test_dequant_bit_exact_vs_reference_golden(tag):
    """The device unpack reproduces the reference's dequantize (golden from its own code),
    rounded once to fp16, bit for bit."""
    from quic_cu_b200 import kernels as K

    g = np.load(os.path.join(GOLDEN, f"dequant_{tag}.npz"))
    n, k = g["reference"].shape
    w = K.W4Weight(n, k, "cuda")
    w.put(torch.from_numpy(g["weight_packed"]), torch.from_numpy(g["weight_scale"]),
          torch.from_numpy(g["weight_zero_point"]))
    got = w.dequant().cpu().numpy()
    assert np.array_equal(got.view(np.uint16), g["reference"].astype(np.float16).view(np.uint16))


@pytest.mark.parametrize("name", list(SHAPES))
def test_dequant_bit_exact_model_shapes(name):
    k, n = SHAPES[name]
    w, w16 = _layer(k, n, seed=n + k)
    assert torch.equal(w.dequant().cpu().view(torch.int16), w16.view(torch.int16))


@pytest.mark.parametrize("name", list(SHAPES))
@pytest.mark.parametrize("m", [1, 4, 16, 64, 256])
def test_linear_matches_oracle(name, m):
    """The linear-op sweep of the benchmark configuration: fp16 N(0,1) activations."""
    from quic_cu_b200 import kernels as K

    k, n = SHAPES[name]
    w, w16 = _layer(k, n, seed=7)
    x = torch.randn(m, k, generator=torch.Generator().manual_seed(m)).half()
    bias = (torch.randn(n, generator=torch.Generator().manual_seed(3)) * 0.02).half() if name == "qkv" else None
    w.bias = bias.cuda() if bias is not None else None
    y = K.w4a16_linear(w, x.cuda())
    want = quic_ref.w4a16_linear(x, w16, bias)
    # fp32 accumulation on both sides; outputs are fp16 of magnitude ~sqrt(K)*0.06
    assert torch.allclose(y.cpu().float(), want.float(), rtol=2e-3, atol=2e-2), \
        (y.cpu().float() - want.float()).abs().max()


def test_linear_is_linear_in_x():
    """Size-independent property at the largest shape: f(x1) + f(x2) == f(x1 + x2) up to fp16."""
    from quic_cu_b200 import kernels as K

    w, _ = _layer(4864, 896, seed=11)
    g = torch.Generator().manual_seed(0)
    x1, x2 = torch.randn(8, 4864, generator=g).half().cuda(), torch.randn(8, 4864, generator=g).half().cuda()
    lhs = K.w4a16_linear(w, x1).float() + K.w4a16_linear(w, x2).float()
    rhs = K.w4a16_linear(w, (x1.float() + x2.float()).half()).float()
    assert torch.allclose(lhs, rhs, rtol=5e-3, atol=8e-2)


def test_rope_pair_row_order_is_a_permutation():
    from quic_cu_b200 import kernels as K
    from quic_cu_b200.checkpoint import synthetic_layer

    layer = synthetic_layer(128, 896, torch.Generator().manual_seed(2))
    nat, per = K.W4Weight(128, 896, "cuda"), K.W4Weight(128, 896, "cuda")
    nat.put(layer["weight_packed"], layer["weight_scale"], layer["weight_zero_point"])
    per.put(layer["weight_packed"], layer["weight_scale"], layer["weight_zero_point"],
            row_order=K.ROWS_ROPE_PAIRS)
    a, b = nat.dequant(), per.dequant()
    # stored row r of a head holds source row (r // 2) + 32 * (r % 2)
    src = torch.arange(128).view(2, 32, 2)
    src = (torch.arange(2)[:, None, None] * 64 + torch.arange(32)[None, :, None] + 32 * torch.arange(2)[None, None, :]).reshape(-1)
    assert torch.equal(b.cpu(), a.cpu()[src])
