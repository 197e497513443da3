"""Shared pytest setup: registers the ``gpu`` marker and loads the package."""

import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import __graft_entry__ as entry  # noqa: E402

entry.load_package()


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def tiny_model():
    """2-layer, vocab-2048 synthetic model on the GPU together with its CPU oracle."""
    import torch

    from oracle.quic_ref import RefModel
    from quic_cu_b200 import model as qmodel
    from quic_cu_b200.checkpoint import qwen_config_dict, synthetic_checkpoint

    state = synthetic_checkpoint(n_layers=2, vocab=2048, seed=1234)
    config = qwen_config_dict(2, 2048)
    net = qmodel.from_state_dict(state, config)
    torch.cuda.synchronize()
    return net, RefModel(state, 2), state, config
