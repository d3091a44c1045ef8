import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 box)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def repo_root():
    return ROOT


@pytest.fixture(scope="session")
def zoo():
    from halite_b200.conf.loader import load_module

    return load_module(os.path.join(ROOT, "configs/models/transformer.py"))


def tiny_llama_conf(zoo, **over):
    """Tiny Llama-style decoder: dim 256, 4 layers, 4 query / 2 KV heads, SwiGLU 688, vocab 1024."""
    from functools import partial

    import torch

    kw = dict(vocab_size=1024, dim=256, n_heads=4, head_dim=64, n_layers=4, intermediate_size=688,
              context_len=512, n_key_value_heads=2, rms_norm_epsilon=1e-5, qkv_split=True,
              gated_ff_split=True, init=partial(torch.nn.init.normal_, std=0.02))
    kw.update(over)
    return zoo.transformer(**kw)
