"""Byte-level H-Net language models (reference: configs/lm/hnet.py).

`stage1_l`: one chunking stage; Mamba-2 encoder / decoder at width 1024 around a 22-layer
attention main network at width 1536.
"""

from halite_b200.conf import field

from ..models.hnet import hnet

conf = field()
conf.model = field()


def stage1_l():
    arch = [
        ({"mixer": "mamba2", "n_layer": 4, "use_ffn": False},),
        ({"mixer": "attention", "n_layer": 22, "use_ffn": True},),
        ({"mixer": "mamba2", "n_layer": 4, "use_ffn": False},),
    ]
    dims = [1024, 1536]
    conf.model.model = hnet(
        arch=arch,
        dims=dims,
        intermediate_sizes=[0, 4096],
        pos_dims=[32, 48],
        attn_kwargs=[
            {"n_heads": 16, "head_dim": dims[0] // 16, "is_causal": True},
            {"n_heads": 16, "head_dim": dims[1] // 16, "is_causal": True},
        ],
        mamba2_kwargs={"chunk_size": 256, "d_conv": 4, "d_state": 128, "expand": 2},
        vocab_size=256,
        context_len=2048,
        target_ratios=[6.0],
    )
    return conf


def stage2_tiny():
    """Two chunking stages at toy widths, for tests and smoke runs."""
    arch = [
        ({"mixer": "mamba2", "n_layer": 1, "use_ffn": False},),
        [
            ({"mixer": "mamba2", "n_layer": 1, "use_ffn": False},),
            ({"mixer": "attention", "n_layer": 2, "use_ffn": True},),
            ({"mixer": "mamba2", "n_layer": 1, "use_ffn": False},),
        ],
        ({"mixer": "mamba2", "n_layer": 1, "use_ffn": False},),
    ]
    dims = [32, 48, 64]
    conf.model.model = hnet(
        arch=arch,
        dims=dims,
        intermediate_sizes=[0, 0, 128],
        pos_dims=[8, 8, 8],
        attn_kwargs=[{"n_heads": 4, "head_dim": d // 4, "is_causal": True} for d in dims],
        mamba2_kwargs={"chunk_size": 16, "d_conv": 4, "d_state": 16, "expand": 2, "headdim": 16},
        vocab_size=256,
        context_len=256,
        target_ratios=[3.0, 3.0],
    )
    return conf
