import json
import os

import pytest
import torch

from halite_b200 import conf as C
from halite_b200.conf.node import FN, PARTIAL, TARGET


def write(tmp_path, name, text):
    p = tmp_path / name
    p.parent.mkdir(parents=True, exist_ok=True)
    p.write_text(text)
    return str(p)


def test_field_and_lazy_record(tmp_path):
    path = write(tmp_path, "configs/a.py", """
from functools import partial
from halite_b200.conf import field, call
from torch import nn, optim

conf = field()
conf.layer = nn.Linear(4, 8, bias=False)
conf.opt = partial(optim.AdamW, lr=1e-3, betas=(0.9, 0.95))
conf.n = call[int](3.7)
conf.init = partial(nn.init.normal_, std=0.02)
""")
    conf = C.load_config(path)
    assert conf.layer[TARGET] == "torch.nn.modules.linear.Linear"
    assert conf.layer.in_features == 4 and conf.layer.out_features == 8 and conf.layer.bias is False
    assert conf.opt[PARTIAL] is True and conf.n == 3
    layer = C.instantiate(conf.layer)
    assert isinstance(layer, torch.nn.Linear) and layer.weight.shape == (8, 4)
    opt = C.instantiate(conf.opt)(layer.parameters())
    assert isinstance(opt, torch.optim.AdamW) and opt.defaults["betas"] == (0.9, 0.95)
    C.instantiate(conf.init)(layer.weight)
    # JSON round trip keeps tuples
    again = C.deserialize(json.dumps(conf.to_dict()))
    assert again.opt.betas == (0.9, 0.95)
    assert isinstance(C.instantiate(again.layer), torch.nn.Linear)


def test_relative_imports_config_fn_and_overrides(tmp_path):
    write(tmp_path, "configs/models/base.py", """
from halite_b200.conf import config_fn
from torch import nn

@config_fn
def mlp(dim, hidden, n):
    return nn.Sequential(*[nn.Linear(dim if i == 0 else hidden, hidden) for i in range(n)])
""")
    path = write(tmp_path, "configs/exp/run.py", """
from halite_b200.conf import field, call
from ..models.base import mlp

conf = field()
conf.hparams = field(dim=8, lr=0.5)
conf.model = call[mlp](conf.hparams.dim, 16, 2)
conf.training = field(lr=conf.hparams.ref.lr, half=conf.hparams.ref.lr / 2, steps=100 // conf.hparams.ref.dim)

def small():
    conf.model = call[mlp](4, 4, 1)
    return conf
""")
    conf = C.load_config(path, overrides=["hparams.lr=0.25", "training.extra=[1,2]"])
    assert conf.training.lr == 0.25 and conf.training.half == 0.125 and conf.training.steps == 12
    assert conf.training.extra == [1, 2]
    model = C.instantiate(conf.model)
    assert isinstance(model, torch.nn.Sequential) and model[0].in_features == 8
    small = C.load_config(path, config_name="small")
    assert C.instantiate(small.model)[0].in_features == 4


def test_tags_annotate_function_external(tmp_path):
    path = write(tmp_path, "configs/t.py", """
from halite_b200.conf import field, tag, annotate, function, external
from torch import nn
import math

class Local:
    def __init__(self, v):
        self.v = v

def helper(x):
    return x + 1

conf = field()
conf.emb = nn.Embedding(tag("n_vocab"), 8)
conf.lin = nn.Linear(annotate("in_features", 3), 5)
conf.fn = function(helper)
conf.local = external[Local](v=7)
conf.pi = math.pi
""")
    conf = C.load_config(path)
    emb = C.instantiate(conf.emb, _tags_={"n_vocab": 11})
    assert emb.num_embeddings == 11
    with pytest.raises(KeyError):
        C.instantiate(conf.emb)
    assert C.instantiate(conf.lin).in_features == 3
    assert C.instantiate(conf.fn)(1) == 2
    assert C.instantiate(conf.local).v == 7
    assert abs(conf.pi - 3.14159) < 1e-4


def test_select_and_patch(zoo):
    from tests.conftest import tiny_llama_conf

    cfg = tiny_llama_conf(zoo, n_layers=2)
    from halite_b200.models.attention import Attention

    flash = zoo.use_flash_attention(cfg)
    procs = []

    def visit(n):
        if isinstance(n, dict):
            if n.get(TARGET, "").endswith("attention.Attention"):
                procs.append(n["processor"])
            for v in n.values():
                visit(v)
        elif isinstance(n, (list, tuple)):
            for v in n:
                visit(v)

    visit(flash)
    assert procs == ["flash_attn", "flash_attn"]
    procs.clear()
    visit(cfg)
    assert procs == ["auto", "auto"]        # the original is untouched
    fused = zoo.use_fused_linear_cross_entropy(cfg, z_loss=1e-4)
    assert fused.head[TARGET].endswith("FusedLinearCrossEntropy") and fused.head.z_loss == 1e-4
    assert fused.head.linear.out_features == 1024


def test_schema_and_arg_config(tmp_path):
    from pydantic import StrictInt

    class Train(C.Config):
        max_iter: StrictInt
        optimizer: C.Instance

    class Main(C.MainConfig):
        training: Train

    path = write(tmp_path, "configs/s.py", """
from functools import partial
from halite_b200.conf import field
from torch import optim
conf = field()
conf.training = field(max_iter=10, optimizer=partial(optim.SGD, lr=0.1))
conf.hparams = field(a=1)
""")
    conf = C.load_arg_config(Main, [path, "training.max_iter=20"])
    assert conf.training.max_iter == 20 and conf.hparams["a"] == 1 and conf.output is None
    opt = C.instantiate(conf.training.optimizer)([torch.nn.Parameter(torch.zeros(1))])
    assert isinstance(opt, torch.optim.SGD)
    text = C.summarize(conf)
    assert "SGD" in text and "max_iter" in text
    with pytest.raises(Exception):
        Main(training={"max_iter": "x", "optimizer": {}})


def test_shipped_experiment_configs_load_and_validate():
    """Every pre-training experiment under configs/lm validates against the LM schema and its
    model builds on the meta device with the expected parameter count."""
    import os

    import torch

    from halite_b200.conf import instantiate, load_config
    from halite_b200.projects.lm.config import LMConfig

    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "configs", "lm")
    expect = {"dense_662m.py": (0.55e9, 0.8e9), "dense_1.7b.py": (1.4e9, 2.0e9), "diff_transformer_383m.py": (0.3e9, 0.5e9),
              "moe_383m.py": (1.5e9, 5e9), "ngpt_383m.py": (0.3e9, 0.5e9), "scale_383m_soap.py": (0.3e9, 0.5e9),
              "scale_383m_shampoo.py": (0.3e9, 0.5e9),
              "dense_scaling.py": (0.3e9, 0.5e9), "diff_transformer_large.py": (0.8e9, 1.1e9),
              "scaling/scale_383m.py": (0.3e9, 0.5e9), "scaling/scale_large.py": (0.8e9, 1.1e9),
              "scaling/moe.py": (1.5e9, 5e9), "stacking/base_900m.py": (0.2e9, 0.4e9),
              "stacking/scratch_900m.py": (0.8e9, 1.0e9)}
    for name, (lo, hi) in expect.items():
        conf = load_config(os.path.join(root, name), schema=LMConfig)
        assert conf.training.train_batch_size == 320 and conf.data.preprocess is not None
        with torch.device("meta"):
            model = instantiate(conf.model.model)
        n = sum(p.numel() for p in model.parameters())
        assert lo < n < hi, (name, n)
    # hyper-parameter driven experiment: overrides of `hparams` reach every dependent value
    conf = load_config(os.path.join(root, "farseer.py"), "scale_202m", overrides=["hparams.batch_size=32"],
                       schema=LMConfig)
    assert conf.training.train_batch_size == 32 and conf.training.max_iter == 8192 * 10 ** 6 // 2048 // 32
    assert instantiate(conf.output.name)(conf.hparams).startswith("202m@lr-0.00781_batch-32")
    small = load_config(os.path.join(root, "scaling", "scale_1.py"), schema=LMConfig)
    assert small.training.train_batch_size == 64
    # data specs: one file per Nemotron-CC tier plus the 200B sample the MoE run trains on
    data_root = os.path.join(os.path.dirname(root), "data")
    tiers = {"high": "high", "medium_high": "medium-high", "medium": "medium", "medium_low": "medium-low", "low": "low"}
    for stem, source in tiers.items():
        assert dict(load_config(os.path.join(data_root, f"nemotron_cc_{stem}.py")).ratios) == {source: 1.0}
    moe = load_config(os.path.join(root, "scaling", "moe.py"), schema=LMConfig)
    assert dict(moe.data.train.ratios) == {"nemotron-cc": 1.0}
