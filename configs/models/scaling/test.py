"""Smoke script: build `scale_1` with a 128-token vocabulary on CPU and run one forward.
`python configs/models/scaling/test.py`."""

import os

import torch

from halite_b200.conf import instantiate, load_config

if __name__ == "__main__":
    conf = load_config(os.path.join(os.path.dirname(os.path.abspath(__file__)), "scale_1.py"))
    model = instantiate(conf.model, _tags_={"n_vocab": 128})
    model.init_weights("cpu")
    out = model(torch.tensor([[1, 2, 3], [4, 5, 6]]))
    print(out.logits.shape)
