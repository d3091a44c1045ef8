"""Top-level schema of a language-model pre-training / SFT run (reference: projects/lm/config.py)."""

from halite_b200.conf import MainConfig
from halite_b200.projects.common.config import Data, Model, Output, Training


class LMConfig(MainConfig):
    model: Model
    data: Data
    training: Training
    output: Output
