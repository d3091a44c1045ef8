"""Schema of a diffusion-transformer run (reference: projects/dit/config.py)."""

from halite_b200.conf import Instance, MainConfig
from halite_b200.projects.common.config import Data, Model, Output, Training


class DiTTraining(Training):
    ema: float = 0.9999
    pretuning_epoch: int = 0
    pretuning_scheduler: Instance | None = None
    freeze_encoder: bool = False


class DiTOutput(Output):
    sampling_step: int


class DiTConfig(MainConfig):
    model: Model
    data: Data
    training: DiTTraining
    output: DiTOutput
