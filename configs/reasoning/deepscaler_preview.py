"""GRPO on the DeepScaleR preview problems: the MATH recipe with the larger prompt set, no
evaluation split, and microbatches of 8 (reference: configs/reasoning/deepscaler_preview.py)."""

from halite_b200.conf import call

from ..data.deepscaler_preview import conf as data_conf
from . import math as math_recipe


def _retarget(conf):
    conf.data.train = data_conf
    conf.data.eval = None
    conf.training.ppo_microbatch_size = 8
    return conf


def qwen3_0_6b_grpo():
    return _retarget(call[math_recipe.qwen3_grpo]("/data/halite/qwen3-0.6b"))


def qwen3_8b_grpo():
    return _retarget(call[math_recipe.qwen3_grpo]("/data/halite/qwen3-8b"))
