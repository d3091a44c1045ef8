from .activation import GEGLU, BloomGELU, SwiGLU
from .init import kaiming_linear_, kaiming_normal_, normal_
from .loss import CrossEntropyLoss
from .normalization import L2Norm, LayerNorm, RMSNorm

__all__ = ["GEGLU", "BloomGELU", "SwiGLU", "kaiming_linear_", "kaiming_normal_", "normal_",
           "CrossEntropyLoss", "L2Norm", "LayerNorm", "RMSNorm"]
