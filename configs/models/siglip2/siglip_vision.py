"""SigLIP2 vision encoders (bidirectional ViT, LayerNorm, GELU-tanh MLP, learned positions)."""

from torch import nn

from halite_b200.conf import call, field, function
from halite_b200.models.embedding import PatchEmbedding
from halite_b200.models.position import LearnedPositionEmbedding

from ..transformer import transformer
from .checkpoint_vision import to_halite_postprocess, weight_maps


def vision_config(dim, n_heads, n_layers, intermediate_size, image_size, patch_size, use_conv=True, qkv_split=True):
    context_len = (image_size // patch_size) ** 2
    return field(
        vocab_size=0, dim=dim, n_heads=n_heads, head_dim=dim // n_heads, n_layers=n_layers, context_len=context_len,
        intermediate_size=intermediate_size, norm=nn.LayerNorm(dim, eps=1e-6), pos_embed=None, attention_bias=True,
        is_causal=False, ffn_bias=True, ffn_activation="gelu_tanh",
        embedding=PatchEmbedding(3, dim, patch_size, LearnedPositionEmbedding(dim, context_len), use_bias=True,
                                 use_conv=use_conv),
        qkv_split=qkv_split, use_head=False)


def _named(cfg, **extra):
    conf = field()
    conf.model = call[transformer](**cfg)
    conf.model_conf = field(**{k: v for k, v in cfg.items() if k not in ("norm", "embedding", "pos_embed")},
                            dtype="bfloat16", **extra)
    conf.policy = field(weight_maps=weight_maps, to_halite_postprocess=function(to_halite_postprocess))
    return conf


def siglip2_large_patch16_256():
    return _named(vision_config(1024, 16, 24, 4096, 256, 16), use_conv=True)


def siglip2_so400m_patch14_896():
    return _named(vision_config(1152, 16, 27, 4304, 896, 14), use_conv=True)


conf = siglip2_large_patch16_256()
