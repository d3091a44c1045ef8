from .attention import Attention, DiffAttention, SelfAttention, SelfAttentionQKV
from .block import FusedTransformerEncoderBlock, NGPTBlock, ResidualBlock, TransformerEncoderBlock
from .config import TransformerConfig
from .embedding import MultiModalEmbedding, PatchEmbedding, TextEmbedding
from .feedforward import (FeedForward, FusedLinearCrossEntropy, GatedFeedForward, SequenceParallelWrapper,
                          VocabParallelLinear)
from .position import ALiBi, LearnedPositionEmbedding, LinearRoPE, Llama3RoPE, RotaryEmbedding, apply_rotary_emb
from .transformer import TransformerDecoder
from .types import TransformerDecoderOutput, UnpadParams
