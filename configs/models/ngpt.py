"""nGPT: every hidden vector and weight row lives on the unit hypersphere; residual updates are
learned interpolations (reference: configs/models/ngpt.py:26-121). Pair with the
`ngpt_normalize` post-step hook."""

from copy import deepcopy
from functools import partial

from torch import nn

from halite_b200.conf import call, config_fn, field
from halite_b200.models.attention import Attention, SelfAttentionQKV
from halite_b200.models.block import NGPTBlock, TransformerEncoderBlock
from halite_b200.models.embedding import TextEmbedding
from halite_b200.models.feedforward import GatedFeedForward, VocabParallelLinear
from halite_b200.models.normalization import L2Norm, LinearLayer, Scale
from halite_b200.models.position import RotaryEmbedding, apply_rotary_emb
from halite_b200.models.transformer import TransformerDecoder


@config_fn
def ngpt(vocab_size, dim, n_heads, n_layers, intermediate_size, max_position_embeddings, softcap=0.0,
         attention_processor="native"):
    init = partial(nn.init.kaiming_normal_, nonlinearity="linear")
    attention = Attention(n_heads, dim // n_heads, attn_drop=0, apply_pos_emb_fn=partial(apply_rotary_emb),
                          processor=attention_processor, softcap=softcap, is_causal=True, normalize=dim ** 0.5)
    l2norm = L2Norm()
    step = Scale(dim, 1 / n_layers, dim ** -0.5, apply_abs=True)
    block = TransformerEncoderBlock(
        NGPTBlock(
            SelfAttentionQKV(q=nn.Linear(dim, dim, bias=False), k=nn.Linear(dim, dim, bias=False),
                             v=nn.Linear(dim, dim, bias=False), attention=attention,
                             out=nn.Linear(dim, dim, bias=False), scaler=Scale(dim, 1, dim ** -0.5),
                             q_init=init, k_init=init, v_init=init, out_init=init),
            post_norm=l2norm, skip_norm=l2norm, scale=deepcopy(step)),
        NGPTBlock(
            GatedFeedForward(
                LinearLayer(nn.Linear(dim, intermediate_size, bias=False), Scale(intermediate_size, 1, 1)),
                LinearLayer(nn.Linear(dim, intermediate_size, bias=False), Scale(intermediate_size, 1, 1, dim ** 0.5)),
                nn.SiLU(), nn.Linear(intermediate_size, dim, bias=False),
                linear_proj_init=init, linear_gate_init=init, linear_out_init=init),
            post_norm=l2norm, skip_norm=l2norm, scale=deepcopy(step)))
    return TransformerDecoder(
        embedding=TextEmbedding(nn.Embedding(vocab_size, dim), 0, embed_init=init),
        pos_embed=RotaryEmbedding(dim // n_heads, max_position_embeddings),
        blocks=[deepcopy(block) for _ in range(n_layers)],
        head=VocabParallelLinear(LinearLayer(nn.Linear(dim, vocab_size, bias=False), Scale(vocab_size, 1, dim ** -0.5)),
                                 linear_init=init),
        tie_embeds=False, use_position_ids=True, attention_processor=attention_processor)


conf = field(model=call[ngpt](32000, 96, 4, 3, call[int](96 * 3.5), 2048, 1e-6))
