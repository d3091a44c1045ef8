"""Feed-forward blocks and output heads (reference: transformers/feedforward.py:16-225)."""

from __future__ import annotations

import torch
from torch import nn

from halite_b200 import ops
from halite_b200.models.initialize import init_weights
from halite_b200.nn.activation import GEGLU, SwiGLU
from halite_b200.ops.activation import gated_act, gated_act_packed


class FusedLinearCrossEntropy(nn.Module):
    """Head that returns the loss directly: the [tokens, vocab] logits are produced and
    consumed chunk by chunk (`ops.fused_linear_cross_entropy`)."""

    def __init__(self, linear, linear_init=None, ignore_index=-100, z_loss=0):
        super().__init__()
        self.linear = linear
        self.linear_init = linear_init
        self.ignore_index = ignore_index
        self.z_loss = z_loss
        self.tie_weight_key = "linear.weight"

    def init_weights(self):
        init_weights(self.linear, self.linear_init)

    def tie_weight(self, weight):
        self.linear.weight = weight

    @property
    def weight(self):
        return self.linear.weight

    def forward(self, input, target=None):
        if target is None:
            return ops.linear(input, self.linear.weight, self.linear.bias)
        losses, z_losses = ops.fused_linear_cross_entropy(
            input.reshape(-1, input.shape[-1]), self.linear.weight, target.reshape(-1),
            ignore_index=self.ignore_index, z_loss=self.z_loss)
        # mean over all positions, as the reference's head does (ignored rows contribute 0)
        loss = losses.mean()
        loss_dict = {"cross entropy": loss.detach()}
        if self.z_loss > 0:
            z = z_losses.detach().mean()
            loss_dict["z-loss"] = z
            loss_dict["cross entropy"] = (losses.detach() - z_losses.detach()).mean()
        return loss, loss_dict

    def tp_plan(self):
        return {"linear": "vocab_head"}


def _project(module, x):
    """A plain `nn.Linear` goes straight to the GEMM; a composite (e.g. a `LinearLayer` with a
    learned scale behind the linear) is called as a module."""
    if type(module) is nn.Linear:
        return ops.linear(x, module.weight, module.bias)
    return module(x)


class VocabParallelLinear(nn.Module):
    def __init__(self, linear, linear_init=None, scale=None):
        super().__init__()
        self.linear = linear
        self.linear_init = linear_init
        self.scale = None
        if scale:
            self.scale = nn.Parameter(torch.ones(self._lin().out_features))
        self.tie_weight_key = "linear.weight" if type(linear) is nn.Linear else "linear.0.weight"

    def init_weights(self):
        init_weights(self.linear, self.linear_init)
        if self.scale is not None:
            nn.init.ones_(self.scale)

    def _lin(self):
        """The projection itself (the head may be a `LinearLayer` = linear + learned scale)."""
        return self.linear if type(self.linear) is nn.Linear else self.linear[0]

    def forward(self, input):
        out = _project(self.linear, input)
        if self.scale is not None:
            out = out * self.scale
        return out

    def tie_weight(self, weight):
        self._lin().weight = weight

    @property
    def n_vocab(self):
        return self._lin().weight.shape[0]

    @property
    def weight(self):
        return self._lin().weight

    @property
    def bias(self):
        return self._lin().bias

    def tp_plan(self):
        return {"linear": "vocab_head"}


class SequenceParallelWrapper(nn.Module):
    """Marks a module (the final norm) as running on sequence-sharded activations under TP."""

    def __init__(self, module):
        super().__init__()
        self.module = module

    def forward(self, input, residual=None):
        if residual is not None:
            return self.module(input + residual)
        return self.module(input)

    def tp_plan(self):
        return {"module": "sequence"}


class FeedForward(nn.Module):
    """linear2(act(linear1(x))); with a gated activation, linear1 emits [gate | up]."""

    def __init__(self, linear1, activation, linear2, dropout=0, linear1_init=None, linear2_init=None):
        super().__init__()
        self.linear1 = linear1
        self.activation = activation
        self.dropout = nn.Dropout(dropout)
        self.linear2 = linear2
        self.linear1_init = linear1_init
        self.linear2_init = linear2_init

    def init_weights(self):
        init_weights(self.linear1, self.linear1_init)
        init_weights(self.linear2, self.linear2_init)

    def forward(self, input):
        tp = getattr(self, "_hb_tp", None)
        if tp is not None:
            from halite_b200.parallel.tensor_parallel import ag_linear, linear_rs

            x = input.reshape(-1, input.shape[-1])
            h, _ = ag_linear(x, self.linear1.weight, tp)
            out = linear_rs(self.activation(h), self.linear2.weight, tp)
            return out.view(1, -1, out.shape[-1])
        out = ops.linear(input, self.linear1.weight, self.linear1.bias)
        out = self.activation(out)
        out = self.dropout(out)
        if getattr(self, "_infer_tp", None) is not None:       # inference engine, row-parallel output
            from halite_b200.infer.tensor_parallel import row_parallel_linear

            return row_parallel_linear(self, out, self.linear2)
        return ops.linear(out, self.linear2.weight, self.linear2.bias)

    def tp_plan(self):
        gated = isinstance(self.activation, (SwiGLU, GEGLU))
        return {"linear1": "colwise_gated" if gated else "colwise", "linear2": "rowwise"}


class GatedFeedForward(nn.Module):
    """linear_out(linear_proj(x) * act(linear_gate(x)))."""

    def __init__(self, linear_proj, linear_gate, activation, linear_out, dropout=0,
                 linear_proj_init=None, linear_gate_init=None, linear_out_init=None):
        super().__init__()
        self.linear_proj = linear_proj
        self.linear_gate = linear_gate
        self.activation = activation
        self.dropout = nn.Dropout(dropout)
        self.linear_out = linear_out
        self.linear_proj_init = linear_proj_init
        self.linear_gate_init = linear_gate_init
        self.linear_out_init = linear_out_init

    def init_weights(self):
        init_weights(self.linear_proj, self.linear_proj_init)
        init_weights(self.linear_gate, self.linear_gate_init)
        init_weights(self.linear_out, self.linear_out_init)

    def fusable_linears(self):
        if not (isinstance(self.linear_proj, nn.Linear) and isinstance(self.linear_gate, nn.Linear)):
            return {}
        return {"proj_gate": ("linear_proj", "linear_gate")}

    def pack_weights(self):
        """Inference: copy [up | gate] into one matrix (the two parameters become views of it)
        so both projections are a single GEMM."""
        from torch import nn as _nn

        if not self.fusable_linears():
            return
        ws = [self.linear_proj.weight, self.linear_gate.weight]
        if self.linear_proj.bias is not None or self.linear_gate.bias is not None or ws[0].is_meta:
            return
        packed = torch.cat([w.detach() for w in ws], 0).contiguous()
        n = ws[0].shape[0]
        self.linear_proj.weight = _nn.Parameter(packed[:n], requires_grad=False)
        self.linear_gate.weight = _nn.Parameter(packed[n:], requires_grad=False)
        self._hb_fused = {"proj_gate": packed}

    def _act_kind(self):
        if isinstance(self.activation, nn.SiLU):
            return "silu"
        if isinstance(self.activation, nn.GELU) and self.activation.approximate == "tanh":
            return "gelu_tanh"
        return None

    def forward(self, input):
        kind = self._act_kind()
        fused = getattr(self, "_hb_fused", {}).get("proj_gate")
        tp = getattr(self, "_hb_tp", None)
        if tp is not None:
            from halite_b200.parallel.tensor_parallel import ag_linear, linear_rs

            x = input.reshape(-1, input.shape[-1])
            w = fused if fused is not None else torch.cat([self.linear_proj.weight, self.linear_gate.weight], 0)
            pg, _ = ag_linear(x, w, tp)
            if kind is not None:
                act = gated_act_packed(pg, kind, gate_first=False)
            else:
                proj, gate = pg.chunk(2, -1)
                act = proj * self.activation(gate)
            out = linear_rs(act, self.linear_out.weight, tp)
            return out.view(1, -1, out.shape[-1])
        if fused is not None and kind is not None and ops.use_sm100(input):
            # one GEMM for [up | gate], one pass for act(gate) * up
            pg = ops.linear(input, fused)
            out = gated_act_packed(pg, kind, gate_first=False)
        else:
            proj = _project(self.linear_proj, input)
            gate = _project(self.linear_gate, input)
            if kind is not None:
                out = gated_act(gate, proj, kind)
            else:
                out = proj * self.activation(gate)
        out = self.dropout(out)
        if getattr(self, "_infer_tp", None) is not None:       # inference engine, row-parallel output
            from halite_b200.infer.tensor_parallel import row_parallel_linear

            return row_parallel_linear(self, out, self.linear_out)
        return _project(self.linear_out, out)

    def tp_plan(self):
        return {"linear_proj": "colwise", "linear_gate": "colwise", "linear_out": "rowwise"}
