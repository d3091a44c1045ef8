"""Training criterion (reference: nn/loss.py:12-106): cross entropy in fp32 with optional
z-loss, micro-averaging and a loss dictionary for logging."""

from __future__ import annotations

from torch import nn

from halite_b200 import ops


class CrossEntropyLoss(nn.Module):
    def __init__(self, ignore_index=-100, z_loss=0.0, fast=False, micro_average=True, softcap=0.0,
                 label_smoothing=0.0):
        super().__init__()
        self.ignore_index = ignore_index
        self.z_loss = z_loss
        self.fast = fast
        self.micro_average = micro_average
        self.softcap = softcap
        self.label_smoothing = label_smoothing

    def forward(self, input, target, inplace=False):
        """input [..., V] logits, target [...] ids -> (loss, loss_dict)."""
        logits = input.reshape(-1, input.shape[-1])
        tgt = target.reshape(-1)
        rows, z_rows, _ = ops.cross_entropy_rows(logits, tgt, self.ignore_index, self.z_loss,
                                                 self.softcap, 1.0, self.label_smoothing, inplace)
        n_targets = (tgt != self.ignore_index).sum()
        if self.micro_average:
            denom = n_targets.clamp(min=1).to(rows.dtype)
            loss = rows.sum() / denom
            z = z_rows.sum() / denom
        else:
            # mean over tokens of each sequence, then over sequences
            r = rows.view(target.shape)
            valid = (target != self.ignore_index).to(rows.dtype)
            per_seq = r.sum(-1) / valid.sum(-1).clamp(min=1)
            loss = per_seq.mean()
            z = (z_rows.view(target.shape).sum(-1) / valid.sum(-1).clamp(min=1)).mean()
        loss_dict = {"cross entropy": (loss - z).detach(), "n_targets": n_targets}
        if self.z_loss > 0:
            loss_dict["z-loss"] = z.detach()
        return loss, loss_dict
