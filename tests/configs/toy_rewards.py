"""Toy reward functions for the RL entry-point tests."""

import torch


class FractionOfLetter:
    """Reward of a sample = share of its characters equal to `letter`."""

    def __init__(self, letter):
        self.letter = letter

    def __call__(self, texts):
        return torch.tensor([t.count(self.letter) / max(len(t), 1) for t in texts], dtype=torch.float32)
