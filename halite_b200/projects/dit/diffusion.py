"""Flow-matching objective with x-prediction and its ODE samplers
(reference: projects/dit/diffusion.py:6-182).

Path z_t = t x + (1 - t) e, t ~ sigmoid(N(p_mean, p_std)); the network predicts x, the loss is on
the implied velocity v = (x - z_t) / (1 - t). Sampling integrates dz/dt = v from noise (t = 0)
to data (t = 1) with Euler or Heun steps and classifier-free guidance applied only inside
`guidance_interval`.
"""

from __future__ import annotations

import torch
from torch import nn
from torch.nn import functional as F


class Diffusion(nn.Module):
    def __init__(self, input_shape, n_labels, steps=50, method="heun", guidance_interval=(0.0, 1.0),
                 guidance_scale=1.0, label_drop_p=0.1, p_mean=-0.8, p_std=0.8, noise_scale=1.0, eps_t=5e-2):
        super().__init__()
        self.input_shape, self.n_labels = tuple(input_shape), n_labels
        self.steps, self.method = steps, method
        self.guidance_interval, self.guidance_scale = guidance_interval, guidance_scale
        self.label_drop_p, self.p_mean, self.p_std = label_drop_p, p_mean, p_std
        self.noise_scale, self.eps_t = noise_scale, eps_t

    # ------------------------------------------------------------------ training
    def sample_t(self, batch, device=None):
        return torch.sigmoid(torch.randn(batch, device=device) * self.p_std + self.p_mean)

    def drop_labels(self, labels):
        drop = torch.rand(labels.shape[0], device=labels.device) < self.label_drop_p
        return torch.where(drop, torch.full_like(labels, self.n_labels), labels)

    def _coefficient(self, t):
        return 1.0

    def _net_time(self, t):
        return t.flatten()

    def loss(self, fn, input, labels=None, **forward_kwargs):
        if labels is not None and self.training:
            labels = self.drop_labels(labels)
        t = self.sample_t(input.shape[0], input.device).view(-1, *([1] * (input.ndim - 1)))
        noise = torch.randn_like(input) * self.noise_scale
        z = t * input + (1 - t) * noise
        c = self._coefficient(t)
        denom = (1 - t).clamp_min(self.eps_t)
        v = c * (input - z) / denom
        x_pred = fn(z, self._net_time(t), labels, **forward_kwargs).float()
        return F.mse_loss((x_pred - c * z) / denom, v)

    # ------------------------------------------------------------------ sampling
    def _velocity(self, fn, z, t, labels, **forward_kwargs):
        c = self._coefficient(t)
        denom = (1 - t).clamp_min(self.eps_t)
        v_cond = (fn(z, self._net_time(t), labels, **forward_kwargs).float() - c * z) / denom
        if self.guidance_scale == 1.0:
            return v_cond
        v_unc = (fn(z, self._net_time(t), torch.full_like(labels, self.n_labels)).float() - c * z) / denom
        low, high = self.guidance_interval
        inside = (t < high) & ((low == 0) | (t > low))
        w = torch.where(inside, self.guidance_scale, 1.0)
        return v_unc + w * (v_cond - v_unc)

    _forward_fn = _velocity

    def _euler_step(self, fn, z, t, t_next, labels, **kw):
        return z + (t_next - t) * self._velocity(fn, z, t, labels, **kw)

    def _heun_step(self, fn, z, t, t_next, labels, **kw):
        v0 = self._velocity(fn, z, t, labels, **kw)
        v1 = self._velocity(fn, z + (t_next - t) * v0, t_next, labels, **kw)
        return z + (t_next - t) * 0.5 * (v0 + v1)

    @torch.no_grad()
    def generate(self, fn, labels, seed=None, **forward_kwargs):
        device, batch = labels.device, labels.shape[0]
        gen = torch.Generator(device=device).manual_seed(seed) if seed is not None else None
        z = self.noise_scale * torch.randn(batch, *self.input_shape, generator=gen, device=device)
        shape = (batch, *([1] * len(self.input_shape)))
        ts = torch.linspace(0, 1, self.steps + 1, device=device)
        if self.method not in ("euler", "heun"):
            raise NotImplementedError(f"Method {self.method} not implemented")
        step = self._euler_step if self.method == "euler" else self._heun_step
        for i in range(self.steps - 1):
            z = step(fn, z, ts[i].expand(shape), ts[i + 1].expand(shape), labels, **forward_kwargs)
        # the last step ends at t = 1 where the velocity is singular: plain Euler
        return self._euler_step(fn, z, ts[-2].expand(shape), ts[-1].expand(shape), labels)


class EquilibriumMatchingJiT(Diffusion):
    """Time-unconditional variant: the network never sees t (it is fed 0) and the target
    velocity is scaled by a fixed schedule c(t) that decays to zero at the data end."""

    def get_c_t(self, t, interp=0.8, start=1.0):
        return torch.minimum(start - (start - 1) / interp * t, 1 / (1 - interp) - 1 / (1 - interp) * t) * 4

    def _coefficient(self, t):
        return self.get_c_t(t)

    def _net_time(self, t):
        return t.flatten() * 0
