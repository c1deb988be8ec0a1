"""Class-conditional latent Diffusion Transformer (DiT) with adaLN-Zero blocks on FP8 linears.

Architecture of the reference experiment model (experiments/dit.py:10-78: patch embedding by a
strided convolution, sinusoidal timestep features through a 2-layer MLP, a 1001-entry label table
whose last row is the unconditional class, fixed 2-D sin/cos position table, blocks with
LayerNorm(no affine) -> modulate -> attention / MLP gated by adaLN-Zero, zero-initialised adaLN and
output layers), generalised to any size: ``DiT.xl_2()`` is DiT-XL/2 (28 blocks, width 1152, 16
heads, patch 2), ``DiT.b_4()`` the reference's DiT-B/4.  The five matrices of every block
(qkv, proj, fc1, fc2, adaLN) are :class:`viola_b200.nn.Linear`; attention is PyTorch SDPA.
"""

from __future__ import annotations

import math

import torch
from torch import nn
from torch.nn import functional as F

from ..nn import Linear, gated_residual, norm_modulate_linear, norm_modulate_mlp
from ..nn.attention import packed_attention


def position_embedding(size, width):
    y, x = torch.meshgrid(torch.arange(size), torch.arange(size), indexing="ij")
    omega = 1 / 10000 ** (torch.arange(width // 4).float() / (width // 4))
    x, y = x.flatten()[:, None] * omega, y.flatten()[:, None] * omega
    return torch.cat((x.sin(), x.cos(), y.sin(), y.cos()), dim=-1)[None]


def modulate(x, shift, scale):
    """x * (1 + scale) + shift with per-sample vectors, as one fused multiply-add."""
    return torch.addcmul(shift[:, None], x, (1 + scale)[:, None])


class Block(nn.Module):
    def __init__(self, width, heads, mlp_ratio=4, linear_options=None):
        super().__init__()
        options = dict(linear_options or {})
        self.heads = heads
        self.norm1 = nn.LayerNorm(width, elementwise_affine=False, eps=1e-6)
        self.qkv = Linear(width, 3 * width, **options)
        self.proj = Linear(width, width, **options)
        self.norm2 = nn.LayerNorm(width, elementwise_affine=False, eps=1e-6)
        self.fc1 = Linear(width, mlp_ratio * width, **options)
        self.fc2 = Linear(mlp_ratio * width, width, **options)
        self.ada = Linear(width, 6 * width, **options)

    def forward(self, x, c, activated=None):
        """``activated`` = SiLU(c) when the caller computed it once for all blocks (it is the same for each)."""
        s1, a1, g1, s2, a2, g2 = self.ada(F.silu(c) if activated is None else activated).chunk(6, dim=-1)
        b, n, d = x.shape
        # LayerNorm + modulate are folded into the FP8 quantiser of qkv / fc1, GELU into that of fc2 (forward)
        # and into the fc2 dgrad epilogue (backward)
        # ``carry``: the residual connection takes x back from the fused function, so that its gradient is added
        # inside the LayerNorm backward kernel
        qkv, x = norm_modulate_linear(x, s1, a1, self.qkv, eps=self.norm1.eps, carry=True)
        h = packed_attention(qkv.view(b, n, 3, self.heads, d // self.heads))
        x = gated_residual(x, g1, self.proj(h))
        h, x = norm_modulate_mlp(x, s2, a2, self.fc1, self.fc2, "gelu", eps=self.norm2.eps, carry=True)
        return gated_residual(x, g2, h)


class DiT(nn.Module):
    def __init__(self, width=768, depth=12, heads=12, patch=4, *, latent=32, channels=4, classes=1000, mlp_ratio=4,
                 linear_options=None):
        super().__init__()
        self.patch, self.channels, self.classes = patch, channels, classes
        self.input = nn.Conv2d(channels, width, patch, stride=patch)
        self.time = nn.Sequential(nn.Linear(256, width), nn.SiLU(), nn.Linear(width, width))
        self.label = nn.Embedding(classes + 1, width)
        self.register_buffer("position", position_embedding(latent // patch, width))
        self.blocks = nn.ModuleList([Block(width, heads, mlp_ratio, linear_options) for _ in range(depth)])
        self.norm = nn.LayerNorm(width, elementwise_affine=False, eps=1e-6)
        self.final_ada = nn.Sequential(nn.SiLU(), nn.Linear(width, 2 * width))
        self.output = nn.Linear(width, patch * patch * channels)
        self.reset_parameters()

    @classmethod
    def xl_2(cls, **kwargs):
        return cls(width=1152, depth=28, heads=16, patch=2, **kwargs)

    @classmethod
    def b_4(cls, **kwargs):
        return cls(width=768, depth=12, heads=12, patch=4, **kwargs)

    @torch.no_grad()
    def reset_parameters(self):
        def init_linear(layer, zero=False):
            if isinstance(layer, Linear):
                master = layer.weight if layer.weight_dtype != "fp8" else layer._initial_weight
                nn.init.zeros_(master) if zero else nn.init.xavier_uniform_(master)
                nn.init.zeros_(layer.bias)
                layer.weight_quantizer.history.zero_()
                layer.weight_quantizer.index = 0
                layer.refresh_weight(master)
            else:
                nn.init.zeros_(layer.weight) if zero else nn.init.xavier_uniform_(layer.weight)
                nn.init.zeros_(layer.bias)

        for block in self.blocks:
            for layer in (block.qkv, block.proj, block.fc1, block.fc2):
                init_linear(layer)
            init_linear(block.ada, zero=True)
        nn.init.xavier_uniform_(self.input.weight.flatten(1))
        nn.init.zeros_(self.input.bias)
        nn.init.normal_(self.label.weight, std=0.02)
        for layer in (self.time[0], self.time[2]):
            nn.init.normal_(layer.weight, std=0.02)
            nn.init.zeros_(layer.bias)
        init_linear(self.final_ada[-1], zero=True)
        init_linear(self.output, zero=True)

    def timestep_features(self, t):
        freqs = torch.exp(-math.log(10000) * torch.arange(128, device=t.device).float() / 128)
        phase = t.float()[:, None] * freqs[None]
        return torch.cat((phase.cos(), phase.sin()), -1)

    def forward(self, x, t, y):
        """``x`` latents [B, C, H, W]; ``t`` timesteps in [0, 1000); ``y`` labels in [0, classes]."""
        c = self.time(self.timestep_features(t).to(x.dtype)) + self.label(y)
        # the residual stream stays in the input's dtype (fp32 under autocast, as in experiments/dit.py:72-75):
        # the fused block kernels read and write it as stored
        x = self.input(x).flatten(2).transpose(1, 2) + self.position.to(x.dtype)
        activated = F.silu(c)            # every block's modulation reads SiLU(c): one kernel instead of one per block
        if x.is_cuda and torch.is_autocast_enabled("cuda"):
            activated = activated.to(torch.get_autocast_dtype("cuda"))
        for block in self.blocks:
            x = block(x, c, activated)
        shift, scale = self.final_ada(c).chunk(2, -1)
        x = self.output(modulate(self.norm(x), shift, scale))
        b, n, _ = x.shape
        h, p = math.isqrt(n), self.patch
        return x.view(b, h, h, p, p, self.channels).permute(0, 5, 1, 3, 2, 4).reshape(b, self.channels, h * p, h * p)


class NoiseSchedule:
    """Linear-beta DDPM schedule for the epsilon-prediction objective: MSE between the model output and the noise."""

    def __init__(self, steps=1000, beta_start=1e-4, beta_end=2e-2, device=None):
        betas = torch.linspace(beta_start, beta_end, steps, dtype=torch.float64, device=device)
        alphas = torch.cumprod(1 - betas, dim=0)
        self.sqrt_alpha = alphas.sqrt().float()
        self.sqrt_one_minus_alpha = (1 - alphas).sqrt().float()

    def add_noise(self, latents, noise, timesteps):
        a = self.sqrt_alpha.to(latents.device)[timesteps][:, None, None, None]
        b = self.sqrt_one_minus_alpha.to(latents.device)[timesteps][:, None, None, None]
        return a * latents + b * noise


def diffusion_loss(model, schedule, latents, labels, timesteps, noise):
    noisy = schedule.add_noise(latents, noise, timesteps)
    return F.mse_loss(model(noisy, timesteps, labels).float(), noise.float())


def muon_parameter_groups(model, *, lr=1e-4, weight_decay=0.01):
    """Hidden block matrices -> Muon, everything else -> AdamW (experiments/train_dit.py:109-118)."""
    muon, adam = [], []
    for name, param in model.named_parameters():
        (muon if name.startswith("blocks.") and param.ndim == 2 else adam).append(param)
    return [dict(params=muon, use_muon=True, lr=lr, momentum=0.95, weight_decay=weight_decay, nesterov=True),
            dict(params=adam, use_muon=False, lr=lr, betas=(0.9, 0.95), eps=1e-8, weight_decay=weight_decay)]
