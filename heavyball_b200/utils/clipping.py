"""Norm clips and amplitude compressors applied to gradients (``gradient_clipping=``) or updates
(``update_clipping=``).  Every function takes a tensor or list of tensors, works in fp32, stores with
stochastic rounding and returns the list, so they can be named by string in optimizer constructors.

Behavioural parity targets: ``heavyball/utils.py:3226-3373`` (clips, compressors) and
``heavyball/utils.py:3437-3455`` (trust region).
"""

from __future__ import annotations

import math

import torch

from .core import copy_stochastic_, list_guard, promote


def _rescale_to(x, norm, clip_at, eps=1e-8):
    # (x / max(norm, eps)) clipped to clip_at  ==  x * clip_at / max(norm, clip_at, eps)
    x32 = promote(x)
    copy_stochastic_(x, x32 * (clip_at / norm.clamp(min=max(clip_at, eps))))


def l2_clip_(x, clip_at: float = 1.0):
    x = list_guard(x)
    for t in x:
        _rescale_to(t, promote(t).norm(), clip_at)
    return x


def l2_normalization_(x, clip_at: float = 1e-8):
    return l2_clip_(x, clip_at)


def rmsnorm_clip_(x, clip_at: float = 1.0):
    x = list_guard(x)
    for t in x:
        _rescale_to(t, promote(t).square().mean().sqrt(), clip_at)
    return x


def rmsnorm_normalize_(x, clip_at: float = 1e-6):
    return rmsnorm_clip_(x, clip_at)


def _global_sq_sum(x):
    total = 0
    for t in x:
        total = total + promote(t).square().sum()
    return total


def global_l2norm_clip(x, clip_at: float = 1.0, eps: float = 1e-8):
    x = list_guard(x)
    scale = clip_at / (_global_sq_sum(x) ** 0.5).clamp(min=max(clip_at, eps))
    for t in x:
        copy_stochastic_(t, promote(t) * scale)
    return x


def global_rmsnorm_clip(x, clip_at: float = 1.0, eps: float = 1e-8):
    x = list_guard(x)
    numel = sum(t.numel() for t in x)
    scale = clip_at / ((_global_sq_sum(x) / numel) ** 0.5).clamp(min=max(clip_at, eps))
    for t in x:
        copy_stochastic_(t, promote(t) * scale)
    return x


def mu_law_compress(x, mu=127.0):
    """``sign(x) * log1p(mu |x|) / log1p(mu)``"""
    x = list_guard(x)
    for t in x:
        t32 = promote(t)
        copy_stochastic_(t, (t32.abs() * mu).log1p().div(math.log1p(mu)).copysign(t32))
    return x


def a_law_compress(x, A=87.6):
    """A-law companding: linear below ``1/A``, logarithmic above."""
    x = list_guard(x)
    for t in x:
        t32 = promote(t)
        xa = t32.abs() * A
        xa = torch.where(xa < 1, xa, 1 + xa.log()).copysign(t32)
        copy_stochastic_(t, xa * (1 / (1 + math.log(A))))
    return x


def softsign_compress(x):
    x = list_guard(x)
    for t in x:
        t32 = promote(t)
        copy_stochastic_(t, 2.0 * t32 / (1.0 + t32.abs()))
    return x


def trust_region_clip_(grad, lerp=0.9, scale=1.5):
    """Blend of ``tanh`` and signed ``log1p`` (weights ``lerp`` / ``1 - lerp``) at scale ``scale``,
    hard-limited to ±2: small values pass, outliers are squashed."""
    grad = list_guard(grad)
    for t in grad:
        x = promote(t) / scale
        tanh = x.tanh()
        x = x.abs().log1p().copysign(tanh) * (1 - lerp) + tanh * lerp
        copy_stochastic_(t, (x * scale).clamp(min=-2, max=2))
    return grad
