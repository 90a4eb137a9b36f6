"""First-order update rules on lists of tensors (fp32 math, stochastic / ECC stores).

Each ``*_`` function mutates optimizer state in place.  ``fused_*`` variants also write the parameter
(``update_by_*`` transforms); plain variants overwrite ``grad``/``update`` with the new direction
(``scale_by_*`` transforms).

Behavioural parity targets: Adam family ``heavyball/utils.py:1852-2334``; momentum variants
``heavyball/utils.py:736-776``; schedule-free and MSAM ``heavyball/utils.py:132-230``; AdEMAMix
schedulers ``heavyball/utils.py:290-334``; NAdam helpers ``heavyball/utils.py:341-410``; MARS
``heavyball/utils.py:3616-3627``; OrthoGrad ``heavyball/utils.py:3630-3649``; hyperball
``heavyball/utils.py:3665-3699``; adaptation rules ``heavyball/utils.py:3745-3804``; SAM ascent
``heavyball/utils.py:3853-3872``.

On CUDA the same arithmetic runs inside ``heavyball_b200.ops`` multi-tensor kernels; these
functions define the semantics and serve CPU, odd dtypes and user-composed chains.
"""

from __future__ import annotations

import math
from typing import List, Optional

import torch
from torch import Tensor

from .core import (
    _caution_impl,  # noqa: F401  (re-exported for monkeypatch parity)
    _decay_factor,
    _lerp,
    _segmented_dot,
    as_float,
    as_int,
    beta_debias,
    copy_stochastic_,
    copy_stochastic_list_,
    eps_sqrt,
    hasattr_none,
    list_guard,
    promote,
    stochastic_add_,
    stochastic_lerp_,
    update_param_,
)
from . import core as _core


def _caution(g, u):
    return _core._caution_impl(g, u)


# ---------------------------------------------------------------------------------------- EMA kit


def _second_moment(state: List[Tensor], g32: List[Tensor], beta2, eps) -> List[Tensor]:
    """Updates the second-moment EMA and returns ``max(sqrt(v), eps)`` in fp32."""
    v32 = _lerp(state, [g * g for g in g32], beta2)
    return [eps_sqrt(v, eps) for v in v32]


def exp_avg_sq_(state, grad, beta2, eps, out=None):
    state, grad = list_guard(state, grad)
    denom = _second_moment(state, promote(list(grad)), beta2, eps)
    if out is None or (isinstance(out, (list, tuple)) and out[0] is None):
        return denom
    out = list_guard(out)
    copy_stochastic_list_(out, denom)
    return out


def _compilable_exp_avg_sq_(state, grad, beta2, eps, out):
    return exp_avg_sq_(state, grad, beta2, eps, out)


def scale_by_exp_avg_sq_(exp_avg_sq, grad, beta2, eps):
    grad, exp_avg_sq = list_guard(grad, exp_avg_sq)
    g32 = promote(list(grad))
    denom = _second_moment(exp_avg_sq, g32, beta2, eps)
    copy_stochastic_list_(grad, [g / d for g, d in zip(g32, denom)])
    return grad


def scale_by_exp_avg_(state, grad, beta):
    state, grad = list_guard(state, grad)
    copy_stochastic_list_(grad, _lerp(state, grad, beta))
    return grad


def heavyball_momentum(state, grad, beta):
    state, grad = list_guard(state, grad)
    for s_, g_ in zip(state, grad):
        v = promote(s_) * beta + promote(g_)
        copy_stochastic_(s_, v)
        copy_stochastic_(g_, v)
    return grad


def nesterov_momentum(state, grad, beta):
    state, grad = list_guard(state, grad)
    for s_, g_ in zip(state, grad):
        g32 = promote(g_)
        v = promote(s_) * beta + g32
        copy_stochastic_(s_, v)
        copy_stochastic_(g_, g32 + v * beta)
    return grad


def nesterov_ema(state, grad, beta):
    state, grad = list_guard(state, grad)
    ema32 = _lerp(state, grad, beta)
    stochastic_add_(grad, ema32, 1)
    return grad


# ---------------------------------------------------------------------------------------- Adam family


def adam_(exp_avg, exp_avg_sq, grad, beta1, beta2, step, eps: float = 1e-8):
    exp_avg, exp_avg_sq, grad = map(list_guard, (exp_avg, exp_avg_sq, grad))
    b1, b2 = beta_debias(beta1, step), beta_debias(beta2, step)
    g32 = promote(list(grad))
    m32 = _lerp(exp_avg, g32, b1)
    denom = _second_moment(exp_avg_sq, g32, b2, eps)
    copy_stochastic_list_(grad, [m / d for m, d in zip(m32, denom)])
    return grad


def fused_adam_(y, exp_avg, exp_avg_sq, update, grad, beta1, beta2, step, lr, eps, decay, caution, cautious_decay=False):
    y, exp_avg, exp_avg_sq, update, grad = list_guard(y, exp_avg, exp_avg_sq, update, grad)
    b1, b2 = beta_debias(beta1, step), beta_debias(beta2, step)
    u32, g32 = promote(list(update)), promote(list(grad))
    m32 = _lerp(exp_avg, u32, b1)
    denom = _second_moment(exp_avg_sq, u32, b2, eps)
    update_param_(y, [m / d for m, d in zip(m32, denom)], lr, decay, caution, cautious_decay, g32)


def unscaled_adam_(exp_avg, exp_avg_sq, grad, beta1, beta2, step, eps: float = 1e-8):
    exp_avg, exp_avg_sq, grad = map(list_guard, (exp_avg, exp_avg_sq, grad))
    b1, b2 = beta_debias(beta1, step), beta_debias(beta2, step)
    g32 = promote(list(grad))
    denom = _second_moment(exp_avg_sq, g32, b2, eps)
    m32 = _lerp(exp_avg, [g / d for g, d in zip(g32, denom)], b1)
    copy_stochastic_list_(grad, [m * d for m, d in zip(m32, denom)])
    return grad


def laprop_(exp_avg, exp_avg_sq, grad, beta1, beta2, step, eps: float = 1e-8):
    exp_avg, exp_avg_sq, grad = list_guard(exp_avg, exp_avg_sq, grad)
    b1, b2 = beta_debias(beta1, step), beta_debias(beta2, step)
    g32 = promote(list(grad))
    denom = _second_moment(exp_avg_sq, g32, b2, eps)
    copy_stochastic_list_(grad, _lerp(exp_avg, [g / d for g, d in zip(g32, denom)], b1))
    return grad


def fused_laprop_(
    y, exp_avg, exp_avg_sq, update, grad, beta1, beta2, step, lr, decay, caution, cautious_decay=False, eps: float = 1e-8
):
    y, exp_avg, exp_avg_sq, update, grad = list_guard(y, exp_avg, exp_avg_sq, update, grad)
    b1, b2 = beta_debias(beta1, step), beta_debias(beta2, step)
    u32, g32 = promote(list(update)), promote(list(grad))
    denom = _second_moment(exp_avg_sq, u32, b2, eps)
    m32 = _lerp(exp_avg, [u / d for u, d in zip(u32, denom)], b1)
    update_param_(y, m32, lr, decay, caution, cautious_decay, g32)


def adopt(grad, exp_avg_sq, exp_avg, beta1, beta2, step, eps: float = 1e-8):
    """ADOPT: normalise by the *previous* second moment, then refresh it."""
    exp_avg, exp_avg_sq, grad = list_guard(exp_avg, exp_avg_sq, grad)
    g32, v32 = promote(list(grad)), promote(list(exp_avg_sq))
    m32 = _lerp(exp_avg, [g / eps_sqrt(v, eps) for g, v in zip(g32, v32)], beta_debias(beta1, step))
    stochastic_lerp_(exp_avg_sq, [g * g for g in g32], 1 - beta_debias(beta2, step + 1))
    copy_stochastic_list_(grad, m32)
    return grad


def fused_adopt_(y, update, grad, exp_avg_sq, exp_avg, beta1, beta2, step, lr, eps, decay, caution, cautious_decay=False):
    y, update, grad, exp_avg_sq, exp_avg = list_guard(y, update, grad, exp_avg_sq, exp_avg)
    u32, g32, v32 = promote(list(update)), promote(list(grad)), promote(list(exp_avg_sq))
    m32 = _lerp(exp_avg, [u / eps_sqrt(v, eps) for u, v in zip(u32, v32)], beta_debias(beta1, step))
    update_param_(y, m32, lr, decay, caution, cautious_decay, g32)
    stochastic_lerp_(exp_avg_sq, [u * u for u in u32], 1 - beta_debias(beta2, step + 1))


# ---------------------------------------------------------------------------------------- AdEMAMix


def linear_warmup_scheduler(step, alpha_end: float, alpha_start: float = 0.0, warmup: Optional[int] = None) -> float:
    if warmup is None or warmup <= 0 or step >= warmup:
        return alpha_end
    a = step / float(warmup)
    return (1.0 - a) * alpha_start + a * alpha_end


def linear_hl_warmup_scheduler(step, beta_end: float, beta_start: float, warmup: Optional[int] = None, eps: float = 1e-8):
    """Interpolates linearly in EMA half-life rather than in beta."""
    if warmup is None or warmup <= 0 or step >= warmup:
        return beta_end
    half_life = lambda b: math.log(0.5) / math.log(b + eps) - 1  # noqa: E731
    a = step / float(warmup)
    t = (1.0 - a) * half_life(beta_start) + a * half_life(beta_end)
    return min(max(math.pow(0.5, 1.0 / (t + 1.0)), 0.0), 1.0 - eps)


def _compute_ademamix_hparams(betas, step, alpha, beta3_warmup, alpha_warmup):
    if len(betas) != 3:
        raise ValueError("AdEMAMix expects betas=(beta1, beta2, beta3).")
    beta1, beta2, beta3 = betas
    step = as_int(step)
    return (
        beta1,
        beta2,
        linear_hl_warmup_scheduler(step, beta_end=beta3, beta_start=beta1, warmup=beta3_warmup),
        linear_warmup_scheduler(step, alpha_end=alpha, alpha_start=0.0, warmup=alpha_warmup),
    )


def _ademamix_direction(fast, slow, sq, update, beta1, beta2, beta3, step, alpha, eps):
    u32 = promote(list(update))
    f32 = _lerp(fast, u32, beta_debias(beta1, step))
    s32 = _lerp(slow, u32, beta3)
    denom = _second_moment(sq, u32, beta_debias(beta2, step), eps)
    return [(f + s * alpha) / d for f, s, d in zip(f32, s32, denom)]


def ademamix_(exp_avg_fast, exp_avg_slow, exp_avg_sq, grad, betas, step, eps, alpha, beta3_warmup=None, alpha_warmup=None):
    exp_avg_fast, exp_avg_slow, exp_avg_sq, grad = list_guard(exp_avg_fast, exp_avg_slow, exp_avg_sq, grad)
    if not grad:
        return grad
    b1, b2, b3, a = _compute_ademamix_hparams(betas, step, alpha, beta3_warmup, alpha_warmup)
    copy_stochastic_list_(grad, _ademamix_direction(exp_avg_fast, exp_avg_slow, exp_avg_sq, grad, b1, b2, b3, step, a, eps))
    return grad


def fused_ademamix_(
    y, exp_avg_fast, exp_avg_slow, exp_avg_sq, update, grad, betas, step, lr, eps, decay, alpha, caution,
    cautious_decay=False, beta3_warmup=None, alpha_warmup=None,
):  # fmt: skip
    y, exp_avg_fast, exp_avg_slow, exp_avg_sq, update, grad = list_guard(
        y, exp_avg_fast, exp_avg_slow, exp_avg_sq, update, grad
    )
    if not y:
        return
    b1, b2, b3, a = _compute_ademamix_hparams(betas, step, alpha, beta3_warmup, alpha_warmup)
    g32 = promote(list(grad))
    u32 = _ademamix_direction(exp_avg_fast, exp_avg_slow, exp_avg_sq, update, b1, b2, b3, step, a, eps)
    update_param_(y, u32, lr, decay, caution, cautious_decay, g32)


# ---------------------------------------------------------------------------------------- NAdam


def _nadam_moments(beta1, step, momentum_decay):
    step = as_float(step)
    beta1 = as_float(beta1)
    mu = beta1 * (1 - 0.5 * 0.96 ** (step * momentum_decay))
    mu_next = beta1 * (1 - 0.5 * 0.96 ** ((step + 1) * momentum_decay))
    return mu, mu_next


def _nadam_direction(exp_avg, exp_avg_sq, mu_product, u32, beta1, beta2, step, eps, mu, mu_next):
    m32 = _lerp(exp_avg, u32, beta1)
    denom = _second_moment(exp_avg_sq, u32, beta_debias(beta2, step), eps)
    for mp in mu_product:
        mp.mul_(mu)
    out = []
    for u, m, d, mp in zip(u32, m32, denom, promote(list(mu_product))):
        gw = (1 - mu) / (1 - mp)
        ew = mu_next / (1 - mp * mu_next)
        out.append(u / d * gw + m / d * ew)
    return out


def nadam_(param, exp_avg, exp_avg_sq, mu_product, update, beta1, beta2, step, momentum_decay, eps, weight_decay,
           decoupled_weight_decay):  # fmt: skip
    param, exp_avg, exp_avg_sq, mu_product, update = map(list_guard, (param, exp_avg, exp_avg_sq, mu_product, update))
    if not param:
        return update
    wd = float(weight_decay)
    coupled = wd != 0 and not decoupled_weight_decay
    u32 = [promote(u) for u in update]
    p32 = [promote(p) for p in param]
    if coupled:
        u32 = [u + p * wd for u, p in zip(u32, p32)]
    mu, mu_next = _nadam_moments(beta1, step, momentum_decay)
    u32 = _nadam_direction(exp_avg, exp_avg_sq, mu_product, u32, beta1, beta2, step, eps, mu, mu_next)
    if coupled:
        u32 = [u - p * wd for u, p in zip(u32, p32)]
    copy_stochastic_list_(update, u32)
    return update


def fused_nadam_(param, exp_avg, exp_avg_sq, mu_product, update, grad, beta1, beta2, step, lr, eps, momentum_decay,
                 weight_decay, decoupled_weight_decay, caution, cautious_decay=False):  # fmt: skip
    param, exp_avg, exp_avg_sq, mu_product, update, grad = list_guard(
        param, exp_avg, exp_avg_sq, mu_product, update, grad
    )
    if not param:
        return
    wd = float(weight_decay)
    coupled = wd != 0 and not decoupled_weight_decay
    u32 = [promote(u) for u in update]
    g32 = [promote(g) for g in grad]
    p32 = [promote(p) for p in param]
    if coupled:  # L2 regularisation: the decay joins the gradient seen by the moments and by caution
        u32 = [u + p * wd for u, p in zip(u32, p32)]
        g32 = [g + p * wd for g, p in zip(g32, p32)]
    mu, mu_next = _nadam_moments(beta1, step, momentum_decay)
    u32 = _nadam_direction(exp_avg, exp_avg_sq, mu_product, u32, beta1, beta2, step, eps, mu, mu_next)
    if coupled:
        u32 = [u - p * wd for u, p in zip(u32, p32)]
    copy_stochastic_list_(update, u32)
    decay = wd if (wd != 0 and decoupled_weight_decay) else 0.0
    update_param_(param, u32, lr, decay, caution, cautious_decay, g32)


# ---------------------------------------------------------------------------------------- schedule-free / MSAM


def _schedule_free_apply(p, z, ckp1, update, lr, beta1, decay, grad, caution, cautious_decay):
    for op, oz, u_, g_ in zip(p, z, update, grad):
        p32, z32, u32 = promote(op), promote(oz), promote(u_.view_as(op))
        if decay != 0:
            u32 = u32 + p32 * _decay_factor(p32, u32, decay, cautious_decay)
        if caution:
            u32 = _caution(g_, u32)
        p32 = torch.lerp(p32, z32, ckp1) if not isinstance(ckp1, Tensor) else p32 + (z32 - p32) * ckp1
        p32 = p32 + u32 * (lr * (beta1 * (1 - ckp1)) - lr)
        z32 = z32 + u32 * -lr
        copy_stochastic_(op, p32)
        copy_stochastic_(oz, z32)


_compilable_schedule_free_ = _schedule_free_apply


def schedule_free_(lr, weight_lr_power, weight_sum, beta1, parameters, z, update, grad, caution=False, r=0.0, step=0,
                   decay=0.0, cautious_decay=False):  # fmt: skip
    weight = abs(lr) ** weight_lr_power * max(step, 1) ** r
    weight_sum = weight_sum + weight
    ckp1 = weight / weight_sum if weight_sum != 0 else 0
    update, parameters, z, grad = list_guard(update, parameters, z, grad)
    _schedule_free_apply(parameters, z, ckp1, update, lr, beta1, decay, grad, caution, cautious_decay)
    return weight_sum


def msam_(lr, beta1, param, z, update, grad, exp_avg, caution, weight_decay, sam_step_size, cautious_decay=False):
    """Momentum-SAM: ``z`` holds the unperturbed weights, the parameter sits at the ascent point."""
    param, z, update, grad, exp_avg = list_guard(param, z, update, grad, exp_avg)
    m32 = _lerp(exp_avg, update, beta1)
    for u32, g_, z_, p_ in zip(m32, grad, z, param):
        u32 = u32.view_as(z_)
        z32 = promote(z_)
        if caution:
            u32 = _caution(g_, u32)
        d = _decay_factor(z32, u32, weight_decay, cautious_decay)
        z32 = z32 * (1 - d * lr) + u32 * -lr
        copy_stochastic_(z_, z32)
        copy_stochastic_(p_, z32 + u32 / u32.norm().clamp(min=1e-8) * -sam_step_size)


# ---------------------------------------------------------------------------------------- MARS / sign / OrthoGrad / hyperball


def mars_correction(g, old_g, beta1, gamma):
    """``g <- g + gamma*beta1/(1-beta1) * (g - g_prev)``; ``g_prev <- g`` (uncorrected)."""
    a = -gamma * beta1 / (1 - beta1)
    g, old_g = list_guard(g), list_guard(old_g)
    raw = [x.clone() for x in g]
    stochastic_lerp_(g, old_g, a)
    copy_stochastic_list_(old_g, raw)


def _compilable_grafting(magnitude: Tensor, direction: Tensor) -> Tensor:
    return direction * (magnitude.norm() / direction.norm().clamp(min=1e-6))


def sign_(grad, graft: bool = True):
    grad = list_guard(grad)
    for g_ in grad:
        s = g_.sign()
        copy_stochastic_(g_, _compilable_grafting(g_, s) if graft else s)
    return grad


def orthogonalize_grad_to_param(weight, grad, eps, graft=True):
    """OrthoGrad: remove the component of the gradient along the weight vector."""
    weight, grad = list_guard(weight, grad)
    dots = _segmented_dot(list(weight) + list(weight), list(grad) + list(weight)) if weight else None  # w.g then w.w
    for i, (w, g) in enumerate(zip(weight, grad)):
        w32, g32 = promote(w), promote(g)
        wg, ww = ((w32 * g32).sum(), (w32 * w32).sum()) if dots is None else (dots[i], dots[len(weight) + i])
        out = g32 - (wg / (ww + eps)) * w32
        copy_stochastic_(g, _compilable_grafting(g32, out) if graft else out)
    return grad


def hyperball_step_(param, update, init_norm, lr, decay, caution, grad, cautious_decay=False):
    param, update, init_norm = list_guard(param, update, init_norm)
    grad = list_guard(grad) if caution else [None] * len(param)
    for op, u_, n_, g_ in zip(param, update, init_norm, grad):
        u32, p32 = promote(u_.view_as(op)), promote(op)
        if decay != 0:
            u32 = u32 + p32 * _decay_factor(p32, u32, decay, cautious_decay)
        if caution:
            u32 = _caution(g_, u32)
        u32 = u32 / u32.norm().clamp(min=1e-12)
        p32 = p32 - lr * u32 * n_
        copy_stochastic_(op, p32 * (n_ / p32.norm().clamp(min=1e-12)))


# ---------------------------------------------------------------------------------------- decay-to-reference variants


def weight_decay_to_ema_(p, ema, ema_decay, weight_decay):
    p, ema = list_guard(p, ema)
    _lerp(p, _lerp(ema, p, ema_decay), 1 - weight_decay)


def l1_weight_decay_to_ema_(p, ema, ema_decay, weight_decay):
    p, ema = list_guard(p, ema)
    for p_, e32 in zip(p, _lerp(ema, p, ema_decay)):
        p32 = promote(p_)
        copy_stochastic_(p_, p32 + (p32 - e32).sign() * weight_decay)


# ---------------------------------------------------------------------------------------- learned step sizes


def d_adaptation(grads, update, state, delta):
    grads, update, state, delta = list_guard(grads, update, state, delta)
    for g_, u_, s_, d_ in zip(grads, update, state, delta):
        g, u, s, d = promote(g_), promote(u_), promote(s_), promote(d_)
        nxt = d * (g * s).sum()
        s = s + u * d
        nxt = torch.maximum(nxt / s.abs().sum(), d)
        copy_stochastic_(u_, u * d)
        copy_stochastic_(d_, nxt)
        copy_stochastic_(s_, s)


def _lr_adapt(grads, update, state, delta, lr_lr, pointwise: bool):
    grads, update, state, delta = list_guard(grads, update, state, delta)
    for g_, u_, s_, d_ in zip(grads, update, state, delta):
        g, u, s, d = promote(g_), promote(u_), promote(s_), promote(d_)
        sig = d.sigmoid()
        corr = s * g if pointwise else (s * g).mean()
        d = d - sig * (1 - sig) * corr * lr_lr
        copy_stochastic_(d_, d)
        copy_stochastic_(u_, u * d.sigmoid())
        copy_stochastic_(s_, u)


def lr_adaptation(grads, update, state, delta, lr_lr):
    _lr_adapt(grads, update, state, delta, lr_lr, False)


def pointwise_lr_adaptation(grads, update, state, delta, lr_lr):
    _lr_adapt(grads, update, state, delta, lr_lr, True)


# ---------------------------------------------------------------------------------------- SAM / AGC


def sam_step(parameters, ball_size, adaptive: bool = True):
    """Ascent step of (adaptive) SAM; returns clones of the pre-perturbation parameters."""
    saved = []
    for p in parameters:
        saved.append(p.detach().clone())
        if not hasattr_none(p, "grad"):
            continue
        g = promote(p.grad)
        if adaptive:
            g = g * promote(p).square()
        stochastic_add_(p.data, g, ball_size)
        p.grad.zero_()
    return saved


def adaptive_gradient_clipping_(parameters, gradients, clip_val: float, minimum: float = 1e-3, eps: float = 1e-8):
    if clip_val <= 0:
        return gradients
    parameters, gradients = list_guard(parameters, gradients)
    for p, g in zip(parameters, gradients):
        p32, g32 = promote(p), promote(g)
        scale = (p32.norm().clamp(min=minimum) / g32.norm().clamp(min=eps) * clip_val).clamp(max=1)
        copy_stochastic_(g, g32 * scale)
    return gradients


# ---------------------------------------------------------------------------------------- rank-1 curvature sketch (SUDS)
# parity: heavyball/utils.py:3177-3223


def _householder_vec_e1_to_v(v: Tensor, eps: float = 1e-12) -> Tensor:
    """``w`` such that ``H = I - 2 w w^T`` maps ``e1`` to the unit vector ``v`` (``w = 0`` if ``v = e1``)."""
    v = v / v.norm().clamp(min=eps)
    e1 = torch.zeros_like(v)
    e1[0] = 1.0
    w = e1 - v
    return w / w.norm().clamp(min=eps)


def eigvecs_product_rank1(G: Tensor, v: Tensor, w: Optional[Tensor] = None, eps: float = 1e-12):
    """``G @ V`` for an eigenvector matrix ``V`` of ``lambda I + sigma v v^T`` (a Householder
    reflector whose first column is ``v``), never materialising ``V``.  Returns ``(G V, w)``."""
    if w is None:
        w = _householder_vec_e1_to_v(v, eps)
    return G - 2.0 * torch.einsum("...i,i,j->...j", G, w, w), w


def oja_update(v: Tensor, g: Tensor, lr: float = 1e-2, eps: float = 1e-12) -> Tensor:
    """One step of Oja's rule towards the top eigenvector of ``E[g g^T]``; result is unit norm."""
    gv = g @ v
    v = v + lr * (gv * g - (gv * gv) * v)
    return v / v.norm().clamp(min=eps)
