"""PSGD preconditioners: Kronecker-factored (triangular / diagonal factors), the PRO (Procrustes)
variant and the low-rank approximation, with the spectral-norm estimators they rely on.

Tensors carry a leading *slot* dimension: a triangular factor is ``(slots, d, d)``, a diagonal one
``(slots, d)``.  With ``store_triu_as_line`` a triangular factor is kept as ``(shape, packed)`` where
``packed`` is the row-major upper triangle ``(slots, d (d + 1) / 2)``.

Behavioural parity targets: ``heavyball/utils.py:2425-2594`` (init scale, factor layout),
``heavyball/utils.py:2597-2605, 2875-2910, 3051-3122`` (Kron update), ``heavyball/utils.py:3125-3174``
(PRO), ``heavyball/utils.py:3503-3613`` (apply), ``heavyball/utils.py:2523-2533, 2608-2805`` (LRA),
``heavyball/utils.py:2913-3048`` (spectral estimators), ``heavyball/utils.py:3458-3482`` (packing),
``heavyball/utils.py:3494-3500, 3702-3723`` (update schedule).
"""

from __future__ import annotations

import functools
import math
import sys
from typing import List, Optional, Tuple, Union

import numpy as np
import torch
import torch.nn.functional as F
from torch import Tensor

from .core import (
    apply_flat_add,
    copy_stochastic_,
    flatten,
    list_guard,
    min_dtype,
    multi_flatten,
    promote,
    stochastic_add_,
    stochastic_multiply_,
    stochastic_round_,
    update_param_,
    warn_once,
)
from . import core as _core
from .core import _mm, _mm_upper, _segmented_absmax_rows, _solve_right_upper, _tc_matmul
from .orthogonal import inplace_orthogonal_
from .soap import compiled_einsum, einsum_base

TriuOrLine = Union[List[Tensor], List[Tuple[Optional[List[int]], Tensor]]]


def _settings():
    return sys.modules[__package__]


# ---------------------------------------------------------------------------------------- schedules


def psgd_should_update(group, prob, name: str = "cumulative_prob"):
    """Deterministic thinning: fires whenever the running sum of probabilities crosses an integer."""
    key = f"{name}_prob_step"
    group[key] = group.get(key, 0) + 1
    if not isinstance(prob, float):
        prob = prob(group[key])
        if isinstance(prob, Tensor):
            prob = float(prob)
    before = group.get(name, 0)
    group[name] = before + prob
    return int(group[name]) > int(before)


def _inner_precond_update_prob_schedule(n, max_prob=1.0, min_prob=0.03, decay=0.999, flat_start=1000):
    return max(min_prob, max_prob * decay ** max(n - flat_start, 0))


def precond_update_prob_schedule(max_prob=1.0, min_prob=0.03, decay=0.999, flat_start=1000):
    """Flat at ``max_prob`` for ``flat_start`` steps, then exponential anneal down to ``min_prob``."""
    return functools.partial(
        _inner_precond_update_prob_schedule, max_prob=max_prob, min_prob=min_prob, decay=decay, flat_start=flat_start
    )


# ---------------------------------------------------------------------------------------- packing


@functools.lru_cache(maxsize=64)
def _triu_index(d0: int, d1: int, device) -> Tuple[Tensor, Tensor]:
    rows, cols = torch.triu_indices(d0, d1, device=device)
    return rows, cols


def _triu_kernels(t: Tensor, square: bool):
    """The extension when its packed-triangle kernels apply (batched square CUDA matrices, 2- or 4-byte elements)."""
    if not (t.is_cuda and square and t.element_size() in (2, 4) and t.shape[0] <= 65535 and not t.is_complex()):
        return None
    from .. import ops

    return ops.load() if ops.available() else None


def _pack_upper(q: Tensor):
    """``(shape, packed)``: the row-major upper triangle of a dense factor; vectors (diagonal factors) pass through
    with ``shape=None``."""
    if q.dim() < 3:
        return None, q
    ext = _triu_kernels(q, q.dim() == 3 and q.shape[-2] == q.shape[-1])
    if ext is not None:
        return tuple(q.shape), ext.triu_pack(q.contiguous())
    rows, cols = _triu_index(q.shape[-2], q.shape[-1], q.device)
    return tuple(q.shape), q[..., rows, cols]


def triu_to_line(Q_list: List[Tensor]):
    return [_pack_upper(q) for q in Q_list]


def line_to_triu(Q_list):
    out = []
    for shape, q in Q_list:
        if shape is not None:
            d0, d1 = shape[-2], shape[-1]
            ext = _triu_kernels(q, q.dim() == 2 and d0 == d1)
            if ext is not None:
                q = ext.triu_unpack(q.contiguous(), d0)
            else:
                rows, cols = _triu_index(d0, d1, q.device)
                dense = torch.zeros(q.shape[:-1] + (d0, d1), device=q.device, dtype=q.dtype)
                dense[..., rows, cols] = q
                q = dense
        out.append(q)
    return out


# ---------------------------------------------------------------------------------------- init


def stable_exp(x: Tensor):
    return torch.where(x > 0, 1 / (-x).exp(), x.exp())


def _lse_mean(x: Tensor, pow: float, eps: float) -> Tensor:
    # log( mean(|x|^pow) ^ (1 / (2 pow)) ), evaluated in log space
    logs = x.double().abs().clamp(min=eps).log() * pow
    return (logs.flatten().logsumexp(dim=0) - math.log(x.numel())) / pow / 2


def mean_root(x: Tensor, pow: float, eps=1e-12):
    return stable_exp(-_lse_mean(x, pow, eps))


def divided_root(x: Tensor, y: Tensor, pow0: float, pow1: float, eps=1e-12):
    return stable_exp(_lse_mean(x, pow0, eps) - _lse_mean(y, pow1, eps))


class PrecondInitError(ValueError):
    pass


_SCALE_HINT = " Set it manually using `precond_init_scale=0.1`"


def _explain_bad_scale(tensors):
    """Raises with the reason an automatic initial scale came out unusable, if the inputs show one."""
    for t in tensors:
        if t is None:
            continue
        if torch.allclose(t, torch.zeros_like(t)):
            raise PrecondInitError(f"Grad or HVP is all 0s, causing NaNs in precond_init_scale computation.{_SCALE_HINT}")
        if not bool(torch.isfinite(t).all()):
            raise PrecondInitError("Grad or HVP is not finite")


def precond_init_scale(scale, scale_scale, scale_power, grad, hessian_vector, vector, scale_max: float = 100):
    """Initial scale of the preconditioner.  A user-given ``scale`` is taken as it is (with advice against combining it
    with the multiplier / exponent knobs).  Otherwise it is estimated in log space: from the fourth-moment root of the
    gradient, or, when a probe / Hessian-vector pair is at hand, from their ratio; multiplied by ``scale_scale`` and
    raised to ``scale_power`` (default 1/2)."""
    multiplier = 1 if scale_scale is None else scale_scale
    given = scale is not None
    if given:
        warn_once("It's recommended to use precond_init_scale=None (default since 1.7.x), which uses advanced heuristics.")
        for knob, text in (
            (multiplier != 1, "precond_init_scale_scale multiplies the precond_init_scale by a constant factor. "),
            (scale_power is not None, "precond_init_scale_power is used to compute precond_init_scale ** precond_init_scale_power. "),
        ):
            if knob:
                warn_once(text + "With a fixed precond_init_scale, you should explicitly fuse it.")
        value = scale
    else:
        root = mean_root(grad, 4) if hessian_vector is None else divided_root(vector, hessian_vector, 2, 4)
        value = (root * multiplier) ** (0.5 if scale_power is None else scale_power)
    value = value.item() if isinstance(value, Tensor) else value

    finite = bool(np.isfinite(value))
    if finite and value <= scale_max:
        return value
    if finite:
        warn_once(f"The computed precond_init_scale {value} is outside of the expected range.{_SCALE_HINT}")
    if given:
        raise PrecondInitError("The manually set precond_init_scale is not finite")
    _explain_bad_scale((grad, hessian_vector, vector))
    if finite:
        return value
    raise PrecondInitError(f"Computed precond_init_scale is not finite.{_SCALE_HINT}")


def _max_idx(x):
    return len(x) - 1 - int(np.argmax(x[::-1]))


def init_Q_exprs(grad, scale, scale_scale, scale_power, max_size, min_ndim_triangular, memory_save_mode,
                 hessian_vector, vector, dtype=None):  # fmt: skip
    """One factor per non-slot dim: dense upper-triangular ``scale^(1/k) I`` or, for size-1 /
    oversize / memory-saving dims, a diagonal vector."""
    scale = precond_init_scale(scale, scale_scale, scale_power, grad, hessian_vector, vector)
    dtype = grad.dtype if dtype is None else dtype
    n, shape = grad.shape[0], grad.shape[1:]
    if len(shape) == 0:
        return [scale * torch.ones_like(grad, dtype=dtype)]
    scale = scale ** (1 / len(shape))

    if memory_save_mode is None:
        diag = [False] * len(shape)
    elif memory_save_mode == "one_diag":
        diag = [False] * len(shape)
        diag[_max_idx(shape)] = True
    elif memory_save_mode == "smart_one_diag":
        diag = [False] * len(shape)
        ordered = sorted(shape)
        if len(shape) >= 2 and ordered[-1] > ordered[-2]:
            diag[_max_idx(shape)] = True
    elif memory_save_mode == "one_triu":
        diag = (np.argsort(np.argsort(shape)) != 0).tolist()
    elif memory_save_mode == "all_diag":
        diag = [True] * len(shape)
    else:
        raise ValueError(
            f"Invalid memory_save_mode: {memory_save_mode}, must be one of [None, 'one_diag', 'all_diag', 'smart_one_diag']"
        )

    Q = []
    for size, is_diag in zip(shape, diag):
        if size == 1 or size > max_size or len(shape) < min_ndim_triangular or is_diag:
            Q.append(scale * torch.ones(n, size, dtype=promote(dtype), device=grad.device))
        else:
            Q.append(scale * torch.eye(size, dtype=dtype, device=grad.device).expand(n, size, size).contiguous())
    return Q


def init_lra(grad, param_count, scale, scale_scale, scale_power, rank, hessian_vector, vector, dtype=None, eps: float = 10):
    """Low-rank preconditioner ``(I + U V^T) diag(d)`` at its start: ``d`` constant at the initial scale, ``U`` and ``V``
    Gaussian with standard deviation ``(param_count (rank + eps))^-1/2``, so ``U V^T`` starts as a small perturbation."""
    d0 = precond_init_scale(scale, scale_scale, scale_power, grad, hessian_vector, vector)
    spread = 1.0 / math.sqrt(param_count * (rank + eps))
    like = dict(dtype=dtype, device=grad.device)
    U, V = (torch.randn((*grad.shape, rank), **like) * spread for _ in range(2))
    return U, V, torch.full_like(grad, d0, **like)


# ---------------------------------------------------------------------------------------- spectral estimators


def max_singular_value_exact(A, use_lobpcg: bool = False):
    try:
        if use_lobpcg:
            val, _ = torch.lobpcg(A @ A.mT, k=1, largest=True)
            return val[..., 0].sqrt()
        kwargs = {"driver": "gesvdj"} if A.is_cuda else {}
        return torch.linalg.svd(promote(A), **kwargs)[1].amax(dim=-1).to(A.dtype)
    except (torch.linalg.LinAlgError, RuntimeError):
        return max_singular_value_power_iter(promote(A), iterations=2)


def _seed_from_largest_row(A: Tensor):
    norms = A.norm(dim=-1)
    top, idx = norms.max(dim=-1)
    top = promote(top).clamp(min=torch.finfo(torch.float32).tiny)
    gather = idx[..., None, None].expand(*A.shape[:-2], 1, A.shape[-1])
    return A.gather(-2, gather).squeeze(-2) / top[..., None], top


def max_singular_value_power_iter(A_outer: Tensor, iterations: int = 5):
    """Power iteration on ``A^T A`` started from the largest row; the matrix is scaled to unit
    largest-row norm and held in bf16 (stochastically rounded) for the matvecs."""
    x, top = _seed_from_largest_row(A_outer)
    A = stochastic_round_(A_outer / top[..., None, None])

    def mv(v):
        return promote((A.mT @ (A @ v[..., None].to(A.dtype))).squeeze(-1))

    for _ in range(iterations):
        x = F.normalize(mv(x), dim=-1)
    return ((x * mv(x)).sum(dim=-1).sqrt() * top).to(top.dtype)


def max_singular_value_cholesky(A: Tensor, max_abs: Optional[Tensor] = None):
    """Sketch: top-k columns by norm -> orthogonalise -> project -> orthogonalise -> exact k x k."""
    if max_abs is None:
        max_abs = A.abs().amax(dim=(-2, -1), keepdim=True).clamp(min=1e-8)
    k = 2 ** math.ceil(math.log2(math.log2(min(A.shape[-2:]))))
    cols = A.square().sum(-2).topk(k, largest=True).indices
    Y = A.gather(-1, cols.unsqueeze(-2).expand(*A.shape[:-1], k)) / max_abs
    precise = _settings().precise_zeroth_power_mode
    Qm = inplace_orthogonal_(Y, precise) / max_abs
    Z = A.mT @ Qm
    W = inplace_orthogonal_(Z, precise)
    return max_singular_value_exact(Z.mT @ W) * max_abs.squeeze(-1).squeeze(-1)


def max_singular_value(A: Tensor, max_svd: int = 0, use_cholesky: bool = False, power_iter: int = 16) -> Tensor:
    """Spectral norm estimate.  Dispatch: vectors -> largest magnitude; matrices no larger than ``max_svd`` -> exact;
    ``use_cholesky`` (or a negative iteration count) -> the top-k sketch; otherwise power iteration."""
    if A.ndim < 2:
        return A.abs().max()
    small = min(A.shape[-2:]) <= max_svd
    if small:
        return max_singular_value_exact(A)
    sketch = use_cholesky or power_iter < 0
    return max_singular_value_cholesky(A) if sketch else max_singular_value_power_iter(A, iterations=power_iter)


def clamped_max_singular_value(A: Tensor, min: float, max_svd: int = 0, use_cholesky: bool = False, power_iter: int = 16):
    return max_singular_value(A, max_svd, use_cholesky, power_iter).clamp(min=min)


def max_eigenvalue_spd(A_outer: Tensor, power_iter: int = 4) -> Tensor:
    """Largest eigenvalue of (a batch of) SPD matrices by power iteration on ``A^2``."""
    if A_outer.ndim < 2:
        return A_outer.max()
    x, top = _seed_from_largest_row(A_outer)
    A = promote(A_outer) / top[..., None, None]

    def mv(v):
        return promote(((v[..., None, :] @ A.mT) @ A.mT).squeeze(-2))

    for _ in range(power_iter):
        x = F.normalize(mv(x), dim=-1)
    return (x * mv(x)).sum(dim=-1).sqrt() * top


def min_singular_value(A: Tensor, power_iter: int = 5, safety: float = 1.05, max_svd: int = 32):
    """Smallest eigenvalue of a symmetric PSD matrix via shifted power iteration, with a
    moment-based bound as fallback."""
    if A.ndim < 2:
        return A.abs().min()
    n = A.size(0)
    if n <= max_svd:
        try:
            return torch.linalg.eigvalsh(promote(A)).min().to(A.dtype)
        except torch.linalg.LinAlgError:
            pass
    upper = max_singular_value(A, power_iter=power_iter) * safety
    tiny = torch.finfo(torch.float32).tiny
    _, idx = A.norm(dim=1).min(dim=0)
    v = A.index_select(0, idx.reshape(1)).flatten()
    v = v + torch.randn_like(v) * torch.finfo(v.dtype).tiny
    v = v / promote(v.norm().clamp(min=tiny))
    for _ in range(power_iter):
        v = upper * v - promote(A.mv(v.to(A.dtype)))
        v = v / promote(v.norm().clamp(min=tiny))
    mu_hat = promote(v) @ (upper * promote(v) - promote(A.mv(v.to(A.dtype))))
    est = upper - mu_hat
    mu = A.trace() / n
    var = A.square().sum() / n - mu**2
    approx = mu - (var / (n - 1)).sqrt()
    return torch.where((~torch.isfinite(est)) | (est <= 0), approx, est).squeeze()


# ---------------------------------------------------------------------------------------- Kron: expressions


def ndim_tuple(Q) -> tuple:
    return tuple(q.ndim for q in Q)


@functools.lru_cache(maxsize=None)
def cached_precond_grad_expr(Q_dim, grad_dim):
    """einsum applying one factor per mode once: ``A = (Q_1 x Q_2 x ...) g``."""
    parts = [f"...{c.upper()}{c}" if d == 3 else f"...{c}" if d == 2 else "..." for c, d in zip(einsum_base, Q_dim)]
    joined = ",".join(parts)
    g = einsum_base[: grad_dim - 1]
    out = "".join(c.upper() if c.upper() in joined else c for c in g)
    return f"{joined},...{g}->...{out}"


@functools.lru_cache(maxsize=None)
def precond_grad_expr(Q_dim, grad_dim):
    """einsum applying every factor twice: ``P g = Q^T Q g`` per mode."""
    parts = [
        f"...{c2}{c.upper()},...{c2}{c}" if d == 3 else f"...{c},...{c}" if d == 2 else "...,..."
        for c, c2, d in zip(einsum_base, einsum_base[13:], Q_dim)
    ]
    joined = ",".join(parts)
    g = einsum_base[: grad_dim - 1]
    out = "".join(c.upper() if c.upper() in joined else c for c in g)
    return f"{joined},...{g}->...{out}"


@functools.lru_cache(maxsize=None)
def calcG_expr(q_dim, g_dim):
    """Per-mode contraction of ``A`` (or ``conjB``) with itself over all other modes."""
    base = einsum_base[: g_dim - 1]
    exprs = []
    for i, d in enumerate(q_dim):
        other = list(base)
        if d == 3:
            other[i] = "Z"
            out = f"{base[i]}Z"
        elif d == 2:
            out = base[i]
        else:
            out = ""
        exprs.append(f"...{base},...{''.join(other)}->...{out}")
    return exprs


def casted_einsum(expr: str, *args: Tensor) -> Tensor:
    return compiled_einsum(expr, *[promote(a) for a in args]).to(args[-1].dtype)


def _kron_apply(g: Tensor, factors, twice: bool) -> Tensor:
    """Applies one Kronecker factor per non-slot mode of ``g``: ``Q_i g`` (``twice=False``) or
    ``Q_i^T Q_i g`` (``twice=True``); 2-D factors are diagonals, 1-D ones per-slot scalars.

    Equivalent to the multi-operand einsums of :func:`cached_precond_grad_expr` /
    :func:`precond_grad_expr`, but contracted one mode at a time starting from ``g``: a left-to-right
    einsum over ``(Q_1, Q_2, ..., g)`` would first form the outer product of the factors
    (``slots x d1^2 x d2^2`` elements) unless an external contraction-path optimiser is installed."""
    out = g
    for i, q in enumerate(factors):
        dim = i + 1
        if q.ndim == 3:
            moved = out.movedim(dim, -1)
            lead = moved.shape
            flat = moved.reshape(lead[0], -1, lead[-1])
            flat = _mm(flat, q, False, True)
            if twice:
                flat = _mm(flat, q)
            out = flat.reshape(*lead[:-1], flat.shape[-1]).movedim(-1, dim)
        else:
            scale = q * q if twice else q
            if q.ndim == 2 and out.ndim > 1:
                shape = [q.shape[0]] + [1] * (out.ndim - 1)
                shape[dim] = -1
                scale = scale.view(shape)
            elif out.ndim > 1:
                scale = scale.view(-1, *([1] * (out.ndim - 1)))
            out = out * scale
    return out


# ---------------------------------------------------------------------------------------- Kron: update


def psgd_balance_Q(Q):
    """Rescales factors (per slot) to a common max-abs, leaving their Kronecker product unchanged."""
    peaks = _segmented_absmax_rows(Q)  # one launch over every slot of every factor on sm_100a
    if peaks is None:
        peaks = [promote(q.abs().amax(dim=tuple(range(1, q.ndim)))) for q in Q]
    logs = [pk.log() for pk in peaks]
    mean = sum(logs) / len(Q)
    for q, lg in zip(Q, logs):
        q *= (mean - lg).exp().view(-1, *([1] * (q.ndim - 1)))


def _balance_to_triu(Q):
    """Balances the factors in whatever form they are stored (the packed triangle scales like the dense factor) and
    returns them dense."""
    packed = isinstance(Q[0], tuple)
    psgd_balance_Q([entry[1] for entry in Q] if packed else Q)
    return line_to_triu(Q) if packed else Q


def dampen_grad(g: Tensor, damp: float = 1e-9):
    v = torch.randn_like(g)
    return v, g + (damp + torch.finfo(torch.float32).eps * g.abs()) * v


def dampen_multiple(g: List[Tensor], damp: float = 1e-9):
    vs, gs = zip(*[dampen_grad(x, damp) for x in g])
    return flatten(list(vs)), flatten(list(gs))


def psgd_calc_A_and_conjB(G: Tensor, Q, conjB: Optional[Tensor]):
    """``A = Q g`` and ``conjB = v Q^-1`` (diagonal factors by division, triangular ones by a right
    triangular solve per mode)."""
    if conjB is None:
        conjB = torch.randn_like(G)
    A = _kron_apply(promote(G), [promote(q) for q in Q], twice=False).to(G.dtype)
    conjB = promote(conjB)
    tri = []
    for i, q in enumerate(Q):
        q = promote(q)
        if q.dim() <= 2:
            if conjB.ndim == 1:
                conjB = conjB / q
            else:
                shape = [q.shape[0]] + [1] * (conjB.ndim - 1)
                shape[i + 1] = -1
                conjB = conjB / q.view(shape)
        else:
            tri.append((i + 1, q))
    n = G.shape[0]
    for dim, q in tri:
        moved = conjB.movedim(dim, -1).contiguous()
        solved = _solve_right_upper(q, moved.reshape(n, -1, moved.shape[-1]))
        conjB = solved.reshape(moved.shape).movedim(-1, dim).contiguous()
    return A, conjB


def _outer(expr: str, x: Tensor, mode: int, dense: bool = True) -> Tensor:
    """Per-mode second moment (fp32): ``x_(mode) x_(mode)^T`` for a dense factor (matrices take the tensor-core
    product), only its diagonal for a diagonal factor."""
    if dense and x.ndim == 3:
        x32 = promote(x)
        out = _tc_matmul(x32, x32, mode == 1, mode == 0)
        if out is not None:
            return out
    return promote(compiled_einsum(expr, x, x))


def _update_lb(ell: Tensor, lb_state: Tensor, beta) -> Tensor:
    ell, old = promote(ell), promote(lb_state)
    ell = ell.maximum(old + (ell - old) * (1 - beta))
    copy_stochastic_(lb_state, ell)
    return ell


def psgd_update_precond(G, precond_lr, oq, store_triu_as_line, beta2, V, running_lower_bound, lower_bount_beta, power_iter):
    """One Lie-group step on every Kronecker factor from the pair ``(V, G)``:
    ``Q_i <- Q_i - lr * triu(A A^T - B B^T)_i Q_i / L_i`` with ``L_i`` a running lower bound of the
    spectral norm of ``A A^T + B B^T``."""
    Q = _balance_to_triu(oq)
    exprs = calcG_expr(ndim_tuple(Q), G.ndim)
    A, conjB = psgd_calc_A_and_conjB(G, Q, V)
    del V
    for mode, (oq_i, q, expr, lb) in enumerate(zip(oq, Q, exprs, running_lower_bound)):
        t1 = _outer(expr, A, mode, q.ndim == 3)
        t2 = _outer(expr, conjB, mode, q.ndim == 3)
        if q.ndim < 3:
            total = t1 + t2
            ell = _update_lb(total if q.ndim == 1 else total.amax(dim=-1), lb, lower_bount_beta)
            step = promote(q) * (t1 - t2)
        else:
            ell = _update_lb(max_eigenvalue_spd(t1 + t2, power_iter=power_iter), lb, lower_bount_beta)
            step = _mm_upper((t1 - t2).triu(), promote(q))  # q is upper triangular as well
            if store_triu_as_line:
                step = triu_to_line([step])[0][1]
        target = oq_i[1] if isinstance(oq_i, tuple) else oq_i
        ell = ell.view(-1, *([1] * (step.ndim - 1)))
        copy_stochastic_(target, promote(target) - step / ell * precond_lr)


def psgd_pro_update_precond(G, precond_lr, Q, running_lower_bound, lower_bount_beta, power_iter, dampening,
                            max_step_size: float = 1 / 8):  # fmt: skip
    """PRO (Q^0.5 E Q^1.5) update: whiten-to-identity step followed by a second-order rotation that
    keeps each dense factor close to symmetric."""
    psgd_balance_Q(Q)
    exprs = calcG_expr(ndim_tuple(Q), G.ndim)
    noise = dampening + torch.finfo(torch.float32).eps * G.abs()
    Pg = psgd_precond_grad(G + noise * torch.randn_like(G), Q)
    total = G.numel()
    for q, expr, lb in zip(Q, exprs, running_lower_bound):
        cov = compiled_einsum(expr, Pg, Pg)
        q32 = promote(q)
        if q.ndim < 3:
            target = total / max(1, q.numel())
            ell = _update_lb((cov if q.ndim == 1 else cov.amax(dim=-1)) + target, lb, lower_bount_beta)
            ell = ell if q.ndim == 1 else ell.unsqueeze(-1)
            copy_stochastic_(q, q32 - q32 * (cov - target) / ell * precond_lr)
            continue
        target = total / (q.shape[0] * q.shape[-1])
        ell = _update_lb(max_eigenvalue_spd(cov, power_iter=power_iter) + target, lb, lower_bount_beta)
        q32 = q32 - (_mm(cov, q32) - target * q32) / ell[..., None, None] * precond_lr
        R = (q32.mT - q32).contiguous()
        R = R / (max_singular_value(R, power_iter=power_iter)[..., None, None] + torch.finfo(R.dtype).smallest_normal)
        RQ = _mm(R, q32)
        RRQ = _mm(R, RQ)
        c1 = RQ.diagonal(dim1=-2, dim2=-1).sum(dim=-1)
        c2 = RRQ.diagonal(dim1=-2, dim2=-1).sum(dim=-1)
        a = torch.where(c2 < 0, (-c1 / c2).clamp(min=0, max=0.5), 0.5)[..., None, None]
        copy_stochastic_(q, q32 + a * RQ + (0.5 * a * a) * RRQ)


# ---------------------------------------------------------------------------------------- Kron: apply


def precond_grad_cached_(ea: Tensor, cached_q: List[Tensor], caution: bool = False, grad: Optional[Tensor] = None):
    if caution:
        ea = _core._caution_impl(grad, ea)
    return _kron_apply(promote(ea), [promote(q) for q in cached_q], twice=False)


def psgd_precond_grad(ea: Tensor, preconds, caution: bool = False, grad: Optional[Tensor] = None,
                      store_triu_as_line: bool = False, sqrt: bool = False):  # fmt: skip
    """``P g`` with ``P = kron_i Q_i^T Q_i``; ``sqrt=True`` applies each factor once (``Q g``)."""
    if caution:
        ea = _core._caution_impl(grad, ea)
    if store_triu_as_line:
        preconds = line_to_triu(preconds)
    qs = [promote(q) for q in preconds]
    return _kron_apply(promote(ea), qs, twice=not sqrt)


def fused_precond_grad_cached_(ea, param, lr, grad, decay, caution, cached_q, cautious_decay: bool = False):
    out = precond_grad_cached_(ea, cached_q, caution=caution, grad=grad)
    update_param_(param, out, lr, decay, caution=False, cautious_decay=cautious_decay)


def fused_psgd_precond_grad(ea, param, lr, grad, decay, caution, preconds, store_triu_as_line: bool = False,
                            cautious_decay: bool = False, sqrt: bool = False):  # fmt: skip
    out = psgd_precond_grad(ea, preconds, caution=caution, grad=grad, store_triu_as_line=store_triu_as_line, sqrt=sqrt)
    update_param_(param, out, lr, decay, caution=False, cautious_decay=cautious_decay)


# ---------------------------------------------------------------------------------------- LRA


def low_rank_mm(U: Tensor, V: Tensor, x: Tensor) -> Tensor:
    """``(I + U V^T) x`` without forming the matrix."""
    dtype = min_dtype([U, V, x])
    # contracted right to left (V^T x first): the intermediate is rank-sized, never numel x numel
    return x + (U.to(dtype) @ (V.to(dtype).T @ x.to(dtype))).to(x.dtype)


def lra_precond(U: Tensor, V: Tensor, d: Tensor, g: Tensor):
    """``P g`` with ``Q = (I + U V^T) diag(d)`` and ``P = Q^T Q``."""
    return d * low_rank_mm(V, U, low_rank_mm(U, V, d * g))


def _lra_flatten_and_balance(U, V, d):
    """Equalises ``|U|_F`` and ``|V|_F`` (their product is what matters) by ``(|U| / |V|)^1/2`` and returns the flat
    ``[numel, rank]`` / ``[numel]`` views of the three parts."""
    sq = [sum(t.square().sum().double() for t in side) for side in (U, V)]
    ratio = (sq[0] / sq[1]) ** 0.25
    usable = torch.isfinite(ratio) & (ratio > 1e-6)
    ratio = torch.where(usable, ratio, torch.ones_like(ratio))
    stochastic_multiply_(U, [ratio.reciprocal()] * len(U))
    stochastic_multiply_(V, [ratio] * len(V))
    return multi_flatten((U, 1), (V, 1), (d, 0))


def _d_step(d, d_orig, invQtv, vector, inv_precond_vector, hessian_vector, precond_hessian_vector, eps, step, delayed):
    Ph, h, v = promote(precond_hessian_vector), promote(hessian_vector), promote(vector)
    inv = promote(invQtv) - promote(inv_precond_vector)
    d32 = promote(d)
    nabla = d32.square() * Ph * h - v * inv
    # normaliser: product of the two largest sketch entries, re-evaluated in fp64 at the arg-max
    a0, a1, b0, b1 = d32 * Ph, v, inv / d32, h
    idx = ((a0.square() + a1.square()) * (b0.square() + b1.square())).bfloat16().flatten().argmax().reshape(1)
    pick = lambda t: t.index_select(0, idx).double().square()  # noqa: E731
    div = ((pick(a0) + pick(a1)) * (pick(b0) + pick(b1))).sqrt().clamp(min=eps)
    scale = (-step / div).to(nabla.dtype)
    apply_flat_add(d_orig, nabla, scale)
    if not delayed:
        copy_stochastic_(d, d32 - nabla * scale)


def _skinny_gram(A: Tensor, B: Tensor) -> Tensor:
    """``A^T B`` for tall matrices ``[n, r]`` with a small ``r``: on sm_100a one pass of the long-dimension product
    kernel (partial sums per slice of rows, added up afterwards); the library runs this shape as a SIMT GEMM with the
    whole reduction inside one tile."""
    if (A.is_cuda and A.dtype == torch.float32 and B.dtype == torch.float32 and A.ndim == 2 and A.shape == B.shape
            and A.shape[1] <= 32 and A.is_contiguous() and B.is_contiguous()):  # fmt: skip
        from .. import ops

        if ops.available():
            ops.launch_counter.count += 1
            return ops.load().tall_t_mul(A.unsqueeze(0), A.shape[1], B.unsqueeze(0)).sum(0)[0]
    return compiled_einsum("br,bn->rn", A, B)


def update_lra_precond_(U, V, d, vector, hessian_vector, eps, step, delayed, precond_u):
    """One fitting step of the low-rank preconditioner (alternating between ``U`` and ``V``)."""
    U_orig, V_orig, d_orig = U, V, d
    U, V, d = _lra_flatten_and_balance(U, V, d)
    dtype = min_dtype([U, V, vector, hessian_vector])
    U, V, d, vector, hessian_vector = (t.to(dtype) for t in (U, V, d, vector, hessian_vector))

    Qh = low_rank_mm(U, V, d * hessian_vector)
    Ph = low_rank_mm(V, U, Qh)
    rank = U.size(1)
    VtU = _skinny_gram(V, U)
    IpVtU = torch.eye(rank, dtype=VtU.dtype, device=VtU.device) + VtU
    invQtv = vector / d

    back = lambda: (U.to(U_orig[0].dtype), V.to(V_orig[0].dtype), d.to(d_orig[0].dtype))  # noqa: E731
    try:
        LU, piv = torch.linalg.lu_factor(promote(IpVtU))
    except RuntimeError:  # singular factor: skip this fitting step, retry on the next one
        return back()
    rhs = (U.T @ invQtv).view(-1, 1).to(LU.dtype)
    invQtv = invQtv - (V @ torch.linalg.lu_solve(LU, piv, rhs, adjoint=True).to(V.dtype)).flatten()
    rhs = (V.T @ invQtv).view(-1, 1).to(LU.dtype)
    invPv = (U @ torch.linalg.lu_solve(LU, piv, rhs).to(U.dtype)).flatten()

    _d_step(d, d_orig, invQtv, vector, invPv, hessian_vector, Ph, eps, step, delayed)

    a, b = Qh, invQtv
    fac = V if precond_u else U
    atV = compiled_einsum("b,br->r", a, fac)
    btV = compiled_einsum("b,br->r", b, fac)
    atVVt = compiled_einsum("r,br->b", atV, fac)
    btVVt = compiled_einsum("r,br->b", btV, fac)
    precond_step = step / (a.norm() * atVVt.norm() + b.norm() * btVVt.norm()).clamp(min=eps)
    if precond_u:
        a = compiled_einsum("b,r,rg->bg", a, atV, IpVtU)
        b = compiled_einsum("b,r,rg->bg", b, btV, IpVtU)
    else:
        a = compiled_einsum("b,r->br", a + compiled_einsum("br,r->b", V, atV), atV)
        b = compiled_einsum("b,r->br", b + compiled_einsum("br,r->b", V, btV), btV)
    apply_flat_add(U_orig if precond_u else V_orig, b - a, precond_step)
    if not delayed:
        stochastic_add_([U if precond_u else V], [b - a], precond_step)
    return back()


def apply_lra_update(params, update, U, V, d, lr, decay, caution, grads, cautious_decay: bool = False):
    params, grads = list_guard(params, grads)
    flat = lra_precond(U, V, d, flatten(list_guard(update))).flatten()
    start = 0
    for p, g in zip(params, grads):
        n = p.numel()
        update_param_(p, flat[start : start + n].view_as(p), lr, decay, caution, cautious_decay, g)
        start += n
