"""Shampoo / SOAP algebra: Kronecker-factor statistics, eigenbasis projection and refresh.

All tensors carry a leading *slot* dimension (size = number of same-shape parameters batched
together), so a factor for a mode of size ``d`` is ``(slots, d, d)``.

Behavioural parity targets: ``heavyball/utils.py:1362-1411`` (init, projection),
``heavyball/utils.py:1205-1278`` (statistics, KL variants), ``heavyball/utils.py:829-1038``
(eigenbasis refresh, PSGD eigenbasis, robust eigh), ``heavyball/utils.py:240-287, 3726-3742``
(dimension merging), ``heavyball/utils.py:2409-2418`` (refresh schedules).
"""

from __future__ import annotations

import functools
import gc
import string
import sys
from typing import List, Optional

import torch
from torch import Tensor

from .core import copy_stochastic_, promote, stochastic_lerp_
from .core import _mm, _tc_matmul
from .orthogonal import _qr_basis, inplace_orthogonal_

einsum_base = string.ascii_lowercase


def _settings():
    return sys.modules[__package__]


def compiled_einsum(expr, *args):
    return torch.einsum(expr, *args)


def clean():
    if torch.cuda.is_available():
        torch.cuda.empty_cache()
    gc.collect()


# ---------------------------------------------------------------------------------------- shape handling


def append_or_extend(base: list, new):
    (base.extend if isinstance(new, list) else base.append)(new)


def dim_merger(grad: Tensor, max_precond_dim: int, split: bool = False):
    """Greedily merges trailing dims (never fan-out into fan-in) while the product stays within
    ``max_precond_dim``; with ``split`` also cuts over-long dims into chunks."""
    merged, run = [], 1
    for s in reversed(grad.shape[1:]):
        if run * s > max_precond_dim:
            if run > 1:
                merged.append(run)
                run = s
            else:
                merged.append(s)
                run = 1
        else:
            run *= s
    if run > 1:
        merged.append(run)
    shape = [grad.shape[0], *reversed(merged)]
    out = grad.reshape(shape)
    if not split:
        return out

    pieces = [out]
    for i in reversed(range(len(shape))):
        if shape[i] == 1:
            pieces = [p.squeeze(dim=i) for p in pieces]
        elif shape[i] > max_precond_dim:
            pieces = [c for p in pieces for c in p.split(max_precond_dim, dim=i)]
    if len(pieces) == 1:
        return out
    result = []
    for p in pieces:
        append_or_extend(result, dim_merger(p, max_precond_dim, split))
    return result


def merge_group(group, *tensors):
    if not group.get("merge_dims", False):
        return tensors
    if isinstance(tensors[0], list):
        return [merge_group(group, *t) for t in tensors]
    limit = group["max_size_triangular"] if "max_size_triangular" in group else group["max_precond_dim"]
    out = []
    for t in tensors:
        append_or_extend(out, dim_merger(t, limit, group.get("split", False)))
    return out


# ---------------------------------------------------------------------------------------- refresh schedule


def precond_schedule(step, precond_scheduler):
    p = torch.as_tensor(step, dtype=torch.float32).clamp(min=1) ** precond_scheduler[0]
    p = torch.log10(p) ** precond_scheduler[1] + 1
    return 1 / p


def get_soap_precond_schedule(precond_scheduler):
    return functools.partial(precond_schedule, precond_scheduler=precond_scheduler)


# ---------------------------------------------------------------------------------------- eigen decompositions


def _is_device_failure(err: RuntimeError, m: Tensor) -> bool:
    return m.is_cuda and ("CUDA" in str(err) or "illegal memory access" in str(err))


def _stable_symmetric_basis(m: Tensor, max_eps: float = 1e-3, min_eps: float = 1e-30, *, out_device=None, out_dtype=None):
    """Eigenvectors of a symmetric matrix, largest eigenvalue first.  ``eigh`` is retried down a ladder until it succeeds:
    out of device memory or a device-side solver failure -> the same problem on the CPU; a failure in fp32 -> fp64; a
    failure in fp64 -> more diagonal jitter (``eps <- eps^(2/3)``, starting at ``min_eps``) up to ``max_eps``."""
    target = dict(device=m.device if out_device is None else out_device, dtype=m.dtype if out_dtype is None else out_dtype)
    work, jitter = promote(m.data), min_eps
    while True:
        to_cpu = False
        try:
            shifted = work + jitter * torch.eye(work.shape[-1], device=work.device, dtype=work.dtype)
            vectors = torch.linalg.eigh(shifted)[1]
            return vectors.flip(-1).contiguous().to(**target)
        except torch.OutOfMemoryError:
            if not work.is_cuda:
                raise
            to_cpu = True
        except RuntimeError as err:
            if _is_device_failure(err, work):
                to_cpu = True
            elif work.dtype != torch.float64:
                work = work.double()
            elif jitter < max_eps:
                jitter = jitter ** (2 / 3)
            else:
                raise
        if to_cpu:
            torch.cuda.synchronize(work.device)
            clean()
            work = work.cpu()
        clean()


def get_orthogonal_matrix(mat, max_eps: float = 1e-3, min_eps: float = 1e-30):
    return [None if m is None else _stable_symmetric_basis(m, max_eps=max_eps, min_eps=min_eps) for m in mat]


# ---------------------------------------------------------------------------------------- statistics


def _skip_stats(grad: Tensor, max_precond_dim, precondition_1d) -> bool:
    return grad.dim() == 2 and (not precondition_1d or grad.shape[1] > max_precond_dim)


def _mode_outer_expr(ndim_without_slot: int, idx: int) -> str:
    g0 = einsum_base[:ndim_without_slot]
    b = einsum_base[idx]
    return f"...{g0},...{g0.replace(b, b.upper())}->...{b + b.upper()}"


def update_ggt(grad, GG, max_precond_dim, precondition_1d, beta):
    """``GG_i <- beta GG_i + (1-beta) * G_(i) G_(i)^T`` for every preconditioned mode ``i``."""
    if _skip_stats(grad, max_precond_dim, precondition_1d):
        return
    for idx, m in enumerate(GG):
        if isinstance(m, Tensor):
            outer = None
            if grad.dim() == 3:  # (slot, rows, cols): G G^T / G^T G as one symmetric product
                g32 = promote(grad)
                outer = _tc_matmul(g32, g32, idx == 1, idx == 0)
            if outer is None:
                outer = compiled_einsum(_mode_outer_expr(grad.dim() - 1, idx), grad, grad)
            stochastic_lerp_(m, outer, 1 - beta)


def _kl_eigvals(q: Tensor, m: Tensor) -> Tensor:
    return compiled_einsum("...ji,...jk,...ki->...i", promote(q), promote(m), promote(q))


def update_ggt_kl(grad, GG, Q, max_precond_dim, precondition_1d, beta, eps, *, heavy: bool = False):
    """KL-Shampoo statistics (arXiv:2509.03378): each side's outer product is whitened by the
    other side's current eigenvalues.  Falls back to plain statistics unless the gradient is a
    (slot, rows, cols) matrix with at least one live factor."""
    if _skip_stats(grad, max_precond_dim, precondition_1d):
        return
    if grad.dim() != 3 or not any(isinstance(m, Tensor) and q is not None for m, q in zip(GG, Q)):
        return update_ggt(grad, GG, max_precond_dim, precondition_1d, beta)

    g32 = promote(grad)
    sides = []
    for idx, (m, q) in enumerate(zip(GG, Q)):
        if not isinstance(m, Tensor) or q is None:
            sides.append(None)
            continue
        eig = _kl_eigvals(q, m)
        inv = torch.where(eig > eps, eig.reciprocal(), 0.0) if heavy else eig.clamp_min(eps).reciprocal()
        proj = compiled_einsum("...ji,...jk->...ik" if idx == 0 else "...ij,...jk->...ik", g32, promote(q))
        sides.append((proj, inv / grad.shape[idx + 1]))

    for idx, (m, other) in enumerate(zip(GG, reversed(sides))):
        if not isinstance(m, Tensor):
            continue
        if other is None:
            outer = compiled_einsum(_mode_outer_expr(2, idx), g32, g32)
        else:
            proj, scale = other
            outer = compiled_einsum("...ik,...k,...jk->...ij", proj, scale, proj)
        stochastic_lerp_(m, outer, 1 - beta)


def init_preconditioner(grad, state, max_precond_dim, precondition_1d, init_factor: float = 0.0):
    """Creates ``state['GG']`` (one factor per non-slot dim, ``None`` where a dim is skipped) and
    ``state['Q']`` (their eigenbases).  ``init_factor > 0`` seeds ``init_factor * I`` instead of the
    first outer product."""
    gg = []
    if grad.numel() > 1 and (grad.ndim > 2 or precondition_1d):
        n = grad.shape[0]
        for sh in grad.shape[1:]:
            if sh > max_precond_dim or sh == 1:
                gg.append(None)
            elif init_factor > 0:
                eye = torch.eye(sh, device=grad.device, dtype=grad.dtype)
                gg.append(eye.expand(n, sh, sh).contiguous() * init_factor)
            else:
                gg.append(torch.zeros(n, sh, sh, device=grad.device, dtype=grad.dtype))
    else:
        gg.append(None)
    state["GG"] = gg
    if init_factor <= 0:
        update_ggt(grad, gg, max_precond_dim, precondition_1d, 0)
    state["Q"] = get_orthogonal_matrix(gg)


# ---------------------------------------------------------------------------------------- projection


def project(grad, Q, back: bool):
    """Rotates every preconditioned mode into (``back=False``) or out of (``back=True``) its
    eigenbasis: ``G x_1 Q_1^T x_2 Q_2^T ...``"""
    modes = einsum_base[: grad.dim() - 1]
    factors = [f"...{(c + c.upper())[::-1 if back else 1]}" for q, c in zip(Q, modes) if q is not None]
    if not factors:
        return grad
    if grad.dim() == 3 and grad.is_cuda:
        res = promote(grad)
        ok = True
        for idx, q in enumerate(Q):
            if q is None:
                continue
            q32 = promote(q)
            # into the basis: Q_l^T G, G Q_r; out of it: Q_l G, G Q_r^T
            nxt = _tc_matmul(q32, res, not back, False) if idx == 0 else _tc_matmul(res, q32, False, back)
            if nxt is None:
                ok = False
                break
            res = nxt
        if ok:
            return res.to(grad.dtype)
    joined = ",".join(factors)
    out = "".join(c.upper() if c.upper() in joined else c for c in modes)
    res = compiled_einsum(f"...{modes},{joined}->...{out}", promote(grad), *[promote(q) for q in Q if q is not None])
    return res.to(grad.dtype)


def _kl_shampoo_kron_scale(grad: Tensor, Q, GG, eps: float):
    out = promote(grad)
    for idx, (q, m) in enumerate(zip(Q, GG)):
        if q is None or m is None:
            continue
        d = _kl_eigvals(q, m).clamp_min(eps).rsqrt()
        shape = [1] * out.ndim
        shape[0], shape[idx + 1] = d.shape[0], -1
        out = out * d.view(shape)
    return out.to(grad.dtype)


def kl_shampoo_precondition(grad, Q, GG, eps):
    """``(kron_i Q_i diag(d_i^-1/2) Q_i^T) g`` with ``d_i = diag(Q_i^T GG_i Q_i)``."""
    return project(_kl_shampoo_kron_scale(project(grad, Q, back=False), Q, GG, eps), Q, back=True)


# ---------------------------------------------------------------------------------------- eigenbasis refresh


def _basis_change_expr(old, new, ndim_without_slot):
    ins = einsum_base[:ndim_without_slot]
    outs = einsum_base[ndim_without_slot : 2 * ndim_without_slot]
    frm = ",".join(f"...{c.upper()}{c}" for q, c in zip(old, ins) if q is not None)
    if not frm:
        return None
    to = ",".join(f"...{c.upper()}{o}" for q, c, o in zip(new, ins, outs) if q is not None)
    res = "".join(o if o in to else c for c, o in zip(ins, outs))
    return f"...{ins},{frm},{to}->...{res}"


def _rotate_states(old_qs, new_qs, states):
    """Moves tensors expressed in the ``old`` eigenbasis into the ``new`` one (per mode
    ``Q_old Q_new^T`` contraction), in place."""
    states = [s for s in states if s is not None]
    if not states or states[0].dim() <= 1:
        return
    assert states[0].dim() < 14
    expr = _basis_change_expr(old_qs, new_qs, states[0].dim() - 1)
    if expr is None:
        return
    if states[0].dim() == 3 and states[0].is_cuda:
        # matrices: S' = R_l S R_r^T with R = Q_new^T Q_old per side, as tensor-core products
        rots = [None if qo is None else _tc_matmul(promote(qn), promote(qo), True, False) for qo, qn in zip(old_qs, new_qs)]
        if all(r is not None or qo is None for r, qo in zip(rots, old_qs)):
            for s in states:
                out = promote(s)
                if rots[0] is not None:
                    out = _mm(rots[0], out)
                if len(rots) > 1 and rots[1] is not None:
                    out = _mm(out, rots[1], False, True)
                copy_stochastic_(s, out)
            return
    old = [promote(q) for q in old_qs if q is not None]
    new = [promote(q) for q in new_qs if q is not None]
    for s in states:
        copy_stochastic_(s, compiled_einsum(expr, promote(s), *old, *new))


def _transform_projected_state(old_qs, new_qs, *states):
    _rotate_states(old_qs, new_qs, states)


def get_orthogonal_matrix_QR(GG, Q, *exp_avg, exp_avg_sq=None, heavy: bool = False):
    """One step of orthogonal (power) iteration per factor: ``Q <- orth(GG Q)`` with columns kept
    in descending Rayleigh-quotient order, followed by a rotation of the first-moment buffers (and,
    for ``heavy``, a Hadamard-square transport of the second moment) into the new basis."""
    if isinstance(Q, list) and not Q:
        return
    ref = exp_avg[0] if exp_avg else exp_avg_sq
    if ref is not None and ref.dim() <= 1:
        Q.clear()
        return
    if ref is not None and ref.dim() - 1 != len(Q):
        raise ValueError(f"ref dim {ref.dim()} (excluding bucket axis) does not match Q length {len(Q)}")

    precise = _settings().precise_zeroth_power_mode
    new_qs = []
    for m, q in zip(GG, Q):
        if m is None:
            new_qs.append(None)
            continue
        m = promote(m.data)
        if heavy:
            basis = inplace_orthogonal_(_mm(m, promote(q.data)), precise)
            ray = compiled_einsum("...ij,...ij->...j", basis, _mm(m, basis))
            order = torch.argsort(ray, descending=True).unsqueeze(-2).expand_as(basis)
            new_qs.append(basis.gather(-1, order))
            continue
        q_old = promote(q.data)
        power = _mm(m, q_old)
        ray = compiled_einsum("...ij,...ij->...j", q_old, power)
        order = torch.argsort(ray, descending=True).unsqueeze(-2).expand_as(power)
        if str(getattr(precise, "value", precise)) == "qr":
            # the old basis in the new column order is what a factor keeps if its factorisation fails
            basis = _qr_basis(power.gather(-1, order), fallback=q_old.gather(-1, order))
        else:
            basis = inplace_orthogonal_(power.gather(-1, order), precise)
        power.scatter_(-1, order, basis)
        new_qs.append(power)

    if ref is not None:
        if exp_avg:
            _rotate_states(Q, new_qs, exp_avg)
        if heavy and exp_avg_sq is not None and any(q is not None for q in Q):
            nd = ref.dim() - 1
            ins, outs = einsum_base[:nd], einsum_base[nd : 2 * nd]
            rsq = [
                compiled_einsum("...ji,...jk->...ik", promote(qo.data), promote(qn)).square()
                for qo, qn in zip(Q, new_qs)
                if qo is not None
            ]
            terms = ",".join(f"...{c}{o}" for q, c, o in zip(Q, ins, outs) if q is not None)
            res = "".join(o if o in terms else c for c, o in zip(ins, outs))
            moved = compiled_einsum(f"...{ins},{terms}->...{res}", promote(exp_avg_sq), *rsq)
            copy_stochastic_(exp_avg_sq, moved.clamp_min(0))

    for q, q_new in zip(Q, new_qs):
        if q is not None:
            copy_stochastic_(q, q_new)


# ---------------------------------------------------------------------------------------- PSGD eigenbasis (LATHER)


def init_psgd_eigenbasis(Q: List[Tensor]):
    """Per dense factor the eigenbasis of ``Q^T Q`` (``None`` for diagonal factors, whose basis is the identity)."""

    def basis(q):
        if q.ndim < 3:
            return None
        wide = promote(q)
        return _stable_symmetric_basis(_mm(wide, wide, True, False), out_device=q.device, out_dtype=q.dtype)

    return [basis(q) for q in Q]


def get_psgd_eigenbasis(Q: List[Tensor], prev: List[Optional[Tensor]]):
    """One subspace-iteration step on ``Q^T Q``: ``Y = Q^T (Q B)``, QR, sort by ``|Q b|^2``,
    sign-align each column with the previous basis."""
    out = []
    for q, old in zip(Q, prev):
        if q.ndim < 3:
            out.append(None)
            continue
        if old is None:
            raise ValueError("get_psgd_eigenbasis requires a previous basis for matrix blocks; use init_psgd_eigenbasis")
        q32, old32 = promote(q), promote(old)
        raw = _qr_basis(_mm(q32, _mm(q32, old32), True, False)).to(dtype=q.dtype)
        proj = _mm(q32, promote(raw))
        order = torch.argsort(compiled_einsum("...ij,...ij->...j", proj, proj), descending=True)
        raw = raw.gather(-1, order.unsqueeze(-2).expand_as(raw))
        align = compiled_einsum("...ij,...ij->...j", old32, promote(raw))
        signs = torch.where(align < 0, -1.0, 1.0).to(raw.dtype)
        out.append(raw * signs.unsqueeze(-2))
    return out


def update_psgd_eigenbasis(Q: List[Tensor], Q_basis: List[Tensor], *states: Tensor):
    new = get_psgd_eigenbasis(Q, Q_basis)
    _rotate_states(Q_basis, new, states)
    for old, fresh in zip(Q_basis, new):
        if old is not None:
            copy_stochastic_(old, fresh)
