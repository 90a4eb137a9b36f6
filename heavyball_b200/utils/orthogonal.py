"""Matrix orthogonalisation (zeroth power / polar factor): quintic Newton–Schulz, Polar Express,
QR and SVD modes, plus the Scion linear-minimisation oracles built on top of them.

Behavioural parity targets: ``heavyball/utils.py:550-657`` (iterations and coefficient tables),
``heavyball/utils.py:784-821`` (mode dispatch and scaling), ``heavyball/utils.py:660-733`` (Scion).

Each polynomial step maps ``X -> (a I + b S + c S^2) X`` with ``S = X X^T``.  On sm_100a the chain runs
as three tcgen05 GEMMs per step (``heavyball_b200.ops.newton_schulz``): the Gram matrix and the
polynomial are symmetric, so only upper-triangular tiles are computed and mirrored; the diagonal
shifts are folded into the GEMM epilogues.  The PyTorch code below is the numerics reference for
that kernel and the path taken on CPU, for fp64 inputs and for batches the kernel does not cover.
"""

from __future__ import annotations

import enum
import itertools
import math
import sys
from typing import List, Union

import torch
from torch import Tensor

from .core import copy_stochastic_, list_guard, promote, stochastic_divide_, stochastic_divide_with_eps_, stochastic_round_
from .core import _mm, _solve_right_upper, _tc_sub_product


def _settings():
    return sys.modules[__package__]


class ZerothPowerMode(enum.Enum):
    newtonschulz = "newtonschulz"
    legacy_newtonschulz = "legacy_newtonschulz"
    qr = "qr"
    svd = "svd"
    legacy_svd = "legacy_svd"
    thinky_polar_express = "thinky_polar_express"


class OrthoScaleMode(enum.Enum):
    none = "none"
    scale = "scale"
    graft = "graft"


# Per-step (a, b, c) of the quintic used by Muon's five-step iteration.
NS5_COEFFS = (
    (4.0848, -6.8946, 2.9270),
    (3.9505, -6.3029, 2.6377),
    (3.7418, -5.5913, 2.3037),
    (2.8769, -3.1427, 1.2046),
    (2.8366, -3.0525, 1.2012),
)

# Polar Express (arXiv:2505.16932v3) minimax polynomials.
ABC_LIST = [
    (8.28721201814563, -23.595886519098837, 17.300387312530933),
    (4.107059111542203, -2.9478499167379106, 0.5448431082926601),
    (3.9486908534822946, -2.908902115962949, 0.5518191394370137),
    (3.3184196573706015, -2.488488024314874, 0.51004894012372),
    (2.300652019954817, -1.6689039845747493, 0.4188073119525673),
    (1.891301407787398, -1.2679958271945868, 0.37680408948524835),
    (1.8750014808534479, -1.2500016453999487, 0.3750001645474248),
    (1.875, -1.25, 0.375),
]
_SAFETY = 1.01
ABC_LIST_STABLE = [(a / _SAFETY, b / _SAFETY**3, c / _SAFETY**5) for a, b, c in ABC_LIST[:-1]] + [ABC_LIST[-1]]

LEGACY_COEFFS = (3.4445, -4.7750, 2.0315)


def _poly_step(x: Tensor, a: float, b: float, c: float) -> Tensor:
    s = x @ x.mT
    y = c * s
    y.diagonal(dim1=-2, dim2=-1).add_(b)
    y = y @ s
    y.diagonal(dim1=-2, dim2=-1).add_(a)
    return y @ x


def _iterate(G: Tensor, coeffs, eps: float) -> Tensor:
    tall = G.size(-2) > G.size(-1)
    Gn = G / G.norm(dim=(-2, -1), keepdim=True).clamp(min=eps)
    x = Gn if G.dtype == torch.float64 else stochastic_round_(Gn)
    if tall:
        x = x.mT
    for a, b, c in coeffs:
        x = _poly_step(x, a, b, c)
    if tall:
        x = x.mT
    return x.to(G.dtype)


def _device_kernel(G: Tensor, coeffs):
    """Returns the fused sm_100a implementation's result, or ``None`` when it does not apply."""
    if not G.is_cuda or G.dtype == torch.float64:
        return None
    from .. import ops

    if not ops.available():
        return None
    return ops.newton_schulz(G, coeffs)


def zeropower_via_newtonschulz5(G: Tensor, steps: int = 5, eps: float = 1e-7) -> Tensor:
    assert G.ndim >= 2
    assert steps == 5
    out = _device_kernel(G, NS5_COEFFS)
    return out if out is not None else _iterate(G, NS5_COEFFS, eps)


def msign(G: Tensor, steps: int = 10, eps: float = 1e-7) -> Tensor:
    """Polar Express iteration for the matrix sign / polar factor."""
    assert G.ndim >= 2
    coeffs = [ABC_LIST_STABLE[min(i, len(ABC_LIST_STABLE) - 1)] for i in range(steps)]
    out = _device_kernel(G, coeffs)
    return out if out is not None else _iterate(G, coeffs, eps)


def legacy_zeropower_via_newtonschulz5(G: Tensor, steps: int = 5, eps: float = 1e-7) -> Tensor:
    assert G.ndim == 2
    x = G.clone()
    x = x if G.dtype == torch.float64 else stochastic_round_(x)
    stochastic_divide_with_eps_(x, G.norm(dim=(-2, -1)), eps)
    tall = G.size(0) > G.size(1)
    if tall:
        x = x.T
    for _ in range(steps):
        x = _poly_step(x, *LEGACY_COEFFS)
    if tall:
        x = x.T
    return x.to(G.dtype)


def _compilable_grafting(magnitude: Tensor, direction: Tensor) -> Tensor:
    return direction * (magnitude.norm() / direction.norm().clamp(min=1e-6))


_QR_PANEL = 32
_QR_PASSES = 3


def _panel_cholesky_qr(x: Tensor, defer_check: bool = False):
    """Orthonormal basis of the columns of ``x`` (``... x n x k``, ``n >= k``), equal to the Q factor of
    Householder QR up to the sign of each column, built from batched GEMM / POTRF / TRSM only.

    Householder QR on the GPU factorises one matrix of a batch at a time, column by column, and
    synchronises with the host; an eigenbasis refresh spends nearly all of its time there.  Here the
    columns are taken in panels of 32.  A panel is projected off the basis found so far (block
    Gram-Schmidt), its columns are normalised, and the panel itself is orthogonalised by Cholesky QR
    (``W^T W = L L^T``, ``W <- W L^-T``); the three steps are repeated three times.  Plain Cholesky QR
    of the whole matrix squares its condition number and fails for the matrices met here (``GG @ Q_old``
    with eigenvalues spread over many decades); within a panel, after the projection has removed the
    dominant directions, the columns are of similar size and nearly orthogonal.  Three passes keep
    ``|Q^T Q - I|`` at fp32 rounding level for spectra spanning 20 decades with an arbitrary ``Q_old``.

    Measured alternatives: a two-level scheme (256-column blocks projected with wide GEMMs, panels inside)
    needs a fourth Cholesky sweep to stay orthogonal and was slower (every skinny product over the long
    dimension costs about 18 us regardless of its width); 64-column panels fail on spectra that fall by more
    than about 0.05 decades per column.

    Returns ``None`` when a panel's Gram matrix is not positive definite or the result is not finite
    (e.g. an all-zero input); the caller then uses Householder QR.  One host synchronisation, at the end.
    With ``defer_check`` nothing is read on the host: the result comes back with one failure count per matrix."""
    batch, (n, k) = x.shape[:-2], x.shape[-2:]
    a = x.reshape(-1, n, k)
    tiny = torch.finfo(a.dtype).tiny
    a = a / a.norm(dim=-2, keepdim=True).clamp_(min=tiny)
    q = torch.empty_like(a)
    bad = torch.zeros(a.shape[0], dtype=torch.int32, device=a.device)
    ext = _skinny_kernels(a)
    for j in range(0, k, _QR_PANEL):
        w = a[..., j : j + _QR_PANEL]
        w = w.contiguous() if ext is not None else w
        done = q[..., :j]
        for _ in range(_QR_PASSES):
            if ext is not None and not w.is_contiguous():  # the triangular solve may hand back a column-major panel
                w = w.contiguous()
            if j:  # w -= done (done^T w); the inner product runs over the long dimension
                coef = ext.tall_t_mul(q, j, w).sum(0) if ext is not None else done.mT @ w
                w = torch.baddbmm(w, done, coef, alpha=-1.0)
            # column scales come from the Gram diagonal (no separate reduction over the long dimension):
            # chol(D G D) with D = diag(G)^-1/2 is the factor of the unit-column panel w D
            gram = ext.tall_t_mul(w, w.shape[-1], w).sum(0) if ext is not None else w.mT @ w
            d = gram.diagonal(dim1=-2, dim2=-1).clamp(min=tiny).rsqrt()
            chol, info = torch.linalg.cholesky_ex(gram * d.unsqueeze(-1) * d.unsqueeze(-2))
            bad += info.ne(0)
            w = torch.linalg.solve_triangular(chol.mT, w * d.unsqueeze(-2), upper=True, left=False)
        q[..., j : j + _QR_PANEL] = w
    bad += (~torch.isfinite(q)).flatten(1).any(dim=1)
    if defer_check:  # caller reads the flags (used under CUDA graph capture, where the host cannot)
        return q.reshape(*batch, n, k), bad
    if int(bad.sum()):
        return None
    return q.reshape(*batch, n, k)


def _skinny_kernels(a: Tensor):
    """The extension when its tall-and-skinny product kernels apply (fp32 CUDA input on sm_100a), else ``None``."""
    if not (a.is_cuda and a.dtype == torch.float32):
        return None
    from .. import ops

    return ops.load() if ops.available() else None


_CHOL_LEAF = 128
_CHOLQR_MIN = 256  # below this width the panel-wise method is already cheap


def _chol_upper_blocked(G: Tensor, R: Tensor, bad: Tensor, lo: int, hi: int, inv: Tensor = None):
    """Upper Cholesky factor of the (batched) SPD block ``G[lo:hi, lo:hi]`` into ``R[lo:hi, lo:hi]``, recursively:
    ``R11 = chol(G11)``, ``R12 = R11^-T G12``, ``R22 = chol(G22 - R12^T R12)``.  Only the 128-wide leaves are
    factorisations proper (one kernel for the whole batch, which also leaves the leaf's inverse in ``inv`` for every
    triangular solve that follows; the library's batched factorisation where the extension does not apply); the
    triangular solves and Schur complements are matrix products, which on sm_100a run on the tensor cores.  ``G`` is
    overwritten; ``bad`` counts failed leaves per matrix."""
    n = hi - lo
    if n <= _CHOL_LEAF:
        if inv is not None:
            from .. import ops

            ops.load().chol_inv_leaf(G, R, inv, lo, n, bad)
            ops.launch_counter.count += 1
            return
        r, info = torch.linalg.cholesky_ex(G[:, lo:hi, lo:hi], upper=True)
        R[:, lo:hi, lo:hi] = r
        bad += info.ne(0)
        return
    mid = lo + max(_CHOL_LEAF, (n // 2) // _CHOL_LEAF * _CHOL_LEAF)
    _chol_upper_blocked(G, R, bad, lo, mid, inv)
    # X^T R11 = G12^T  <=>  X = R11^-T G12 = R12
    xt = _solve_right_upper(R[:, lo:mid, lo:mid], G[:, lo:mid, mid:hi].mT.contiguous(), inv, lo // _CHOL_LEAF, consume_b=True)
    R[:, lo:mid, mid:hi] = xt.mT
    if not _tc_sub_product(G[:, mid:hi, mid:hi], xt, xt, b_transposed=True):  # Schur complement, upper tiles mirrored
        G[:, mid:hi, mid:hi] -= _mm(xt, xt, False, True)
    _chol_upper_blocked(G, R, bad, mid, hi, inv)


def _leaf_inverse_buffer(gram: Tensor):
    """Storage for the inverses of the 128-wide diagonal leaves of a batched factor when the extension's leaf kernel
    applies (fp32 CUDA on sm_100a), else ``None``."""
    if _skinny_kernels(gram) is None or gram.ndim != 3:
        return None
    blocks = (gram.shape[-1] + _CHOL_LEAF - 1) // _CHOL_LEAF
    return torch.empty(gram.shape[0], blocks, _CHOL_LEAF, _CHOL_LEAF, device=gram.device, dtype=gram.dtype)


_CHOLQR_SHIFT = 1e-5  # of the Gram matrix's trace bound; one shifted round lowers the condition number ~300-fold
_CHOLQR_ACCEPT = 1e-4  # largest entry of Q^T Q - I that is accepted (a Householder factor reaches ~1e-6 in fp32)


def _cholesky_qr2(x: Tensor, shifted_rounds: int = 0):
    """Cholesky QR on the column-normalised input: ``G = A^T A = R^T R``, ``A <- A R^-1``, repeated.  Everything is
    matrix products plus 128-wide batched Cholesky leaves, so an ``n x n`` basis costs a few milliseconds instead of
    the hundreds of dependent panel steps of :func:`_panel_cholesky_qr`.

    Two plain rounds are valid while the columns are far from dependent (condition number below about ``eps^-1/2``),
    which is the usual case once an eigenbasis tracks its statistics.  Worse inputs get ``shifted_rounds`` rounds in
    front that factor ``G + s I`` instead (always positive definite; the result is not yet orthonormal but its
    condition number is lower by about ``sqrt(lambda_max / s)``); the product of all triangular factors is still THE
    triangular factor of ``A``, so every variant returns the same ``Q``.  Whether the input was within reach is read off
    the result: ``Q^T Q`` must be the identity to 1e-4 (one more symmetric product).  Returns ``(q, bad)`` with one
    failure count per matrix, nothing read on the host."""
    batch, (n, k) = x.shape[:-2], x.shape[-2:]
    a = x.reshape(-1, n, k)
    tiny = torch.finfo(a.dtype).tiny
    a = a / a.norm(dim=-2, keepdim=True).clamp_(min=tiny)
    bad = torch.zeros(a.shape[0], dtype=torch.int32, device=a.device)
    eye = torch.eye(k, device=a.device, dtype=a.dtype)
    rounds = shifted_rounds + 2
    info = torch.zeros_like(bad)  # failed leaves do not decide: what counts is the orthogonality reached at the end
    for rnd in range(rounds):
        gram = _mm(a, a, True, False)
        if rnd < shifted_rounds:
            # unit columns: the diagonal is 1 and lambda_max <= k
            gram.diagonal(dim1=-2, dim2=-1).add_(_CHOLQR_SHIFT * k)
        r = torch.zeros_like(gram)
        inv = _leaf_inverse_buffer(gram)
        _chol_upper_blocked(gram, r, info, 0, k, inv)
        a = _solve_right_upper(r, a, inv, 0, consume_b=rnd > 0 or a.data_ptr() != x.data_ptr())
        if rnd < shifted_rounds:  # columns shrank by different amounts: back to unit columns for the next round
            a = a / a.norm(dim=-2, keepdim=True).clamp_(min=tiny)
    bad += (_mm(a, a, True, False) - eye).abs().amax(dim=(-2, -1)).gt(_CHOLQR_ACCEPT)
    bad += (~torch.isfinite(a)).flatten(1).any(dim=1)
    return a.reshape(*batch, n, k), bad


_cholqr_graphs = {}
_CHOLQR_LADDER = (0, 1, 3)  # shifted rounds in front of the two plain ones, tried in this order
_cholqr_level, _cholqr_wins = {}, {}  # (device, shape) -> where to start on the ladder / successes so far
# how often each variant produced the basis, and how often all were refused (panel-wise route)
qr_stats = {"cholesky_qr2": 0, "cholesky_qr_shifted_1": 0, "cholesky_qr_shifted_3": 0, "cholesky_qr2_rejected": 0}


def _cholesky_qr2_replayed(x: Tensor, shifted_rounds: int = 0):
    """:func:`_cholesky_qr2` through a CUDA graph per (device, shape, variant), like :func:`_panel_qr_replayed`."""
    key = (x.device, tuple(x.shape), shifted_rounds)
    slot = _cholqr_graphs.get(key)
    if slot is None:
        if len(_cholqr_graphs) >= 2 * _QR_GRAPH_LIMIT:
            return _cholesky_qr2(x, shifted_rounds)
        slot = _cholqr_graphs[key] = [0, None]
    slot[0] += 1
    if slot[1] is False or slot[0] == 1 or not _settings().graph_qr:
        return _cholesky_qr2(x, shifted_rounds)
    if slot[1] is None:
        try:
            static_in = x.clone()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                static_out, static_bad = _cholesky_qr2(static_in, shifted_rounds)
            slot[1] = (graph, static_in, static_out, static_bad)
        except Exception as err:  # noqa: BLE001 - any capture failure means "do not graph this shape"
            slot[1] = False
            import warnings

            warnings.warn(f"CUDA graph capture of the Cholesky QR failed ({type(err).__name__}); running it eagerly")
            return _cholesky_qr2(x, shifted_rounds)
    graph, static_in, static_out, static_bad = slot[1]
    static_in.copy_(x)
    graph.replay()
    return static_out, static_bad


_qr_graphs = {}  # (device, shape) -> [calls seen, (graph, input, output, failure flag) | None | False]
_QR_GRAPH_LIMIT = 16


def _panel_qr_replayed(x: Tensor, fallback: Tensor = None):
    """:func:`_panel_cholesky_qr` through a CUDA graph per (device, shape): an eigenbasis refresh of a
    1024-wide factor is several hundred small launches, and the host, not the GPU, sets its duration.  The first call
    for a shape runs eagerly (library handles and workspaces get created outside capture), the second is
    captured, later ones copy the input into the captured buffer and replay.  If capture is not possible the
    shape stays on the eager path.

    ``fallback`` (same shape, orthonormal columns - the basis being refreshed) makes a replay free of host
    synchronisation: a matrix whose factorisation failed keeps its ``fallback`` columns, chosen on the device."""
    key = (x.device, tuple(x.shape))
    slot = _qr_graphs.get(key)
    if slot is None:
        if len(_qr_graphs) >= _QR_GRAPH_LIMIT:
            return _panel_cholesky_qr(x)
        slot = _qr_graphs[key] = [0, None]
    slot[0] += 1
    if torch.cuda.is_current_stream_capturing():  # part of a larger captured region: no replay, and no host read
        if fallback is None:
            raise RuntimeError("a captured eigenbasis refresh needs a fallback basis (the host cannot read failure flags)")
        out, bad = _panel_cholesky_qr(x, defer_check=True)
        return torch.where(bad.view(*x.shape[:-2], 1, 1) > 0, fallback.to(out.dtype), out)
    if slot[1] is False or slot[0] == 1:
        return _panel_cholesky_qr(x)
    if slot[1] is None:
        try:
            static_in = x.clone()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                static_out, static_bad = _panel_cholesky_qr(static_in, defer_check=True)
            slot[1] = (graph, static_in, static_out, static_bad)
        except Exception as err:  # noqa: BLE001 - any capture failure means "do not graph this shape"
            slot[1] = False
            import warnings

            warnings.warn(f"CUDA graph capture of the refresh QR failed ({type(err).__name__}); running it eagerly")
            return _panel_cholesky_qr(x)
    graph, static_in, static_out, static_bad = slot[1]
    static_in.copy_(x)
    graph.replay()
    if fallback is not None:
        failed = static_bad.view(*x.shape[:-2], 1, 1) > 0
        return torch.where(failed, fallback.to(static_out.dtype), static_out)
    if int(static_bad.sum()):
        return None
    return static_out.clone()


def _qr_basis(x: Tensor, fallback: Tensor = None) -> Tensor:
    """Q factor of ``x``.  ``fallback``: orthonormal matrix to keep where the fast factorisation fails (see
    :func:`_panel_qr_replayed`); without it a failure costs a host synchronisation and Householder QR."""
    x32 = promote(x)
    if (x32.is_cuda and _settings().fast_qr and x32.shape[-2] >= x32.shape[-1] >= _CHOLQR_MIN
            and not torch.cuda.is_current_stream_capturing()):  # fmt: skip
        xc = x32.contiguous()
        key = (xc.device, tuple(xc.shape))
        start = _cholqr_level.get(key, 0)
        for level in range(start, len(_CHOLQR_LADDER)):
            q, bad = _cholesky_qr2_replayed(xc, _CHOLQR_LADDER[level])
            if int(bad.sum()) == 0:  # one host read per attempt; a failure climbs the ladder, then takes the panel-wise route
                qr_stats["cholesky_qr2" if level == 0 else f"cholesky_qr_shifted_{_CHOLQR_LADDER[level]}"] += 1
                # start where it worked next time, and try one step cheaper every eighth success
                wins = _cholqr_wins[key] = _cholqr_wins.get(key, 0) + 1
                _cholqr_level[key] = max(0, level - 1) if wins % 8 == 0 else level
                return q.clone() if q.data_ptr() != x32.data_ptr() else q
        _cholqr_level[key] = len(_CHOLQR_LADDER) - 1
        qr_stats["cholesky_qr2_rejected"] += 1
    if x32.is_cuda and _settings().fast_qr and x32.shape[-2] >= x32.shape[-1] >= 2 * _QR_PANEL:
        q = _panel_qr_replayed(x32.contiguous(), fallback) if _settings().graph_qr else _panel_cholesky_qr(x32)
        if q is not None:
            return q
    return torch.linalg.qr(x32).Q


def _compilable_orthogonal_(x: Tensor, mode, out, scale_mode):
    mode = mode if isinstance(mode, ZerothPowerMode) else ZerothPowerMode(mode)
    scale_mode = scale_mode if isinstance(scale_mode, OrthoScaleMode) else OrthoScaleMode(scale_mode)
    if mode is ZerothPowerMode.newtonschulz or x.shape[-2] != x.shape[-1]:
        y = zeropower_via_newtonschulz5(x, 5)
    elif mode is ZerothPowerMode.thinky_polar_express:
        y = msign(x, 10)
    elif mode is ZerothPowerMode.legacy_newtonschulz:
        y = legacy_zeropower_via_newtonschulz5(x, 5)
    elif mode is ZerothPowerMode.qr:
        y = _qr_basis(x)
    elif mode is ZerothPowerMode.svd:
        u, _, vt = torch.linalg.svd(promote(x))
        y = u @ vt
    elif mode is ZerothPowerMode.legacy_svd:
        u, _, vt = torch.linalg.svd(promote(x))
        y = u @ vt.T
    else:
        raise NotImplementedError(f"Unknown zeroth_power_mode: {mode}")
    if scale_mode is OrthoScaleMode.scale:
        y = y * max(1, x.size(-2) / x.size(-1)) ** 0.5
    elif scale_mode is OrthoScaleMode.graft:
        y = _compilable_grafting(x, y)
    if out is None:
        return y
    out.copy_(y)


def inplace_orthogonal_(x: Tensor, mode=None, out=None, scale_mode: str = "none"):
    return _compilable_orthogonal_(x, mode or _settings().zeroth_power_mode, out, scale_mode)


# ---------------------------------------------------------------------------------------- Scion


def _scion_bias_rms_direction(x: Tensor, eps: float = 1e-8) -> Tensor:
    if x.ndim == 0:
        return x / x.abs().clamp(min=eps)
    rms = x.square().mean(dim=0, keepdim=True).sqrt()
    stochastic_divide_(x, rms, eps=eps)
    return x


def _scion_matrix_direction(x: Tensor, conv: bool) -> Tensor:
    flat = inplace_orthogonal_(x.reshape(x.shape[0], -1))
    if conv:
        spatial = math.prod(x.shape[2:]) if x.ndim > 2 else 1
        scale = math.sqrt(x.shape[0] / max(x.shape[1], 1)) / max(spatial, 1)
    else:
        scale = math.sqrt(x.shape[0] / max(flat.shape[1], 1))
    return flat.reshape_as(x) * scale


def _scion_batched_matrices(update: List[Tensor], scale: float) -> List[Tensor]:
    """Runs the spectral LMO of all 2-D tensors that the Newton-Schulz kernels accept, one batched iteration per shape,
    and returns the tensors that are left for the per-tensor definitions."""
    mode = _settings().zeroth_power_mode
    if str(getattr(mode, "value", mode)) != "newtonschulz" or not update or not update[0].is_cuda:
        return update
    from .. import ops

    if not ops.available():
        return update
    buckets, rest = {}, []
    for t in update:
        if (t.ndim == 2 and t.is_cuda and t.dtype in (torch.float32, torch.bfloat16) and t.is_contiguous()
                and ops.ns_supported(t.shape[0], t.shape[1])):  # fmt: skip
            buckets.setdefault((tuple(t.shape), t.dtype), []).append(t)
        else:
            rest.append(t)
    for ((rows, cols), _), members in buckets.items():
        out = ops.newton_schulz_batched(members, NS5_COEFFS, out_scale=math.sqrt(rows / max(cols, 1)) * scale)
        for t, d in zip(members, out.unbind(0)):
            copy_stochastic_(t, d)
    return rest


def scion_auto_lmo_(update: Union[List[Tensor], Tensor], scale):
    """Norm-constrained LMO chosen by rank: spectral (matrices), unfolded spectral (conv kernels),
    RMS (vectors, scalars)."""
    update = list_guard(update)
    update = _scion_batched_matrices(update, float(scale))  # same-shape matrices in one batched iteration on sm_100a
    for t in update:
        t32 = promote(t)
        if t32.ndim in (3, 4):
            d = _scion_matrix_direction(t32, True)
        elif t32.ndim == 2:
            d = _scion_matrix_direction(t32, False)
        else:
            d = _scion_bias_rms_direction(t32.clone() if t32 is t else t32)
        copy_stochastic_(t, d * float(scale))
    return update


def scion_auto_init_param_(param: Tensor, scale, seed: int = 0):
    """Deterministic (CPU, fp64, seeded) orthogonal re-initialisation of matrices; zeros for the
    rest.  Matches the norm ball the Scion LMO moves on."""
    p32 = promote(param)
    gen = torch.Generator(device="cpu")
    gen.manual_seed(seed)
    if param.ndim >= 2:
        w = p32.clone().cpu().double()
        for idx in itertools.product(*(range(s) for s in w.shape[2:])):
            torch.nn.init.orthogonal_(w[(slice(None), slice(None), *idx)], generator=gen)
        spatial = math.prod(w.shape[2:])
        w.mul_(math.sqrt(w.shape[0] / max(w.shape[1], 1)) / max(spatial, 1))
        init = w.to(dtype=p32.dtype, device=p32.device)
    else:
        init = torch.zeros_like(p32)
    init.mul_(float(scale))
    copy_stochastic_(param, init.to(dtype=param.dtype, device=param.device))
