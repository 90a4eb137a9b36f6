"""Batched matrix stages of the lowered SOAP and PSGD programs.

``lowering`` runs a second-order chain as: one multi-tensor launch that turns gradients into fp32 updates laid out
*bucket-major* (all same-shape matrices of a group adjacent, so a bucket is one ``(B, R, C)`` tensor without any
stacking copy), then a **matrix stage** per bucket, then one multi-tensor launch that applies the result to the
parameters.  This module holds the matrix stages.

State layout.  The reference keeps per-parameter state with a leading slot dim of 1 and stacks / unstacks it around
every call (``heavyball/chainable.py:457-584``).  Here a bucket *adopts* its members' state once: the per-member
tensors are concatenated into batched tensors and every member's state entry is replaced by a view ``batched[j:j+1]``
of them.  ``optimizer.state`` (and so ``state_dict()``) still shows tensors of the checkpoint shape, all stage
arithmetic is in place on the batched tensors, and nothing is copied per step.  If the entries are replaced from
outside (``load_state_dict``), the next step notices the changed addresses and adopts again.

Products.  Every product is written against a small operand interface with two backends: the split-tf32 tensor-core
GEMM of ``ops`` (fp32-level accuracy, element-wise stages fused into GEMM epilogues, rarely-changing matrices kept
in split form between refreshes) and plain ``torch`` matmuls (CPU, small matrices, and the oracle in tests).

Math restated from ``heavyball_b200.utils.soap`` / ``utils.psgd`` (parity targets ``heavyball/chainable.py:1257-1276,
1531-1621`` and ``heavyball/utils.py:829-900, 1205-1259, 1391-1411, 3084-3122, 3557-3576``).
"""

from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch
from torch import Tensor

from . import ops, utils
from .utils.core import _mm

MIN_TC_DIM = 128  # below this a 128 x 128 tensor-core tile is mostly padding: use the library product


# ---------------------------------------------------------------------------------------- operand backends


class _TorchOperand:
    """K-major operand for the torch backend: a dense ``[B, rows, K]`` view."""

    __slots__ = ("dense",)

    def __init__(self, dense):
        self.dense = dense


class TorchBackend:
    """Reference semantics of the operand interface with library matmuls."""

    name = "torch"

    @staticmethod
    def operands(x: Tensor, same: bool = True, trans: bool = False):
        return (_TorchOperand(x) if same else None), (_TorchOperand(x.transpose(-1, -2)) if trans else None)

    @staticmethod
    def gemm(a, b, *, mode=ops.EPI_STORE, alpha=1.0, w=0.0, b1=0.0, b2=0.0, eps=0.0, out=None, split_out=ops.SPLIT_NONE,
             m=None, v=None):  # fmt: skip
        acc = torch.matmul(a.dense, b.dense.transpose(-1, -2))
        if alpha != 1.0:
            acc = acc * alpha
        if mode == ops.EPI_LERP:
            out.add_((acc - out) * w)
            acc = out
        elif mode in (ops.EPI_ADAM, ops.EPI_LAPROP):
            v.lerp_(acc * acc, 1 - b2)
            d = v.sqrt().clamp_(min=eps)
            if mode == ops.EPI_ADAM:
                m.lerp_(acc, 1 - b1)
                acc = m / d
            else:
                m.lerp_(acc / d, 1 - b1)
                acc = m.clone()
        if out is not None and mode != ops.EPI_LERP:
            out.copy_(acc)
        if split_out == ops.SPLIT_ROWS:
            return _TorchOperand(acc)
        if split_out == ops.SPLIT_COLS:
            return _TorchOperand(acc.transpose(-1, -2))
        return None


class _SplitOperand:
    __slots__ = ("data", "K")

    def __init__(self, data, K):
        self.data, self.K = data, K


class TensorCoreBackend:
    """Split-tf32 tcgen05 GEMM with fused epilogues (``ops.tf32_split`` / ``ops.tf32_gemm``)."""

    name = "tcgen05"

    @staticmethod
    def operands(x: Tensor, same: bool = True, trans: bool = False):
        x = x if x.is_contiguous() else x.contiguous()
        s, t = ops.tf32_split(x, same, trans)
        return (_SplitOperand(s, x.shape[-1]) if same else None), (_SplitOperand(t, x.shape[-2]) if trans else None)

    @staticmethod
    def gemm(a, b, *, mode=ops.EPI_STORE, alpha=1.0, w=0.0, b1=0.0, b2=0.0, eps=0.0, out=None, split_out=ops.SPLIT_NONE,
             m=None, v=None):  # fmt: skip
        s = ops.tf32_gemm(a.data, b.data, a.K, mode=mode, alpha=alpha, w=w, b1=b1, b2c=b2, eps=eps, out=out,
                          split_out=split_out, m=m, v=v)  # fmt: skip
        if split_out == ops.SPLIT_NONE:
            return None
        M, N = a.data.shape[1], b.data.shape[1]
        return _SplitOperand(s, N if split_out == ops.SPLIT_ROWS else M)


def backend_for(t: Tensor, dims: Sequence[int]):
    if t.is_cuda and t.dtype == torch.float32 and min(dims) >= MIN_TC_DIM and ops.available() and utils.tensor_core_matmul:
        return TensorCoreBackend
    return TorchBackend


# ---------------------------------------------------------------------------------------- captured regions

GRAPH_MAX_BYTES = 256 << 20  # buckets larger than this run their fit / refresh eagerly (they are device-bound anyway)
use_graphs = True


class Captured:
    """Runs ``fn()`` - a fixed sequence of kernels over tensors at fixed addresses with fixed scalars - eagerly the
    first time (libraries create their handles and workspaces outside capture), captures it into a CUDA graph the
    second time and replays it afterwards.  A preconditioner fit or an eigenbasis refresh is hundreds of small
    launches; replayed, the host no longer sets their duration.  ``key`` names everything the sequence depends on
    (addresses, shapes, scalars): a different key drops the graph.  If capture fails the region stays eager."""

    def __init__(self):
        self.key = None
        self.calls = 0
        self.graph = None
        self.failed = False

    def __call__(self, fn, key, device):
        if not use_graphs or device.type != "cuda" or self.failed or torch.cuda.is_current_stream_capturing():
            return fn()
        if key != self.key:
            self.key, self.calls, self.graph = key, 0, None
        self.calls += 1
        if self.calls == 1:
            return fn()
        if self.graph is None:
            try:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):  # own memory pool: it lives exactly as long as this graph
                    fn()
                self.graph = graph
            except Exception as err:  # noqa: BLE001 - whatever stops capture, the eager sequence is still correct
                self.failed = True
                import warnings

                warnings.warn(f"CUDA graph capture of a preconditioner update failed ({type(err).__name__}: {err}); running it eagerly")
                return fn()
        self.graph.replay()


# ---------------------------------------------------------------------------------------- state adoption


def _is_view_of(t: Tensor, base: Tensor, j: int) -> bool:
    return (
        isinstance(t, Tensor)
        and t.data_ptr() == base.data_ptr() + j * base.stride(0) * base.element_size()
        and t.shape[1:] == base.shape[1:]
        and t.dtype == base.dtype
    )


def adopt(members: List[dict], key: str, batched: Optional[Tensor], pick=None, put=None) -> Optional[Tensor]:
    """Returns the batched tensor behind ``member[key]`` of all members, concatenating and re-pointing the entries
    to views when they are not (or no longer) views of ``batched``.  ``pick`` / ``put`` reach into nested entries."""
    pick = pick or (lambda st: st[key])
    first = pick(members[0])
    if first is None:
        return None
    if batched is not None and all(_is_view_of(pick(st), batched, j) for j, st in enumerate(members)):
        return batched
    parts = [pick(st) for st in members]
    batched = torch.cat(parts, 0).contiguous() if len(parts) > 1 else parts[0].contiguous()
    for j, st in enumerate(members):
        view = batched[j : j + 1]
        if put is None:
            st[key] = view
        else:
            put(st, view)
    return batched


# ---------------------------------------------------------------------------------------- SOAP


class SoapBucket:
    """One shape bucket of a SOAP-family transform: batched moments, eigenbases and statistics."""

    def __init__(self, keys: Dict[str, str], inner: str):
        self.keys = keys  # slot name -> state key
        self.inner = inner  # "adam" | "laprop"
        self.m = self.v = None
        self.Q: List[Optional[Tensor]] = [None, None]
        self.GG: List[Optional[Tensor]] = [None, None]
        self.q_ops = None  # cached operands of the eigenbases, rebuilt after a refresh / re-adoption
        self.q_ptrs = None

    def _adopt(self, members):
        k = self.keys
        self.m = adopt(members, k["exp_avg"], self.m)
        self.v = adopt(members, k["exp_avg_sq"], self.v)
        for name, store in (("Q", self.Q), ("GG", self.GG)):
            n_modes = len(members[0][k[name]])
            for i in range(2):
                if i >= n_modes:
                    store[i] = None
                    continue

                def put(st, view, i=i, name=name):
                    lst = list(st[k[name]])
                    lst[i] = view
                    st[k[name]] = lst

                store[i] = adopt(members, k[name], store[i], pick=lambda st, i=i, name=name: st[k[name]][i], put=put)
        ptrs = tuple(None if q is None else q.data_ptr() for q in self.Q)
        if ptrs != self.q_ptrs:
            self.q_ptrs, self.q_ops = ptrs, None

    def run(self, members: List[dict], U: Tensor, out: Tensor, group, *, b1, b2, eps, stat_w, refresh: bool):
        """``U``: ``(B, R, C)`` fp32 updates of the bucket (read only); ``out``: same shape, receives the
        preconditioned update.  ``b1`` / ``b2``: debiased moment coefficients; ``stat_w``: weight of this step's outer
        products in the statistics; ``refresh``: advance the eigenbases after the statistics."""
        self._adopt(members)
        Ql, Qr = self.Q
        B, R, C = U.shape
        dims = [d for d, q in ((R, Ql), (C, Qr)) if q is not None] + [R, C]
        be = backend_for(U, dims)
        if self.q_ops is None or self.q_ops[0] is not be:
            l_same, l_trans = be.operands(Ql, True, True) if Ql is not None else (None, None)
            r_same, r_trans = be.operands(Qr, True, True) if Qr is not None else (None, None)
            self.q_ops = (be, l_same, l_trans, r_same, r_trans)
        _, l_same, l_trans, r_same, r_trans = self.q_ops
        mode = ops.EPI_ADAM if self.inner == "adam" else ops.EPI_LAPROP
        adam = dict(mode=mode, b1=b1, b2=b2, eps=eps, m=self.m, v=self.v)
        has_l, has_r = Ql is not None, Qr is not None
        need_same = has_l or (has_r and not has_l)
        need_trans = has_l or has_r
        u_same, u_trans = be.operands(U, need_same, need_trans)

        if has_l and has_r:
            p1 = be.gemm(l_trans, u_trans, split_out=ops.SPLIT_ROWS)                      # Ql^T U
            n = be.gemm(p1, r_trans, split_out=ops.SPLIT_ROWS, **adam)                    # (.) Qr, Adam in the eigenbasis
            o1 = be.gemm(n, r_same, split_out=ops.SPLIT_COLS)                             # N Qr^T
            be.gemm(l_same, o1, out=out)                                                  # Ql (.)
        elif has_l:
            n = be.gemm(l_trans, u_trans, split_out=ops.SPLIT_COLS, **adam)
            be.gemm(l_same, n, out=out)
        elif has_r:
            n = be.gemm(u_same, r_trans, split_out=ops.SPLIT_ROWS, **adam)
            be.gemm(n, r_same, out=out)
        else:
            raise RuntimeError("bucket without eigenbases must take the element-wise path")

        # statistics: GG_l <- lerp(GG_l, U U^T), GG_r <- lerp(GG_r, U^T U)
        if self.GG[0] is not None:
            be.gemm(u_same, u_same, mode=ops.EPI_LERP, w=stat_w, out=self.GG[0])
        if len(self.GG) > 1 and self.GG[1] is not None:
            be.gemm(u_trans, u_trans, mode=ops.EPI_LERP, w=stat_w, out=self.GG[1])
        if refresh:  # in place on the adopted state; its orthogonalisation replays its own graphs
            utils.get_orthogonal_matrix_QR(self.GG, self.Q, self.m)
            self.q_ops = None


# ---------------------------------------------------------------------------------------- PSGD (Kron)


class PsgdBucket:
    """One shape bucket of ``scale_by_psgd`` / ``update_by_psgd``: batched factors (packed or dense, as the checkpoint
    stores them), lower bounds, and a dense working copy ``P_i = Q_i^T Q_i`` of every factor that is rebuilt only when
    the preconditioner is fitted, so the per-step application is two products (one per side) instead of four plus a
    scatter of the packed triangle."""

    def __init__(self, keys: Dict[str, str], store_triu_as_line: bool):
        self.keys = keys
        self.line = store_triu_as_line
        self.Q: List[Optional[Tensor]] = []
        self.lb: List[Optional[Tensor]] = []
        self.shapes = None
        self.p_ops = None  # (backend, [operand or diagonal scale per mode])
        self.q_ptrs = None
        self.fit_region = Captured()

    def _adopt(self, members):
        kq, kl = self.keys["Q"], self.keys["running_lower_bound"]
        n_modes = len(members[0][kq])
        if len(self.Q) != n_modes:
            self.Q, self.lb = [None] * n_modes, [None] * n_modes
        shapes = []
        for i in range(n_modes):
            if self.line:

                def put(st, view, i=i):
                    lst = list(st[kq])
                    lst[i] = (lst[i][0], view)
                    st[kq] = lst

                shapes.append(members[0][kq][i][0])
                self.Q[i] = adopt(members, kq, self.Q[i], pick=lambda st, i=i: st[kq][i][1], put=put)
            else:

                def put(st, view, i=i):
                    lst = list(st[kq])
                    lst[i] = view
                    st[kq] = lst

                shapes.append(None)
                self.Q[i] = adopt(members, kq, self.Q[i], pick=lambda st, i=i: st[kq][i], put=put)

            def put_lb(st, view, i=i):
                lst = list(st[kl])
                lst[i] = view
                st[kl] = lst

            self.lb[i] = adopt(members, kl, self.lb[i], pick=lambda st, i=i: st[kl][i], put=put_lb)
        self.shapes = shapes
        ptrs = tuple(q.data_ptr() for q in self.Q)
        if ptrs != self.q_ptrs:
            self.q_ptrs, self.p_ops = ptrs, None

    def _batched_q(self):
        """Factors in the form ``utils.psgd_update_precond`` takes: packed ``(shape, line)`` tuples or dense tensors."""
        if not self.line:
            return list(self.Q)
        out = []
        for shape, q in zip(self.shapes, self.Q):
            out.append((None if shape is None else (q.shape[0], *shape[1:]), q))
        return out

    def _dense(self):
        return utils.line_to_triu(self._batched_q()) if self.line else list(self.Q)

    def fit(self, U: Tensor, group, param_like):
        """Preconditioner fitting step on the batched factors (in place on the adopted state)."""
        scalars = (group["dampening"], group["precond_lr"], utils.get_beta2(group), group["lower_bound_beta"],
                   group["precond_update_power_iterations"])  # fmt: skip

        def run():
            vector, hessian_vector = utils.dampen_grad(U, scalars[0])
            utils.psgd_update_precond(
                hessian_vector, scalars[1], self._batched_q(), self.line, scalars[2], vector, self.lb, scalars[3], scalars[4]
            )

        if U.numel() * 4 <= GRAPH_MAX_BYTES:
            key = (self.q_ptrs, tuple(t.data_ptr() for t in self.lb), U.data_ptr(), tuple(U.shape), scalars)
            self.fit_region(run, key, U.device)
        else:
            run()
        self.p_ops = None

    def run(self, members: List[dict], U: Tensor, out: Tensor, group, *, fit: bool, delayed: bool):
        self._adopt(members)
        if fit and not delayed:
            self.fit(U, group, None)
        B = U.shape[0]
        dims = list(U.shape[1:])
        be = backend_for(U, dims)
        if self.p_ops is None or self.p_ops[0] is not be:
            per_mode = []
            for q in self._dense():
                q32 = utils.promote(q)
                if q32.ndim == 3:
                    pq = _mm(q32, q32, True, False)  # Q^T Q, symmetric
                    per_mode.append(("dense", be.operands(pq.contiguous(), True, False)[0]))
                else:
                    per_mode.append(("diag", (q32 * q32).reshape(B, -1)))
            self.p_ops = (be, per_mode)
        _, per_mode = self.p_ops
        if U.ndim != 3:  # vectors, scalars, higher-order tensors: the general mode-by-mode application
            out.copy_(utils.psgd_precond_grad(U, self._batched_q(), store_triu_as_line=self.line))
            if fit and delayed:
                self.fit(U, group, None)
            return
        (kind_l, P_l), (kind_r, P_r) = per_mode
        x = U
        if kind_l == "diag":
            x = x * P_l.unsqueeze(-1)
        if kind_r == "diag":
            x = x * P_r.unsqueeze(-2)
        if kind_l == "dense" and kind_r == "dense":
            _, x_t = be.operands(x, False, True)
            t = be.gemm(P_l, x_t, split_out=ops.SPLIT_ROWS)   # P_l X  (P symmetric: its rows are its columns)
            be.gemm(t, P_r, out=out)                          # (.) P_r
        elif kind_l == "dense":
            _, x_t = be.operands(x, False, True)
            be.gemm(P_l, x_t, out=out)
        elif kind_r == "dense":
            x_s, _ = be.operands(x, True, False)
            be.gemm(x_s, P_r, out=out)
        else:
            out.copy_(x)
        if fit and delayed:
            self.fit(U, group, None)
