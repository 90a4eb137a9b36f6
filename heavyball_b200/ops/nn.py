"""Model-side ops used by ``heavyball_b200.models`` for bf16-autocast training on sm_100a.  Each has the
framework op it replaces as its fallback (CPU, other dtypes, unsupported shapes).

``linear_cross_entropy``
    The output head's projection + softmax cross-entropy.  ``logits = h @ W^T`` is computed once in bf16
    (library GEMM); one kernel (``csrc/cross_entropy.cu``) sweeps each row three times (the last two from L2),
    returns the per-row loss and overwrites the logits with ``(softmax - onehot) / n_valid``; backward is two
    GEMMs on that buffer.  Against ``F.cross_entropy(logits.float(), targets)`` this removes the fp32 copy of
    the logits, ``log_softmax``, its backward and the cast back: about 26 GB of HBM traffic per step for
    16 x 1024 tokens and a 50k vocabulary, against 3.3 GB.  ``W`` may have more rows than the vocabulary (a
    row count that is a multiple of 64 keeps the GEMMs on their aligned tensor-core kernels: a 50 257-row head
    runs on a legacy unaligned path about 9x slower); the extra columns get zero probability and zero gradient.
``layer_norm`` / ``add_layer_norm`` / ``LayerNorm``
    One kernel each way (``csrc/layer_norm.cu``); under autocast the output is written, and the incoming
    gradient read, in bf16 directly.  ``add_layer_norm`` also performs the residual add that precedes the
    normalisation (and, on the way back, the add of the gradient arriving on the residual stream).
``linear`` / ``Linear`` / ``CastCache``
    ``F.linear`` whose bias gradient comes from a column-sum kernel (``csrc/colsum.cu``), whose weight gradient
    leaves its GEMM in fp32, and whose bf16 weights come from one multi-tensor cast per forward pass.
``split_linear``
    The packed q / k / v projection as one autograd node: three dense outputs, input gradient accumulated inside
    the GEMMs, one packed weight / bias gradient.
``linear_gelu``
    Linear layer followed by tanh-GELU (``csrc/gelu.cu``): the activation's backward kernel also sums the bias
    gradient.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from . import available, launch_counter, load


def _mm_f32(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    try:
        return torch.mm(a, b, out_dtype=torch.float32)
    except (TypeError, RuntimeError):
        return torch.mm(a, b).float()


class _LinearCrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, weight, targets, vocab, ignore_index):
        h16 = h.detach().reshape(-1, h.shape[-1]).to(torch.bfloat16)
        w16 = weight.detach().to(torch.bfloat16)
        flat_targets = targets.reshape(-1).contiguous()
        n_valid = (flat_targets != ignore_index).sum().clamp_(min=1)
        scale = n_valid.to(torch.float32).reciprocal_().reshape(1)
        logits = h16 @ w16.mT
        losses = load().cross_entropy_(logits, flat_targets, scale, vocab, ignore_index)
        launch_counter.count += 1
        ctx.save_for_backward(logits, h16, w16)
        ctx.h_meta, ctx.w_dtype = (h.shape, h.dtype), weight.dtype
        return losses.sum() * scale[0]

    @staticmethod
    def backward(ctx, grad_out):
        dlogits, h16, w16 = ctx.saved_tensors
        (h_shape, h_dtype), w_dtype = ctx.h_meta, ctx.w_dtype
        dh = dw = None
        if ctx.needs_input_grad[0]:
            dh = (dlogits @ w16).mul_(grad_out).reshape(h_shape).to(h_dtype)
        if ctx.needs_input_grad[1]:
            dw = _mm_f32(dlogits.mT, h16).mul_(grad_out).to(w_dtype)
        return dh, dw, None, None, None


def linear_cross_entropy(h: torch.Tensor, weight: torch.Tensor, targets: torch.Tensor, vocab: int | None = None,
                         ignore_index: int = -100) -> torch.Tensor:  # fmt: skip
    """Mean cross-entropy of ``softmax((h @ weight^T)[..., :vocab])`` against ``targets``.

    ``h``: ``[..., d]``; ``weight``: ``[rows >= vocab, d]``; ``targets``: integer tensor with ``h``'s leading
    shape.  On sm_100a the fused kernel path runs (``weight.shape[0]`` must be a multiple of 8); elsewhere the
    same quantity is computed with PyTorch ops."""
    vocab = weight.shape[0] if vocab is None else vocab
    if h.is_cuda and available() and weight.shape[0] % 8 == 0:
        return _LinearCrossEntropy.apply(h, weight, targets, vocab, ignore_index)
    logits = F.linear(h, weight)[..., :vocab]
    return F.cross_entropy(logits.float().reshape(-1, vocab), targets.reshape(-1), ignore_index=ignore_index)


class _LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps, out_bf16):
        y, mean, rstd = load().layer_norm_fwd(x, None, weight, bias, eps, out_bf16)
        launch_counter.count += 1
        ctx.save_for_backward(x, weight, mean, rstd)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, weight, mean, rstd = ctx.saved_tensors
        dx, dw, db = load().layer_norm_bwd(dy.contiguous(), x, weight, mean, rstd, None, False)
        launch_counter.count += 2
        return dx, dw, db, None, None


class _AddLayerNormFn(torch.autograd.Function):
    """``s = x + res``, ``y = LayerNorm(s)`` in one kernel; backward adds the gradient arriving at ``s`` to the
    LayerNorm gradient in the same kernel that computes it."""

    @staticmethod
    def forward(ctx, x, res, weight, bias, eps, out_bf16):
        y, mean, rstd, s = load().layer_norm_fwd(x, res, weight, bias, eps, out_bf16)
        launch_counter.count += 1
        ctx.save_for_backward(s, weight, mean, rstd)
        ctx.res_dtype = res.dtype
        return s, y

    @staticmethod
    def backward(ctx, ds, dy):
        s, weight, mean, rstd = ctx.saved_tensors
        if dy is None:  # the normalised output was not used
            return ds, None if ds is None else ds.to(ctx.res_dtype), None, None, None, None
        ds = None if ds is None else ds.contiguous()
        # a bf16 residual branch gets its gradient from the same kernel (no cast pass over dx)
        out = load().layer_norm_bwd(dy.contiguous(), s, weight, mean, rstd, ds, ctx.res_dtype == torch.bfloat16)
        launch_counter.count += 2
        dx, dw, db = out[:3]
        return dx, out[3] if len(out) == 4 else dx.to(ctx.res_dtype), dw, db, None, None


def _ln_kernel_applies(x: torch.Tensor, weight, bias) -> bool:
    d = x.shape[-1]
    return (
        x.is_cuda and x.dtype == torch.float32 and weight is not None and bias is not None
        and weight.dtype == torch.float32 and d % 128 == 0 and d <= 1024 and x.numel() > 0 and available()
    )  # fmt: skip


def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    """LayerNorm over the last dimension.  For fp32 CUDA activations with a row length that is a multiple
    of 128 (up to 1024) one kernel each way runs; inside a bf16 autocast region the output is written in
    bf16 directly (the dtype the following linear layer would cast it to) and the backward kernel takes the
    bf16 gradient.  Other inputs go to ``F.layer_norm``."""
    if _ln_kernel_applies(x, weight, bias):
        out_bf16 = torch.is_autocast_enabled("cuda") and torch.get_autocast_dtype("cuda") == torch.bfloat16
        return _LayerNormFn.apply(x.contiguous(), weight, bias, eps, out_bf16)
    return F.layer_norm(x, (x.shape[-1],), weight, bias, eps)


def add_layer_norm(x: torch.Tensor, res, weight: torch.Tensor, bias: torch.Tensor, eps: float = 1e-5):
    """``(x + res, LayerNorm(x + res))``: the residual add of a pre-norm transformer block fused into the
    normalisation that follows it (one pass over the stream instead of two each way).  ``res=None`` gives
    ``(x, LayerNorm(x))``."""
    if res is None:
        return x, layer_norm(x, weight, bias, eps)
    if _ln_kernel_applies(x, weight, bias) and res.shape == x.shape and res.dtype in (torch.float32, torch.bfloat16):
        out_bf16 = torch.is_autocast_enabled("cuda") and torch.get_autocast_dtype("cuda") == torch.bfloat16
        return _AddLayerNormFn.apply(x.contiguous(), res.contiguous(), weight, bias, eps, out_bf16)
    s = x + res
    return s, layer_norm(s, weight, bias, eps)


class LayerNorm(torch.nn.LayerNorm):
    """``torch.nn.LayerNorm`` (same parameters and state dict) running :func:`layer_norm`; ``forward(x, res)``
    returns ``(x + res, LayerNorm(x + res))`` through :func:`add_layer_norm`."""

    def forward(self, x, res=None):
        if len(self.normalized_shape) != 1:
            return super().forward(x if res is None else x + res)
        if res is None:
            return layer_norm(x, self.weight, self.bias, self.eps)
        return add_layer_norm(x, res, self.weight, self.bias, self.eps)


def _weight_grad(dy2: torch.Tensor, x2: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """``dy2^T @ x2`` for bf16 operands, written in fp32 (the parameter's dtype) by the GEMM itself instead of in
    bf16 followed by a cast kernel; ``out`` may be a row slice of a packed gradient."""
    if dy2.is_cuda:
        if out is None:
            return torch.mm(dy2.mT, x2, out_dtype=torch.float32)
        return torch.mm(dy2.mT, x2, out_dtype=torch.float32, out=out)
    dw = (dy2.mT @ x2).float()  # the fp32-output GEMM exists on CUDA only
    return dw if out is None else out.copy_(dw)


def _bias_grad(dy2: torch.Tensor) -> torch.Tensor:
    if dy2.is_cuda and dy2.shape[1] % 8 == 0 and dy2.data_ptr() % 16 == 0:
        launch_counter.count += 2
        return load().colsum_bf16(dy2)
    return dy2.float().sum(0)


def _as_bf16_rows(dy: torch.Tensor) -> torch.Tensor:
    dy2 = dy.reshape(-1, dy.shape[-1])
    if dy2.dtype != torch.bfloat16:
        dy2 = dy2.to(torch.bfloat16)
    return dy2 if dy2.is_contiguous() else dy2.contiguous()


class _LinearFn(torch.autograd.Function):
    """``x @ w^T + b`` computed from bf16 copies ``w16`` / ``b16`` of the fp32 parameters; gradients are routed
    to the fp32 parameters (the weight gradient leaves its GEMM in fp32), the bias gradient comes from the
    column-sum kernel."""

    @staticmethod
    def forward(ctx, x, weight, bias, w16, b16):
        x16 = x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)
        ctx.save_for_backward(x16, w16)
        ctx.x_dtype = x.dtype
        return F.linear(x16, w16, b16)

    @staticmethod
    def backward(ctx, dy):
        x16, w16 = ctx.saved_tensors
        dy2 = _as_bf16_rows(dy)
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = (dy2 @ w16).reshape(x16.shape).to(ctx.x_dtype)
        if ctx.needs_input_grad[1]:
            dw = _weight_grad(dy2, x16.reshape(-1, x16.shape[-1]))
        if ctx.needs_input_grad[2]:
            db = _bias_grad(dy2)
        return dx, dw, db, None, None


class _SplitLinearFn(torch.autograd.Function):
    """``n`` projections of the same input by equal row blocks of one packed weight, each into its own dense
    output (packed q / k / v).  Backward accumulates the input gradient inside the GEMMs (``beta = 1``) and writes
    each block of the weight and bias gradients into its rows of one packed gradient; taking the row blocks as
    views instead costs, per block, a zero-filled full-size gradient plus an add, and an add per extra input
    gradient."""

    @staticmethod
    def forward(ctx, x, weight, bias, w16, b16, n):
        x16 = x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)
        ctx.save_for_backward(x16, w16)
        ctx.x_dtype, ctx.n = x.dtype, n
        rows = w16.shape[0] // n
        return tuple(F.linear(x16, w16[i * rows : (i + 1) * rows], b16[i * rows : (i + 1) * rows]) for i in range(n))

    @staticmethod
    def backward(ctx, *dys):
        x16, w16 = ctx.saved_tensors
        n, rows = ctx.n, w16.shape[0] // ctx.n
        x2 = x16.reshape(-1, x16.shape[-1])
        parts = [None if dy is None else _as_bf16_rows(dy) for dy in dys]
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            for i, dy2 in enumerate(parts):
                if dy2 is None:
                    continue
                blk = w16[i * rows : (i + 1) * rows]
                dx = dy2 @ blk if dx is None else dx.addmm_(dy2, blk)
            if dx is not None:
                dx = dx.reshape(x16.shape).to(ctx.x_dtype)
        if ctx.needs_input_grad[1]:
            dw = torch.empty(w16.shape, dtype=torch.float32, device=w16.device)
            for i, dy2 in enumerate(parts):
                if dy2 is None:
                    dw[i * rows : (i + 1) * rows].zero_()
                else:
                    _weight_grad(dy2, x2, out=dw[i * rows : (i + 1) * rows])
        if ctx.needs_input_grad[2]:
            live = [dy2 for dy2 in parts if dy2 is not None]
            if (len(live) == n and n <= 4 and live[0].is_cuda and live[0].shape[1] % 8 == 0
                    and all(dy2.data_ptr() % 16 == 0 for dy2 in live)):  # fmt: skip
                db = load().colsum_bf16_batch(live)  # one launch pair, already concatenated
                launch_counter.count += 2
            else:
                zero = torch.zeros(rows, dtype=torch.float32, device=w16.device)
                db = torch.cat([zero if dy2 is None else _bias_grad(dy2) for dy2 in parts])
        return dx, dw, db, None, None, None


class _LinearGeluFn(torch.autograd.Function):
    """``gelu_tanh(x @ w^T + b)`` for the first half of a transformer MLP.  Forward: the library GEMM (bias in its
    epilogue) and one activation kernel; backward: one kernel gives the gradient at the GEMM output and, from the
    same pass, the bias gradient, then the two gradient GEMMs."""

    @staticmethod
    def forward(ctx, x, weight, bias, w16, b16):
        x16 = x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)
        u = F.linear(x16, w16, b16)
        y = load().gelu_fwd(u)
        launch_counter.count += 1
        ctx.save_for_backward(x16, w16, u)
        ctx.x_dtype = x.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        x16, w16, u = ctx.saved_tensors
        du, db = load().gelu_bwd(_as_bf16_rows(dy), u.reshape(-1, u.shape[-1]))
        launch_counter.count += 2
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = (du @ w16).reshape(x16.shape).to(ctx.x_dtype)
        if ctx.needs_input_grad[1]:
            dw = _weight_grad(du, x16.reshape(-1, x16.shape[-1]))
        return dx, dw, db if ctx.needs_input_grad[2] else None, None, None


def _bf16_training(x: torch.Tensor) -> bool:
    return x.is_cuda and torch.is_autocast_enabled("cuda") and torch.get_autocast_dtype("cuda") == torch.bfloat16 and available()


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None, w16: torch.Tensor | None = None,
           b16: torch.Tensor | None = None) -> torch.Tensor:  # fmt: skip
    """``F.linear`` for training under bf16 autocast on sm_100a: identical forward, but the bias gradient comes from
    a dedicated column-sum kernel (the framework's generic reduction runs at a third of memory bandwidth on the
    ``[tokens, features]`` gradients of a transformer).  ``w16`` / ``b16`` are bf16 copies of the parameters when
    the caller keeps some (:class:`CastCache`); otherwise they are made here.  Elsewhere, and without a bias, it is
    ``F.linear``."""
    if bias is not None and _bf16_training(x):
        if w16 is None:
            w16, b16 = weight.detach().to(torch.bfloat16), bias.detach().to(torch.bfloat16)
        return _LinearFn.apply(x, weight, bias, w16, b16)
    return F.linear(x, weight, bias)


def linear_gelu(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, w16: torch.Tensor | None = None,
                b16: torch.Tensor | None = None) -> torch.Tensor:  # fmt: skip
    """``F.gelu(F.linear(x, weight, bias), approximate="tanh")``.  Under bf16 autocast on sm_100a, with an output
    width that is a multiple of 8, the activation and its backward run in this package's kernels and the backward
    kernel also produces the bias gradient (see :class:`_LinearGeluFn`); elsewhere it is the two framework calls."""
    if bias is not None and weight.shape[0] % 8 == 0 and _bf16_training(x):
        if w16 is None:
            w16, b16 = weight.detach().to(torch.bfloat16), bias.detach().to(torch.bfloat16)
        return _LinearGeluFn.apply(x, weight, bias, w16, b16)
    return F.gelu(linear(x, weight, bias, w16, b16), approximate="tanh")


def split_linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, n: int, w16: torch.Tensor | None = None,
                 b16: torch.Tensor | None = None) -> tuple:  # fmt: skip
    """``n`` outputs ``x @ weight[i]^T + bias[i]`` for the ``n`` equal row blocks of a packed projection (q, k, v),
    each dense.  Under bf16 autocast on sm_100a one autograd node covers all of them (see :class:`_SplitLinearFn`);
    elsewhere it is ``n`` calls of ``F.linear`` on row slices."""
    if n < 1 or weight.shape[0] % n:
        raise ValueError(f"split_linear: {weight.shape[0]} weight rows do not split into {n} equal blocks")
    rows = weight.shape[0] // n
    if _bf16_training(x):
        if w16 is None:
            w16, b16 = weight.detach().to(torch.bfloat16), bias.detach().to(torch.bfloat16)
        return _SplitLinearFn.apply(x, weight, bias, w16, b16, n)
    return tuple(F.linear(x, weight[i * rows : (i + 1) * rows], bias[i * rows : (i + 1) * rows]) for i in range(n))


class Linear(torch.nn.Linear):
    """``torch.nn.Linear`` (same parameters and state dict) running :func:`linear`."""

    w16 = b16 = None  # bf16 copies handed out by a CastCache, valid for the current forward pass

    def forward(self, x):
        return linear(x, self.weight, self.bias, self.w16, self.b16)


class CastCache:
    """bf16 copies of the parameters of a model's :class:`Linear` layers in one slab, made with one
    multi-tensor copy per forward pass instead of one small cast kernel per parameter per use (about 300 launches
    of ~3 us for a 12-layer transformer).  The copies are plain attributes of the layers (``w16`` / ``b16``): not
    parameters, not buffers, absent from ``state_dict``."""

    def __init__(self, model: torch.nn.Module):
        self.layers = [m for m in model.modules() if isinstance(m, Linear) and m.bias is not None]

    def refresh(self, active: bool) -> None:
        if not active or not self.layers:
            for m in self.layers:
                m.w16 = m.b16 = None
            return
        params = [p for m in self.layers for p in (m.weight, m.bias)]
        total = sum((p.numel() + 7) // 8 * 8 for p in params)
        # a fresh slab every time: the previous one may be held by an autograd graph that has not run backward yet
        # (the caching allocator hands the same memory back once that graph is gone)
        slab = torch.empty(total, dtype=torch.bfloat16, device=params[0].device)
        views, off = [], 0
        for p in params:
            views.append(slab[off : off + p.numel()].view(p.shape))
            off += (p.numel() + 7) // 8 * 8  # 16-byte aligned starts
        with torch.no_grad():
            torch._foreach_copy_(views, params)
        for i, m in enumerate(self.layers):
            m.w16, m.b16 = views[2 * i], views[2 * i + 1]
