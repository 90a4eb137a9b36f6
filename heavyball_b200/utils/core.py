"""Numerical substrate: promotion, stochastic rounding, the ULP error-correction codec and the
in-place list arithmetic every transform is built from.

Behavioural parity targets (reference paths): promotion and guards ``heavyball/utils.py:1327-1359,
1077-1116``; stochastic rounding ``heavyball/utils.py:2341-2370``; the ECC codec
``heavyball/utils.py:1288-1324, 3376-3392``; list arithmetic ``heavyball/utils.py:1041-1202``;
parameter-update epilogue ``heavyball/utils.py:2373-2406, 3652-3662``.

Everything here is plain PyTorch and runs on any device.  On a B200 the fused multi-tensor kernels in
``heavyball_b200.ops`` execute whole transform chains in one pass; these functions are the reference
semantics those kernels are tested against, and the fallback for chains that are not lowered.
"""

from __future__ import annotations

import enum
import sys
import warnings
from typing import Iterable, List, Optional, Sequence, Union

import torch
from torch import Tensor
from torch.utils._pytree import tree_map

Number = Union[int, float, Tensor]


def _settings():
    """The ``heavyball_b200.utils`` package namespace holds user-mutable switches (``dither_steps``,
    ``default_division_backend`` ...).  They are looked up at call time so that assignments such as
    ``heavyball_b200.utils.dither_steps = 2`` take effect immediately."""
    return sys.modules[__package__]


# --------------------------------------------------------------------------------------------------
# small helpers
# --------------------------------------------------------------------------------------------------

_warned: set = set()


def warn_once(msg: str):
    if msg not in _warned:
        _warned.add(msg)
        warnings.warn(msg)


def hasattr_none(obj, name) -> bool:
    return getattr(obj, name, None) is not None


def list_guard(*xs):
    out = [x if isinstance(x, (list, tuple)) else [x] for x in xs]
    return out[0] if len(xs) == 1 else out


def scalar_guard(*args):
    """Scalars stay host numbers here: kernels receive them as launch arguments, so nothing is
    staged through 0-d device tensors.  Floating 0-d tensors are widened to the promoted dtype of
    ``ref`` so mixed-precision arithmetic keeps fp32 scalars."""
    *xs, ref = args
    wide = promote(ref.dtype) if isinstance(ref, Tensor) else torch.float32
    out = []
    for x in xs:
        if isinstance(x, Tensor) and x.ndim == 0 and x.is_floating_point():
            x = x.to(wide)
        out.append(x)
    return out[0] if len(xs) == 1 else out


def broadcastable_list_guard(*xs):
    xs = [x if isinstance(x, (list, tuple)) else [x] for x in xs]
    if not any(isinstance(x[0], Tensor) for x in xs):
        raise ValueError("No tensor-valued input given")
    longest = max(len(x) for x in xs)
    return [list(x) if len(x) > 1 else list(x) * longest for x in xs]


def as_float(x: Number) -> float:
    return float(x.item()) if isinstance(x, Tensor) else float(x)


def as_int(x: Number) -> int:
    return int(x.item()) if isinstance(x, Tensor) else int(x)


def beta_debias(beta, step):
    """EMA coefficient whose running average is exactly unbiased after ``step`` samples:
    ``1 - (1 - beta) / (1 - beta ** step)``."""
    if isinstance(step, Tensor) or isinstance(beta, Tensor):
        return 1 - (1 - beta) / (1 - beta**step)
    denom = 1 - beta**step
    if denom == 0:
        return 0.0
    return 1 - (1 - beta) / denom


def get_beta1(group):
    beta = group.get("beta")
    if beta is None and "betas" in group:
        beta = group["betas"][0]
    if beta is None:
        raise ValueError("Beta not found in group.")
    return beta


def get_beta2(group):
    if group.get("palm") is True and "beta2_scale" in group:
        step = group.get("step", 1)
        step = max(as_int(step) if step is not None else 1, 1)
        return 1 - step ** -group["beta2_scale"]
    if "betas" in group:
        return group["betas"][1]
    raise ValueError("Beta2 not found in group.")


def min_dtype(xs: Sequence[Tensor]):
    have = {x.dtype for x in xs}
    for cand in (torch.float32, torch.bfloat16, torch.float16):
        if have <= {cand, torch.float32, torch.float64}:
            return cand
    return torch.float32


def detach(x):
    return x.detach() if isinstance(x, Tensor) else x


def promote_detach(x, should_promote):
    if x is None:
        return None
    return (promote(x) if should_promote else x).detach()


def set_(dst: Tensor, src: Tensor):
    dst.copy_(src)


def zero_(xs):
    for x in list_guard(xs):
        x.zero_()


# --------------------------------------------------------------------------------------------------
# ULP error-correction codec
# --------------------------------------------------------------------------------------------------

_MANTISSA = {torch.float16: 10, torch.bfloat16: 7}
_BIAS = {torch.float16: 15, torch.bfloat16: 127}
_NUM_MANTISSA_BITS = _MANTISSA
_EXPONENT_BIAS = _BIAS


def _log_ulp(x: Tensor) -> Tensor:
    """log2 of the unit-in-last-place of every element of a 16-bit float tensor."""
    m, bias = _MANTISSA[x.dtype], _BIAS[x.dtype]
    biased = (x.view(torch.int16).to(torch.int32) & 0x7FFF) >> m
    return torch.where(biased == 0, 1 - bias - m, biased - (bias + m))


def _scale_by_exp2(x: Tensor, log_scale: Tensor) -> Tensor:
    half = torch.floor(log_scale / 2)
    return (x * torch.exp2(half)) * torch.exp2(log_scale - half)


class _ULPState:
    """A 16-bit float tensor carries a signed integer side-car that stores the rounding residual in
    units of ``ulp / (2 * smax)``.  Decoding adds the residual back; encoding rounds the primary to
    nearest and stochastically floors the residual so the pair is an unbiased ~fp24/fp32 value."""

    __slots__ = ("correction", "smax")
    _SMAX = {torch.int8: 127.0, torch.int16: 32767.0}

    def __init__(self, correction: Tensor, smax: float):
        self.correction = correction
        self.smax = smax

    def decode(self, x: Tensor) -> Tensor:
        half_ulp_log = (_log_ulp(x) - 1).float()
        return x.float() + _scale_by_exp2(self.correction.float() / self.smax, half_ulp_log)

    @staticmethod
    def _bf16_to_f32(x: Tensor) -> Tensor:
        return (x.view(torch.int16).to(torch.int32) << 16).view(torch.float32)

    def compute_correction(self, fp32: Tensor, narrow: Tensor):
        wide = self._bf16_to_f32(narrow) if narrow.dtype == torch.bfloat16 else narrow.float()
        half_ulp_log = (_log_ulp(narrow) - 1).float()
        resid = _scale_by_exp2(fp32 - wide, -half_ulp_log).clamp_(-1.0, 1.0) * self.smax
        resid = torch.floor(resid + torch.rand_like(resid))
        self.correction.copy_(resid.to(self.correction.dtype))

    def encode(self, fp32: Tensor, target: Tensor):
        target.copy_(fp32.to(target.dtype))
        self.compute_correction(fp32, target)


def _promote_one(x):
    if isinstance(x, torch.dtype):
        return torch.float32 if x in (torch.bfloat16, torch.float16, torch.int8) else x
    if isinstance(x, Tensor):
        ecc = getattr(x, "_ecc", None)
        if ecc is not None:
            return ecc.decode(x)
        if x.dtype in (torch.bfloat16, torch.float16):
            return x.float()
    return x


def promote(x):
    """fp32 view of the logical value: decodes ECC pairs, widens 16-bit floats, maps dtypes."""
    if isinstance(x, (Tensor, torch.dtype)):
        return _promote_one(x)
    return tree_map(_promote_one, x)


# --------------------------------------------------------------------------------------------------
# stochastic rounding
# --------------------------------------------------------------------------------------------------


def stochastic_round_(ref: Tensor, source: Optional[Tensor] = None) -> Tensor:
    """Round fp32 to bf16 by adding uniform noise below the kept mantissa and truncating, which is
    unbiased.  ``dither_steps`` independent draws are summed (triangular / higher-order dither)."""
    if source is None:
        source, dtype = ref, torch.bfloat16
    else:
        dtype = ref.dtype
    if dtype != torch.bfloat16 or source.dtype not in (torch.float16, torch.float32, torch.float64):
        return source.to(dtype)
    n = int(getattr(_settings(), "dither_steps", 1))
    bits = source.to(torch.float32).view(torch.int32)
    noise = torch.randint_like(bits, 0, 1 << 16)
    for _ in range(n - 1):
        noise = noise + torch.randint_like(bits, 0, 1 << 16)
    bits = (bits + noise - (n - 1) * (1 << 15)) & -65536
    return bits.view(torch.float32).bfloat16()


def stochastic_round_list_(ref: List[Tensor], source: List[Tensor]):
    return [stochastic_round_(r, s) for r, s in zip(ref, source)]


def copy_stochastic_(target: Tensor, source: Tensor):
    ecc = getattr(target, "_ecc", None)
    if ecc is not None:
        ecc.encode(source if source.dtype == torch.float32 else source.float(), target)
        return
    if target.dtype == torch.bfloat16 and source.dtype in (torch.float16, torch.float32, torch.float64):
        source = stochastic_round_(target, source)
    target.copy_(source)


def copy_stochastic_list_(target: Iterable[Tensor], source: Iterable[Tensor]):
    for t, s in zip(target, source):
        copy_stochastic_(t, s)


# --------------------------------------------------------------------------------------------------
# in-place list arithmetic (fp32 math, stochastic store)
# --------------------------------------------------------------------------------------------------


def stochastic_lerp_(x, y, a: Number):
    x, y = list_guard(x, y)
    for x_, y_ in zip(x, y):
        x32, y32 = promote(x_), promote(y_)
        if y32.dtype != x32.dtype:
            y32 = y32.to(x32.dtype)
        copy_stochastic_(x_, x32 * (1 - a) + y32 * a)


def _lerp(state: List[Tensor], grad: List[Tensor], beta: Number) -> List[Tensor]:
    """``state <- beta * state + (1 - beta) * grad``; returns the fp32 result (before storage
    rounding) so callers keep full precision for the rest of the step."""
    out = []
    w = 1 - beta
    for s_, g_ in zip(state, grad):
        s32, g32 = promote(s_), promote(g_)
        if g32.dtype != s32.dtype:
            g32 = g32.to(s32.dtype)
        new = s32 * (1 - w) + g32 * w
        copy_stochastic_(s_, new)
        out.append(new)
    return out


def stochastic_add_(x, y, alpha: Number = 1):
    x, y = broadcastable_list_guard(x, y)
    for x_, y_ in zip(x, y):
        copy_stochastic_(x_, promote(x_) + promote(y_) * alpha)


def stochastic_add_divide_(x, y, alpha: Number = 1, divisor: Number = 1):
    x, y = broadcastable_list_guard(x, y)
    for x_, y_ in zip(x, y):
        copy_stochastic_(x_, (promote(x_) + promote(y_) * alpha) / divisor)


def stochastic_multiply_(x, y):
    x, y = broadcastable_list_guard(x, y)
    for x_, y_ in zip(x, y):
        copy_stochastic_(x_, promote(x_) * promote(y_))


class DivisionBackend(enum.Enum):
    eps_add = "eps_add"
    eps_clamp = "eps_clamp"
    atan2 = "atan2"
    nan_to_0 = "nan_to_0"


DivisionBackendLike = Union[DivisionBackend, str, None]


def _normalize_division_backend(backend: DivisionBackendLike) -> DivisionBackend:
    if backend is None:
        backend = _settings().default_division_backend
    if isinstance(backend, DivisionBackend):
        return backend
    try:
        return DivisionBackend(backend)
    except ValueError as err:
        raise ValueError(f"Unknown division backend '{backend}'") from err


def _apply_division_backend(x32: Tensor, y32, eps, backend: DivisionBackend) -> Tensor:
    if backend is DivisionBackend.eps_add:
        return x32 / (y32 + eps)
    if backend is DivisionBackend.eps_clamp:
        return x32 / (y32.clamp(min=eps) if isinstance(y32, Tensor) else max(y32, eps))
    if backend is DivisionBackend.atan2:
        s = _settings().atan2_scale
        return torch.atan2(x32.abs() / s, y32.abs()) * x32.sign() * y32.sign() * s
    if backend is DivisionBackend.nan_to_0:
        return torch.nan_to_num(x32 / y32, nan=0.0, posinf=0.0, neginf=0.0)
    raise AssertionError(backend)


def stochastic_divide_with_eps_(x, y, eps: float = 1e-6, *, backend: DivisionBackendLike = DivisionBackend.eps_clamp):
    x, y = broadcastable_list_guard(x, y)
    mode = _normalize_division_backend(backend)
    for x_, y_ in zip(x, y):
        copy_stochastic_(x_, _apply_division_backend(promote(x_), promote(y_), eps, mode))


def stochastic_divide_(x, y, *, backend: DivisionBackendLike = DivisionBackend.eps_clamp, eps: float = 1e-12):
    stochastic_divide_with_eps_(x, y, eps, backend=backend)


def eps_sqrt(item: Tensor, eps) -> Tensor:
    return item.sqrt().clamp(min=eps)


# --------------------------------------------------------------------------------------------------
# caution and the parameter-update epilogue
# --------------------------------------------------------------------------------------------------


def _caution_scaled(g: Tensor, update: Tensor) -> Tensor:
    """Zero the entries whose sign disagrees with the gradient and rescale the survivors so the
    mean magnitude is preserved (``numel / kept``)."""
    mask = g.signbit() ^ update.signbit()
    kept = (mask.numel() - mask.sum()).clamp(min=1)
    return update.masked_fill(mask, 0) * (mask.numel() / kept)


def _caution_unscaled(g: Tensor, update: Tensor) -> Tensor:
    return update.masked_fill(g.signbit() ^ update.signbit(), 0)


_caution_impl = _caution_scaled


def _compilable_cautioning(g: Tensor, update: Tensor) -> Tensor:
    return _caution_impl(g, update)


def caution(g, update):
    return _caution_impl(g, update)


def disable_caution_scaling():
    global _caution_impl
    _caution_impl = _caution_unscaled


def _decay_factor(p32: Tensor, u32: Tensor, decay, cautious: bool):
    if cautious:
        return decay * (1 - (p32.signbit() ^ u32.signbit()).to(p32.dtype))
    return decay


def update_param_(param, update, lr, decay, caution: bool = False, cautious_decay: bool = False, grad=None):
    """``p <- p * (1 - d * lr) - lr * u`` with optional caution mask and sign-aware decay."""
    param, update = list_guard(param, update)
    grad = list_guard(grad) if grad is not None else [None] * len(param)
    if len(grad) != len(param):
        grad = [None] * len(param)
    for p_, u_, g_ in zip(param, update, grad):
        u32 = promote(u_.view_as(p_) if u_.shape != p_.shape else u_)
        p32 = promote(p_)
        if caution:
            u32 = _caution_impl(g_, u32)
        d = _decay_factor(p32, u32, decay, cautious_decay)
        copy_stochastic_(p_, p32 * (1 - d * lr) + u32 * -lr)


_compilable_update_ = lambda p, u, decay, lr, caution, cautious_decay, g: update_param_(  # noqa: E731
    p, u, lr, decay, caution, cautious_decay, g
)


# --------------------------------------------------------------------------------------------------
# flat views over lists of tensors
# --------------------------------------------------------------------------------------------------


def flatten(x: List[Tensor], remaining: int = 0) -> Tensor:
    tail = list(x[0].shape[-remaining:]) if remaining else []
    parts = [t.reshape(-1, *tail) for t in x if t.numel()]
    if not parts:
        return torch.zeros((), dtype=x[0].dtype, device=x[0].device)
    return torch.cat(parts, 0)


def multi_flatten(*xs):
    return [flatten(x, r) for x, r in xs]


def _segments(params: List[Tensor], flat: Tensor):
    flat = flat.flatten()
    start = 0
    for p in params:
        n = p.numel()
        yield p, flat[start : start + n].view_as(p)
        start += n


def extract_from_flat_update(params: List[Tensor], update: Tensor):
    return [seg for _, seg in _segments(params, update)]


def apply_flat_update(params: List[Tensor], update: Tensor):
    for p, seg in _segments(params, update):
        copy_stochastic_(p, seg)


def apply_flat_add(params: List[Tensor], update: Tensor, alpha):
    for p, seg in _segments(params, update):
        stochastic_add_([p], [seg], alpha)


# ---------------------------------------------------------------------------------------- tensor-core products


def _tc_matmul(a: Tensor, b: Tensor, ta: bool = False, tb: bool = False, upper_upper: bool = False):
    """``op(a) @ op(b)`` on the split-tf32 tensor-core kernel when it applies (fp32 CUDA matrices on sm_100a with
    every dimension >= 128 and ``utils.tensor_core_matmul`` on), else ``None``."""
    if not (a.is_cuda and getattr(_settings(), "tensor_core_matmul", True)):
        return None
    from .. import ops

    if not ops.matmul_supported(a, b):
        return None
    return ops.matmul3(a, b, ta, tb, upper_upper=upper_upper)


def _mm(a: Tensor, b: Tensor, ta: bool = False, tb: bool = False) -> Tensor:
    out = _tc_matmul(a, b, ta, tb)
    return out if out is not None else (a.mT if ta else a) @ (b.mT if tb else b)


def _mm_upper(a: Tensor, b: Tensor) -> Tensor:
    """``a @ b`` for upper-triangular ``a`` and ``b`` (entries below their diagonals are zero): the tensor-core kernel
    walks only the K range where both are non-zero."""
    out = _tc_matmul(a, b, upper_upper=True) if a.ndim == 3 and a.shape == b.shape and a.shape[-1] == a.shape[-2] else None
    return out if out is not None else a @ b


# ---------------------------------------------------------------------------------------- blocked triangular solve

_TRSM_LEAF = 128


def _leaf_inverses(q: Tensor):
    """Inverses of the 128-wide diagonal blocks of upper-triangular ``q`` (one kernel for the whole batch) when the
    sm_100a extension applies, else ``None``."""
    if not (q.is_cuda and q.dtype == torch.float32 and q.ndim == 3 and q.stride(-1) == 1):
        return None
    from .. import ops

    if not ops.available():
        return None
    ops.launch_counter.count += 1
    return ops.load().tri_inv_blocks(q)


def _tc_sub_product(c: Tensor, a: Tensor, b: Tensor, b_transposed: bool = False) -> bool:
    """``c -= a @ b`` (``b_transposed``: ``c -= a @ b^T``) in place on the view ``c`` with the subtraction in the
    product's epilogue and the operands split straight from their views; ``False`` when the tensor-core path does not
    apply (the caller then uses plain tensor arithmetic)."""
    if not (c.is_cuda and c.dtype == torch.float32 and c.ndim == 3 and getattr(_settings(), "tensor_core_matmul", True)):
        return False
    from .. import ops

    K = a.shape[-1]
    if not ops.available() or min(c.shape[-2], c.shape[-1], K) < 128:
        return False
    if any(t.stride(-1) != 1 or t.dtype != torch.float32 for t in (a, b, c)) or c.data_ptr() % 16 or c.stride(-2) % 4 or c.stride(0) % 4:
        return False
    a_s, _ = ops.tf32_split(a, True, False)
    if b_transposed:
        b_s = a_s if (b.data_ptr() == a.data_ptr() and b.shape == a.shape and b.stride() == a.stride()) else ops.tf32_split(b, True, False)[0]
    else:
        b_s = ops.tf32_split(b, False, True)[1]
    ops.tf32_gemm(a_s, b_s, K, mode=ops.EPI_ADD, alpha=-1.0, out=c)
    return True


def _solve_right_upper_into(q: Tensor, b: Tensor, x: Tensor, inv: Tensor, first_block: int):
    """``x <- b q^-1`` for upper-triangular ``q`` through the leaf inverses ``inv``; ``b`` is consumed (its columns to the
    right receive the updates in place).  All three are views with unit inner stride; nothing is allocated besides the
    split operands, nothing is concatenated."""
    d = q.shape[-1]
    if d <= _TRSM_LEAF:
        torch.bmm(b, inv[:, first_block, :d, :d], out=x)
        return
    h = max(_TRSM_LEAF, (d // 2) // _TRSM_LEAF * _TRSM_LEAF)
    _solve_right_upper_into(q[..., :h, :h], b[..., :h], x[..., :h], inv, first_block)
    if not _tc_sub_product(b[..., h:], x[..., :h], q[..., :h, h:]):
        torch.baddbmm(b[..., h:], x[..., :h], q[..., :h, h:], alpha=-1.0, out=b[..., h:])
    _solve_right_upper_into(q[..., h:, h:], b[..., h:], x[..., h:], inv, first_block + h // _TRSM_LEAF)


def _solve_right_upper(q: Tensor, b: Tensor, inv: Optional[Tensor] = None, first_block: int = 0, consume_b: bool = False) -> Tensor:
    """``X`` with ``X q = b`` for upper-triangular ``q`` (batched).  Large CUDA problems are split recursively,
    ``X_1 = b_1 q_11^-1``, ``X_2 = (b_2 - X_1 q_12) q_22^-1``, so that everything is matrix products: the off-diagonal
    updates run on the tensor cores (subtraction in the epilogue, in place), and the 128-wide leaves multiply by block
    inverses that one small kernel prepares for the whole batch (the library's right-hand triangular solve walks the
    batch one matrix at a time at a few TFLOP/s and was half of a preconditioner update's GPU time).  ``consume_b``: the
    caller no longer needs ``b`` (it becomes the workspace instead of a copy of it)."""
    d = q.shape[-1]
    fast = q.is_cuda and q.dtype == torch.float32
    if fast and inv is None and d > 1:
        inv = _leaf_inverses(q)
        first_block = 0
    if fast and inv is not None and q.ndim == 3 and b.ndim == 3 and b.dtype == torch.float32:
        work = b if (consume_b and b.stride(-1) == 1) else b.clone(memory_format=torch.contiguous_format)
        x = torch.empty(b.shape, device=b.device, dtype=b.dtype)
        _solve_right_upper_into(q, work, x, inv, first_block)
        return x
    if d <= _TRSM_LEAF or not fast:
        if inv is not None and fast:
            return b @ inv[:, first_block, :d, :d]
        return torch.linalg.solve_triangular(q, b, upper=True, left=False)
    h = max(_TRSM_LEAF, (d // 2) // _TRSM_LEAF * _TRSM_LEAF)
    x1 = _solve_right_upper(q[..., :h, :h], b[..., :h], inv, first_block)
    x2 = _solve_right_upper(q[..., h:, h:], b[..., h:] - _mm(x1, q[..., :h, h:]), inv, first_block + h // _TRSM_LEAF)
    return torch.cat([x1, x2], dim=-1)


# ---------------------------------------------------------------------------------------- segmented reductions


def _reducible(ts) -> bool:
    first = ts[0]
    if not (first.is_cuda and first.dtype in (torch.float32, torch.bfloat16, torch.float16)):
        return False
    from .. import ops

    if torch.cuda.is_current_stream_capturing():
        return False  # these kernels read a pointer table uploaded from host memory, which a graph cannot replay
    return ops.available() and all(t.is_cuda and t.dtype == first.dtype and t.is_contiguous() and t.numel() > 0 for t in ts)


def _segmented_dot(xs, ys):
    """``[sum(x * y) for x, y in zip(xs, ys)]`` as one fp32 tensor from one kernel launch over all pairs, or ``None``
    when the kernel does not apply (CPU, mixed dtypes, non-contiguous tensors).  Block results are combined with
    floating-point atomics, so the last bits can differ between runs."""
    if not xs or len(xs) != len(ys) or not _reducible(list(xs) + list(ys)) or any(x.shape != y.shape for x, y in zip(xs, ys)):
        return None
    from .. import ops

    return ops.dot(xs, ys)


def _segmented_absmax_rows(ts):
    """``[t.abs().amax(dim=all but the first) for t in ts]`` (one fp32 tensor per input) from one kernel launch over
    every leading-index slice, or ``None`` when the kernel does not apply."""
    if not ts or any(t.ndim < 2 for t in ts) or not _reducible(ts):
        return None
    from .. import ops

    out = ops.absmax([row for t in ts for row in t.unbind(0)])
    return list(out.split([t.shape[0] for t in ts]))
