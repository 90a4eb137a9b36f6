"""sm_100a kernels and their Python entry points.

The extension is compiled in-tree (``heavyball_b200/ops/_build``) for ``sm_100a`` only and loaded
lazily.  On a machine with a CUDA device the kernels are *the* implementation: if the extension cannot
be loaded or built, :func:`load` raises instead of silently falling back to PyTorch ops.

Entry points
------------
``fused_chain``      one multi-tensor pass: decode -> MARS -> moment rule -> caution -> decay -> write
``sumsq``            per-tensor sum of squares (segmented reduction)
``dot`` / ``absmax`` per-tensor dot products and absolute maxima (same chunk table)
``newton_schulz``    batched quintic Newton–Schulz / Polar-Express chain on tcgen05 tensor cores
``matmul3``          fp32 matrix product on the tf32 tensor cores (3-term split), for SOAP / PSGD algebra
``nn``               (sub-module) model-side ops: fused head + cross-entropy, LayerNorm (+ residual add), Linear with
                     column-sum bias gradients, bf16 cast cache
``noalloc``          (sub-module) ctypes access to the allocation-free AdamW entry point

The extension also exports ``tall_t_mul`` (product over a long dimension for the eigenbasis-refresh QR) and the peer
flag kernels used by ``heavyball_b200.parallel.ddp``.
"""

from __future__ import annotations

import importlib.util
import os
import threading
from typing import List, Optional, Sequence

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "csrc")
_BUILD = os.path.join(_HERE, "_build")
_NAME = "hb200_ops"
_SOURCES = ["bindings.cpp", "colsum.cu", "cross_entropy.cu", "fused_chain.cu", "gelu.cu", "layer_norm.cu", "ns_gemm.cu", "noalloc_adamw.cu", "peer_sync.cu", "skinny.cu", "tf32_gemm.cu"]
_lock = threading.Lock()
_ext = None
_load_error: Optional[BaseException] = None

# storage kinds (mirror of hb::DType)
F32, BF16, F16, BF16E8, BF16E16, F16E8, F16E16, NONE = range(8)
# algorithms (mirror of hb::Algo)
IDENTITY, ADAM, LAPROP, ADOPT, ADEMAMIX, RMSPROP, UNSCALED_ADAM, EXP_AVG, NESTEROV_EMA, HEAVYBALL, NESTEROV_MOM, NADAM = range(12)
OUT_PARAM, OUT_UPDATE, OUT_SCHEDULE_FREE = 0, 1, 2
CLIP_NONE, CLIP_L2, CLIP_RMS, CLIP_ORTHO = 0, 1, 2, 3
UOP_NONE, UOP_TRUST_REGION, UOP_SIGN_GRAFT, UOP_SIGN = 0, 1, 2, 3  # mirror of hb::UpdateOp
POST_NONE, POST_MSAM, POST_DECAY_IN = 0, 1, 2  # mirror of hb::PostState
MODE_GRAM, MODE_POLY, MODE_APPLY = 0, 1, 2

CUDA_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
    "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_BFLOAT16_CONVERSIONS__",
]  # fmt: skip


def _sources():
    return [os.path.join(_SRC, s) for s in _SOURCES]


def build(verbose: bool = False):
    """Compile the extension for sm_100a into the in-tree build directory (works without a GPU)."""
    from torch.utils.cpp_extension import load

    os.makedirs(_BUILD, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    mod = load(
        name=_NAME, sources=_sources(), build_directory=_BUILD, extra_cuda_cflags=CUDA_FLAGS,
        extra_cflags=["-O2", "-std=c++17"], extra_include_paths=[_SRC], verbose=verbose,
    )  # fmt: skip
    with open(os.path.join(_BUILD, "sources.sha256"), "w") as fh:
        fh.write(_source_digest())
    return mod


def _source_digest() -> str:
    import hashlib

    h = hashlib.sha256()
    for name in sorted(os.listdir(_SRC)):
        with open(os.path.join(_SRC, name), "rb") as fh:
            h.update(name.encode() + b"\0" + fh.read())
    return h.hexdigest()


def _import_prebuilt():
    so = os.path.join(_BUILD, _NAME + ".so")
    if not os.path.exists(so):
        return None
    stamp = os.path.join(_BUILD, "sources.sha256")
    if not os.path.exists(stamp) or open(stamp).read().strip() != _source_digest():
        return None  # sources changed since the library was built: rebuild
    spec = importlib.util.spec_from_file_location(_NAME, so)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def load():
    """Returns the extension module, importing the prebuilt library or compiling it."""
    global _ext, _load_error
    if _ext is not None:
        return _ext
    with _lock:
        if _ext is not None:
            return _ext
        if _load_error is not None:
            raise RuntimeError("heavyball_b200.ops: extension unavailable") from _load_error
        try:
            _ext = _import_prebuilt() or build()
            tile = os.environ.get("HB200_NS_TILE")  # tuning aid: force the 128 or 256 output tile of the Newton-Schulz GEMMs
            if tile:
                _ext.set_ns_gemm_tile(int(tile))
            tile = os.environ.get("HB200_TF32_TILE")  # same for the split-tf32 GEMM
            if tile:
                _ext.set_tf32_gemm_tile(int(tile))
        except BaseException as err:  # noqa: BLE001
            _load_error = err
            raise RuntimeError(
                "heavyball_b200.ops: the sm_100a extension could not be loaded or built; "
                "run `python -c 'import __graft_entry__ as g; g.build()'` from the repository root"
            ) from err
    return _ext


def available() -> bool:
    """True when kernels can run here: a CUDA device of compute capability 10.x is present.  The
    extension itself is loaded on first use and failure to load is an error, not a fallback."""
    if os.environ.get("HB200_DISABLE_OPS") == "1":
        return False
    if not torch.cuda.is_available():
        return False
    major, _ = torch.cuda.get_device_capability()
    return major == 10


class _LaunchCounter:
    """Counts kernel launches issued through this module (benchmarks report it)."""

    def __init__(self):
        self.count = 0

    def reset(self):
        self.count = 0


launch_counter = _LaunchCounter()


# ---------------------------------------------------------------------------------------- element-wise


def dtype_code(t: Optional[torch.Tensor], ecc: Optional[str] = None) -> int:
    if t is None:
        return NONE
    if ecc:
        return {"bf16+8": BF16E8, "bf16+16": BF16E16, "fp16+8": F16E8, "fp16+16": F16E16}[ecc]
    return {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}[t.dtype]


_EMPTY: List = []


def fused_chain(*, p=_EMPTY, pe=_EMPTY, g=_EMPTY, u=_EMPTY, s0=_EMPTY, s0e=_EMPTY, s1=_EMPTY, s1e=_EMPTY, s2=_EMPTY,
                s2e=_EMPTY, mars=_EMPTY, marse=_EMPTY, scale=None, masked=None, gsq=None, **cfg):  # fmt: skip
    cfg["mars"] = 1 if len(mars) else 0
    launch_counter.count += 1
    load().fused_chain(
        list(p), list(pe), list(g), list(u), list(s0), list(s0e), list(s1), list(s1e), list(s2), list(s2e), list(mars),
        list(marse), scale, masked, gsq, cfg,
    )  # fmt: skip


def sumsq(xs: Sequence[torch.Tensor]) -> torch.Tensor:
    launch_counter.count += 1
    return load().sumsq(list(xs), dtype_code(xs[0]))


def dot(xs: Sequence[torch.Tensor], ys: Sequence[torch.Tensor]) -> torch.Tensor:
    """fp32 ``[sum(x_i * y_i)]`` for contiguous tensors of one dtype (fp32 / bf16 / fp16), one launch."""
    launch_counter.count += 1
    return load().segmented_reduce(list(xs), list(ys), dtype_code(xs[0]), 0)


def absmax(xs: Sequence[torch.Tensor]) -> torch.Tensor:
    """fp32 ``[max |x_i|]`` for contiguous tensors of one dtype, one launch; a NaN element gives NaN."""
    launch_counter.count += 1
    return load().segmented_reduce(list(xs), [], dtype_code(xs[0]), 1)


# ---------------------------------------------------------------------------------------- Newton–Schulz


def _round_up(x, m):
    return (x + m - 1) // m * m


_status_cache = {}


def _status(device):
    st = _status_cache.get(device)
    if st is None:
        st = _status_cache[device] = torch.zeros(1, dtype=torch.int32, device=device)
    return st


def check_status(device=None):
    """Raises if any tensor-core kernel reported an expired wait since the last check (host sync)."""
    for dev, st in list(_status_cache.items()):
        if device is not None and dev != device:
            continue
        if int(st.item()) != 0:
            st.zero_()
            raise RuntimeError("heavyball_b200.ops: a Newton–Schulz GEMM aborted on a bounded wait")


def ns_supported(R: int, C: int) -> bool:
    return min(R, C) >= 8 and max(R, C) >= 64


def newton_schulz_batched(mats: Sequence[torch.Tensor], coeffs, out: Optional[torch.Tensor] = None, out_scale=1.0,
                          eps: float = 1e-7, seed: Optional[int] = None, sumsq: Optional[torch.Tensor] = None) -> torch.Tensor:  # fmt: skip
    """Orthogonalises a list of same-shape ``(R, C)`` fp32 / bf16 matrices; returns fp32 ``(B, R, C)``
    holding ``out_scale * polar_factor``.  ``coeffs`` is a sequence of ``(a, b, c)`` per step.  ``sumsq``
    (fp32, one squared Frobenius norm per matrix) skips the reduction pass when the caller already has it."""
    ext = load()
    B = len(mats)
    R, C = mats[0].shape
    dev = mats[0].device
    m, n = (R, C) if R <= C else (C, R)
    ldx, ldxt, lds = _round_up(n, 8), _round_up(m, 8), _round_up(m, 8)
    bf = dict(dtype=torch.bfloat16, device=dev)
    X = [torch.empty(B, m, ldx, **bf) for _ in range(2)]
    XT = [torch.empty(B, n, ldxt, **bf) for _ in range(2)]
    S = torch.empty(B, m, lds, **bf)
    Y = torch.empty(B, m, lds, **bf)
    if out is None:
        out = torch.empty(B, R, C, dtype=torch.float32, device=dev)
    if seed is None:
        seed = int(torch.randint(0, 2**62, (1,)).item())
    srcs = [t.contiguous() for t in mats]
    if sumsq is None:
        norms = ext.sumsq(srcs, dtype_code(mats[0]))
        launch_counter.count += 1
    else:
        norms = sumsq.contiguous()
    if R <= C:
        ext.ns_prepare(srcs, dtype_code(mats[0]), R, C, norms, eps, X[0], ldx, XT[0], ldxt, seed)
    else:  # work on the transpose so that the Gram matrix is the small one
        ext.ns_prepare(srcs, dtype_code(mats[0]), R, C, norms, eps, XT[0], ldxt, X[0], ldx, seed)
    status = _status(dev)
    launch_counter.count += 1 + 3 * len(coeffs)
    # one call issues the three launches of every step (Gram, polynomial, apply; the last apply writes `out`)
    ext.ns_chain(X, XT, S, Y, out, m, n, ldx, ldxt, lds, R, C, [[float(v) for v in abc] for abc in coeffs], float(out_scale),
                 status)  # fmt: skip
    return out


def newton_schulz(G: torch.Tensor, coeffs, out_scale: float = 1.0) -> Optional[torch.Tensor]:
    """Drop-in for the PyTorch iteration on one ``(..., R, C)`` tensor; ``None`` if the shape is not
    covered by the kernel (the caller then uses the PyTorch definition)."""
    if G.ndim < 2 or G.dtype not in (torch.float32, torch.bfloat16):
        return None
    R, C = G.shape[-2:]
    if not ns_supported(R, C):
        return None
    mats = list(G.reshape(-1, R, C).unbind(0))
    res = newton_schulz_batched(mats, coeffs, out_scale=out_scale)
    return res.reshape(G.shape).to(G.dtype)


# ---------------------------------------------------------------------------------------- fp32 matmul on tensor cores


def matmul_supported(a: torch.Tensor, b: torch.Tensor) -> bool:
    """True when :func:`matmul3` applies: fp32 CUDA matrices on sm_100a, large enough for 128 x 128 tiles to pay."""
    return (
        a.is_cuda and b.is_cuda and a.dtype == torch.float32 and b.dtype == torch.float32 and a.ndim >= 2 and b.ndim >= 2
        and min(a.shape[-1], a.shape[-2], b.shape[-1], b.shape[-2]) >= 128 and available()
    )  # fmt: skip


EPI_STORE, EPI_LERP, EPI_ADAM, EPI_LAPROP, EPI_ADD = range(5)  # mirror of hb::Tf32EpilogueMode
SPLIT_NONE, SPLIT_ROWS, SPLIT_COLS = range(3)


def tf32_split(x: torch.Tensor, same: bool = True, trans: bool = False):
    """Split-tf32 operands of an fp32 ``[batch, R, C]`` tensor or view (unit inner stride), one pass over ``x``.  Returns ``(same, trans)``:
    ``same`` has the rows of ``x`` as operand rows (``K = C``), ``trans`` its columns (``K = R``); an orientation that
    was not asked for is ``None``.  Either buffer can be the left or the right operand of :func:`tf32_gemm`, so matrices
    that rarely change (eigenbases, preconditioner factors) are split once and kept."""
    launch_counter.count += 1
    s, t = load().tf32_split(x, same, trans)
    return (s if same else None), (t if trans else None)


def tf32_gemm(a2: torch.Tensor, b2: torch.Tensor, K: int, *, mode: int = EPI_STORE, alpha: float = 1.0, w: float = 0.0,
              b1: float = 0.0, b2c: float = 0.0, eps: float = 0.0, out: Optional[torch.Tensor] = None,
              split_out: int = SPLIT_NONE, m: Optional[torch.Tensor] = None, v: Optional[torch.Tensor] = None):  # fmt: skip
    """``epilogue(A @ B^T)`` over split operands (``a2``: ``[batch, M, 2 kp(K)]``, ``b2``: ``[batch, N, 2 kp(K)]``) at
    fp32-level accuracy on the tf32 tensor cores.

    ``mode``: ``EPI_STORE`` writes ``alpha * acc``; ``EPI_LERP`` updates ``out <- out + (alpha * acc - out) * w`` in place;
    ``EPI_ADD`` updates ``out <- out + alpha * acc`` in place (``out`` may be a view with unit inner stride);
    ``EPI_ADAM`` / ``EPI_LAPROP`` advance the fp32 moments ``m``, ``v`` (``[batch, M, N]``, in place, coefficients ``b1``,
    ``b2c`` already debiased) with ``alpha * acc`` as the gradient and pass the preconditioned value on.
    ``out`` (fp32 ``[batch, M, N]``) receives the result; ``split_out`` additionally (or instead) returns it as a split
    operand for the next product: ``SPLIT_ROWS`` with the result's rows as operand rows, ``SPLIT_COLS`` with its columns."""
    launch_counter.count += 1
    s = load().tf32_gemm(a2, b2, K, mode, alpha, w, b1, b2c, eps, out, split_out, m, v, _status(a2.device))
    return s if split_out else None


def matmul3(a: torch.Tensor, b: torch.Tensor, trans_a: bool = False, trans_b: bool = False, alpha: float = 1.0,
            upper_upper: bool = False) -> torch.Tensor:
    """``alpha * op(a) @ op(b)`` for fp32 matrices (optionally batched, equal leading shapes) on the tf32 tensor
    cores with the 3-term split (measured error about 2^-18 of ``|a| @ |b|``; one tf32 pass gives 2^-11, fp32 SIMT 2^-21).
    ``upper_upper``: ``op(a)`` and ``op(b)`` are upper triangular matrices of one size (entries below their diagonals
    ARE zero): a sixth of the tile products, and exact zeros below the diagonal of the result."""
    lead = a.shape[:-2]
    if b.shape[:-2] != lead:
        lead = torch.broadcast_shapes(a.shape[:-2], b.shape[:-2])
        a, b = a.expand(*lead, *a.shape[-2:]), b.expand(*lead, *b.shape[-2:])
    a3 = a.reshape(-1, *a.shape[-2:]).contiguous()
    b3 = b.reshape(-1, *b.shape[-2:]).contiguous()
    out = load().tf32x3_matmul(a3, b3, trans_a, trans_b, alpha, _status(a.device), upper_upper)
    launch_counter.count += 3
    return out.reshape(*lead, *out.shape[-2:])
