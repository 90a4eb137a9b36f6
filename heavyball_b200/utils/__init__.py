"""``heavyball_b200.utils`` — numerical primitives and the optimizer runtime.

The namespace mirrors the reference's ``heavyball.utils`` module (``heavyball/utils.py``) so code
written against it keeps working: same function names, and the same user-mutable module-level
switches, which are read at call time:

* ``zeroth_power_mode`` / ``precise_zeroth_power_mode`` — orthogonalisation method
* ``default_division_backend`` / ``atan2_scale`` — guarded division flavour
* ``dither_steps`` — number of uniform draws summed for stochastic rounding
* ``fast_qr`` — on CUDA, orthogonalise eigenbasis refreshes with batched panel-wise Cholesky QR instead of Householder QR
* ``graph_qr`` — replay that QR from a CUDA graph per shape (several hundred small launches otherwise)
* ``tensor_core_matmul`` — on sm_100a, fp32 matrix products of SOAP / PSGD with all dimensions >= 128 use the
  3-term split-tf32 tensor-core kernel (error about 2^-18 of ``|a| @ |b|``) instead of fp32 SIMT library GEMMs
* ``compile_mode`` / ``dynamic`` / ``compile_mode_recommended_to_none`` — accepted for source
  compatibility; there is no tracing compiler here, fused execution is done by the sm_100a kernels
  in ``heavyball_b200.ops``.
"""

import torch

compile_mode = "max-autotune-no-cudagraphs"
dynamic = False
compile_mode_recommended_to_none = None
zeroth_power_mode = "newtonschulz"
precise_zeroth_power_mode = "qr"
default_division_backend = "eps_clamp"
atan2_scale = 16.0
dither_steps = 1
fast_qr = True  # CUDA: eigenbasis refreshes use batched panel-wise Cholesky QR (Householder QR when that fails, and on CPU)
graph_qr = True  # replay the panel-wise QR of a given shape from a CUDA graph (it is launch-bound)
tensor_core_matmul = True  # CUDA: large fp32 products of the preconditioners run on the split-tf32 tcgen05 kernel
tiny_bf16 = torch.finfo(torch.bfloat16).tiny

from .core import *  # noqa: E402,F401,F403
from .core import (  # noqa: E402,F401
    _apply_division_backend,
    _compilable_cautioning,
    _compilable_update_,
    _EXPONENT_BIAS,
    _lerp,
    _log_ulp,
    _normalize_division_backend,
    _NUM_MANTISSA_BITS,
    _scale_by_exp2,
    _ULPState,
)
from .first_order import *  # noqa: E402,F401,F403
from .first_order import (  # noqa: E402,F401
    _compilable_exp_avg_sq_,
    _compilable_grafting,
    _compilable_schedule_free_,
    _compute_ademamix_hparams,
    _nadam_moments,
)
from .clipping import *  # noqa: E402,F401,F403
from .orthogonal import *  # noqa: E402,F401,F403
from .orthogonal import _compilable_orthogonal_  # noqa: E402,F401
from .soap import *  # noqa: E402,F401,F403
from .soap import _kl_eigvals, _kl_shampoo_kron_scale, _stable_symmetric_basis, _transform_projected_state  # noqa: E402,F401
from .psgd import *  # noqa: E402,F401,F403
from .psgd import (  # noqa: E402,F401
    _balance_to_triu,
    _inner_precond_update_prob_schedule,
    _lra_flatten_and_balance,
    _lse_mean,
    _max_idx,
    _update_lb,
)
from .optimizer import *  # noqa: E402,F401,F403
from .optimizer import _tensor_key  # noqa: E402,F401


def is_compiling():
    return False


def decorator(func):
    return func


def decorator_knowngood(func, fullgraph: bool = True):
    return func


def decorator_no_fullgraph(func):
    return func


def tree_apply(fn):
    from torch.utils._pytree import tree_map

    return lambda *args: tree_map(fn, *args)


def _ignore_warning(msg):
    import re
    import warnings

    warnings.filterwarnings("ignore", f".*{re.escape(msg)}.*")


def set_torch(benchmark_limit: int = 32, einsum_strategy: str = "auto-hq"):
    """Global PyTorch switches for training speed: cuDNN autotuning, TF32 matmuls for the library
    GEMMs that remain, ``opt_einsum`` contraction ordering when that package is installed.
    Parity: ``heavyball/utils.py:517-547``."""
    from torch.backends import cudnn, opt_einsum

    cudnn.benchmark = True
    cudnn.deterministic = False
    cudnn.benchmark_limit = benchmark_limit
    torch.use_deterministic_algorithms(False)
    torch.set_float32_matmul_precision("high")
    try:
        import opt_einsum as _oe  # noqa: F401

        opt_einsum.set_flags(True)
        opt_einsum.strategy = "auto-hq" if einsum_strategy == "heavyball" else einsum_strategy
    except ImportError:
        pass
    for msg in (
        "Using backward() with create_graph=True will create a reference cycle",
        "We recommend using autograd.grad when creating the graph to avoid this",
        "The .grad attribute of a Tensor that is not a leaf Tensor is being accessed",
    ):
        _ignore_warning(msg)
