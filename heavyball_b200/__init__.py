"""heavyball_b200 — Blackwell-native optimizer library with HeavyBall's API and checkpoint format.

Public surface (parity with ``heavyball/__init__.py:13-1851``): 37 chain-based
``torch.optim.Optimizer`` classes, the ``SplitOpt`` and ``SAMWrapper`` meta-optimizers and
``capture_param_shapes``.  Each class is a thin constructor: it validates keyword arguments, turns
them into param-group defaults and hands a chain of transforms (``heavyball_b200.chainable``) to
``BaseOpt``.  Constructors are generated from one-line signature specs below; ``inspect.signature``
reports the full explicit signature, argument order matches the reference for positional callers.

Class attributes are overridable defaults (``gradient_clipping``, ``update_clipping``, ``palm``,
``auto_fuse``; ``use_precond_schedule`` for the SOAP family; ``delayed`` / ``cached`` /
``exp_avg_input`` / ``sqrt`` for PSGD), so subclassing to change a default keeps working.
"""

from __future__ import annotations

import functools
import inspect
import math
from typing import Type, Union

import torch
import torch.optim

from . import chainable as C
from . import utils

__version__ = "0.1.0"

ShapeMap = dict[int, tuple[int, ...]]
D = C.use_default

# --------------------------------------------------------------------------------------------------
# signature building blocks (order matters: positional compatibility)
# --------------------------------------------------------------------------------------------------
_FLAGS = (
    "multi_tensor=True, storage_dtype='float32', mars=False, caution=False, mars_gamma=0.0025, "
    "gradient_clipping=D, update_clipping=D"
)
_PALM = "palm=D, beta2_scale=0.8"
_TAIL = "compile_step=D, promote=D, ecc=None, param_ecc=None, orig_shapes=None"
_ADAM_HEAD = "lr=0.0025, betas=(0.9, 0.99), eps=1e-8, weight_decay=0, cautious_weight_decay=False, warmup_steps=0"
_ADAM_SIG = f"{_ADAM_HEAD}, {_FLAGS}, {_PALM}, {_TAIL}"
_SF_HEAD = (
    "lr=0.0025, betas=(0.9, 0.99), eps=1e-6, weight_decay=0, cautious_weight_decay=False, warmup_steps=0, r=0.0, "
    "weight_lr_power=2.0"
)
_SOAP_HEAD = (
    "lr=3e-3, betas={betas}, shampoo_beta=0.95, eps=1e-8, weight_decay=0.01, cautious_weight_decay=False, "
    "precondition_frequency=2, max_precond_dim=2048, merge_dims=True, precondition_1d=False, warmup_steps=0, "
    "split=False, multi_tensor=True, mars=False, caution=False, mars_gamma=0.0025, palm=D, "
    "precond_scheduler=(1 / 3, 9), beta2_scale=0.8, use_precond_schedule=D, gradient_clipping=D, update_clipping=D, "
    "storage_dtype='float32', precond_grad_accum=False"
)
_PSGD_EXPERT = (
    "precond_init_scale=None, precond_init_scale_scale=1, precond_init_scale_power=None, precond_lr=0.1"
)
_HVP = "finite_differences=D, fallback_to_finite_differences=D, hvp_interval=D, hessian_approx=D"
_KRON_HEAD = (
    "lr=0.001, beta=None, betas=(0.9, 0.999), {eps}weight_decay=0.0, cautious_weight_decay=False, "
    "preconditioner_update_probability=D, max_size_triangular=2048, min_ndim_triangular=2, memory_save_mode=None, "
    "momentum_into_precond_update=True, warmup_steps=0, merge_dims=False, split=False, {line}multi_tensor=True, "
    "q_dtype='float32', storage_dtype='float32', mars=False, caution=False, mars_gamma=0.0025"
)
_KRON_MID = (
    "gradient_clipping=D, update_clipping=D, precond_grad_accum=False, lower_bound_beta=0.9, dampening=1e-9, "
    "precond_update_power_iterations=2"
)


def _parse(spec: str) -> dict:
    return eval(f"dict({spec})", {"D": D})  # specs are literals defined in this file


def _make_init(spec: str, body):
    """Creates ``__init__(self, params, <spec>, **kwargs)`` that calls ``body(self, L)`` with ``L`` shaped
    like the ``locals()`` of a hand-written constructor."""
    fields = _parse(spec)
    P = inspect.Parameter
    sig = inspect.Signature(
        [P("self", P.POSITIONAL_OR_KEYWORD), P("params", P.POSITIONAL_OR_KEYWORD)]
        + [P(k, P.POSITIONAL_OR_KEYWORD, default=v) for k, v in fields.items()]
        + [P("kwargs", P.VAR_KEYWORD)]
    )

    def __init__(self, *args, **kwargs):
        bound = sig.bind(self, *args, **kwargs)
        bound.apply_defaults()
        L = dict(bound.arguments)
        L.setdefault("kwargs", {})
        L["kwargs"] = dict(L["kwargs"])
        body(self, L)

    __init__.__signature__ = sig
    return __init__


def _simple(fns_of, *, palm=True, check=None):
    """Constructor body for classes that go straight to ``BaseOpt`` with a fixed chain."""

    def body(self, L):
        if check is not None:
            check(L)
        fns = fns_of(L)
        params, defaults = C._build_defaults(L)
        C.BaseOpt.__init__(
            self, params, defaults, L["gradient_clipping"], L["update_clipping"], L["palm"] if palm else D, fns=fns
        )

    return body


def _define(name, spec, body, doc, base=C.BaseOpt, **attrs):
    cls = type(name, (base,), {"__init__": _make_init(spec, body), "__doc__": doc, "__module__": __name__, **attrs})
    cls.__init__.__qualname__ = f"{name}.__init__"
    return cls


def _is_matrix(p):
    return p.ndim >= 2


# --------------------------------------------------------------------------------------------------
# first-order and orthogonalising optimizers
# --------------------------------------------------------------------------------------------------

SGD = _define(
    "SGD",
    f"lr=0.0025, beta=0.9, weight_decay=0, cautious_weight_decay=False, warmup_steps=0, {_FLAGS}, {_TAIL}",
    _simple(lambda L: (C.heavyball_momentum,), palm=False),
    "SGD with heavy-ball momentum.",
)

AdamW = _define(
    "AdamW", _ADAM_SIG, _simple(lambda L: (C.update_by_adam,)),
    "AdamW (Loshchilov & Hutter, https://arxiv.org/abs/1711.05101): decoupled weight decay, debiased EMAs, "
    "``max(sqrt(v), eps)`` denominator.",
)  # fmt: skip

NAdam = _define(
    "NAdam",
    "lr=0.002, betas=(0.9, 0.999), eps=1e-8, weight_decay=0, cautious_weight_decay=False, momentum_decay=4e-3, "
    f"decoupled_weight_decay=False, warmup_steps=0, {_FLAGS}, {_PALM}, {_TAIL}",
    _simple(lambda L: (C.update_by_nadam,)),
    "NAdam (Dozat, 2016): Adam with Nesterov momentum and the 0.96-decay momentum schedule.",
)


def _check_three_betas(L):
    if len(L["betas"]) != 3:
        raise ValueError("AdEMAMix expects betas with three coefficients.")


AdEMAMix = _define(
    "AdEMAMix",
    "lr=0.001, betas=(0.9, 0.999, 0.9999), eps=1e-8, weight_decay=0, cautious_weight_decay=False, alpha=2.0, "
    f"beta3_warmup=None, alpha_warmup=None, warmup_steps=0, {_FLAGS}, {_TAIL}",
    _simple(lambda L: (C.update_by_ademamix,), palm=False, check=_check_three_betas),
    "AdEMAMix (https://arxiv.org/abs/2409.03137): fast + slow gradient EMAs mixed with weight ``alpha``.",
)

UnscaledAdamW = _define(
    "UnscaledAdamW", _ADAM_SIG, _simple(lambda L: (C.scale_by_unscaled_adam,)),
    "AdamW whose momentum is taken over normalised gradients and rescaled by the current denominator.",
)  # fmt: skip

SUDSAdamW = _define(
    "SUDSAdamW",
    f"{_ADAM_HEAD}, {_FLAGS}, {_PALM}, precond_lr=1e-2, {_TAIL}",
    _simple(lambda L: (C.scale_by_suds,)),
    "AdamW in the eigenbasis of a rank-1 curvature sketch tracked with Oja's rule.",
)


def _check_scion(L):
    if L["lr"] < 0:
        raise ValueError(f"Invalid learning rate: {L['lr']}")
    if len(L["betas"]) == 0:
        raise ValueError("Scion expects at least one beta.")
    if not 0 <= L["betas"][0] <= 1:
        raise ValueError(f"Invalid momentum value: {L['betas'][0]}")


def _scion_body(self, L):
    _check_scion(L)
    betas = L["betas"]
    beta1 = betas[0]
    beta2 = betas[1] if len(betas) > 1 else beta1
    params, defaults = C._build_defaults({**L, "beta1": beta1, "beta2": beta2})
    defaults["betas"] = (beta1, beta2)
    defaults["scale"] = L["scale"]
    C.BaseOpt.__init__(
        self, params, defaults, L["gradient_clipping"], L["update_clipping"], fns=(C.exp_avg, C.scion_auto_norm)
    )


Scion = _define(
    "Scion",
    f"{_ADAM_HEAD}, {_FLAGS}, scale=1.0, {_TAIL}",
    _scion_body,
    "Scion (https://arxiv.org/abs/2502.07529): momentum followed by a norm-constrained LMO chosen per tensor rank "
    "(spectral for matrices and conv kernels, RMS for vectors).",
)


def _adamc_body(self, L):
    if L["max_lr"] is None:
        utils.warn_once(
            "max_lr was not set. setting it to the current learning rate, under the assumption that it strictly decreases"
        )
        L = {**L, "max_lr": L["lr"]}
    _simple(lambda _: (C.update_by_adamc,))(self, L)


AdamC = _define(
    "AdamC",
    "lr=0.0025, betas=(0.9, 0.99), eps=1e-8, weight_decay=0, cautious_weight_decay=False, max_lr=None, "
    f"warmup_steps=0, {_FLAGS}, {_PALM}, {_TAIL}",
    _adamc_body,
    "AdamC (https://arxiv.org/abs/2506.02285): weight decay scaled by ``lr / max_lr``.",
)

RMSprop = _define(
    "RMSprop", f"{_SF_HEAD}, {_FLAGS}, {_PALM}, {_TAIL}", _simple(lambda L: (C.scale_by_exp_avg_sq,)),
    "Debiased RMSprop (not ``torch.optim.RMSprop``): second-moment scaling with Adam's bias correction.",
)  # fmt: skip

HyperBallAdamW = _define(
    "HyperBallAdamW",
    _ADAM_SIG,
    _simple(lambda L: (C.scale_by_exp_avg_sq, C.route((_is_matrix, C.update_by_hyperball), default=C.apply_update))),
    "Second-moment scaling; matrices then move on a sphere of their initial norm, other tensors take a plain step.",
)


def _muon_momentum(L):
    if L.get("heavyball_momentum"):
        return C.nesterov_momentum if L["nesterov"] else C.heavyball_momentum
    return C.nesterov_ema if L["nesterov"] else C.exp_avg


MuonAdamW = _define(
    "MuonAdamW",
    f"{_ADAM_HEAD}, {_FLAGS}, {_PALM}, nesterov=True, {_TAIL}",
    _simple(
        lambda L: (C.route((_is_matrix, (_muon_momentum(L), C.orthogonalize_update)), default=C.scale_by_adam),)
    ),
    "Muon for tensors with two or more dims, AdamW for the rest, in one optimizer.",
)

SFAdamW = _define(
    "SFAdamW", f"{_SF_HEAD}, {_FLAGS}, {_PALM}, {_TAIL}",
    _simple(lambda L: (C.scale_by_exp_avg_sq, C.update_by_schedule_free)),
    "Schedule-Free AdamW (https://arxiv.org/abs/2405.15682).  Call ``.eval()`` / ``.train()`` around evaluation.",
    base=C.ScheduleFree,
)  # fmt: skip

MSAMLaProp = _define(
    "MSAMLaProp", f"{_SF_HEAD}, {_FLAGS}, {_PALM}, sam_step_size=0.1, {_TAIL}",
    _simple(lambda L: (C.scale_by_exp_avg_sq, C.update_by_msam)),
    "RMSprop-scaled Momentum-SAM (https://arxiv.org/abs/2401.12033).  Call ``.eval()`` / ``.train()`` around "
    "evaluation.",
    base=C.MSAM,
)  # fmt: skip

ADOPT = _define(
    "ADOPT", _ADAM_SIG, _simple(lambda L: (C.update_by_adopt,)),
    "ADOPT (https://arxiv.org/abs/2411.02853): normalise by the previous second moment; first step only seeds it.",
)  # fmt: skip

Muon = _define(
    "Muon",
    f"{_ADAM_HEAD}, {_FLAGS}, {_PALM}, nesterov=True, heavyball_momentum=False, {_TAIL}",
    _simple(lambda L: (_muon_momentum(L), C.orthogonalize_update)),
    "Muon (https://kellerjordan.github.io/posts/muon/): momentum, then Newton–Schulz orthogonalisation of every "
    "matrix-shaped update, scaled by ``max(1, rows/cols)**0.5``.",
)

LaProp = _define(
    "LaProp", _ADAM_SIG, _simple(lambda L: (C.update_by_laprop,)),
    "LaProp (https://arxiv.org/abs/2002.04839): momentum over second-moment-normalised gradients.",
)  # fmt: skip

MuonLaProp = _define(
    "MuonLaProp", _ADAM_SIG, _simple(lambda L: (C.scale_by_laprop, C.orthogonalize_update)),
    "LaProp feeding Muon's orthogonalisation.",
)  # fmt: skip

SignLaProp = _define(
    "SignLaProp", _ADAM_SIG, _simple(lambda L: (C.scale_by_laprop, C.sign)),
    "LaProp followed by a norm-preserving sign of the update.",
)  # fmt: skip

OrthoLaProp = _define(
    "OrthoLaProp", _ADAM_SIG, _simple(lambda L: (C.orthogonalize_grad_to_param, C.scale_by_laprop)),
    "OrthoGrad (https://arxiv.org/abs/2501.04697) applied to the gradient, then LaProp.",
)  # fmt: skip

LaPropOrtho = _define(
    "LaPropOrtho", _ADAM_SIG, _simple(lambda L: (C.scale_by_laprop, C.orthogonalize_grad_to_param)),
    "LaProp, then OrthoGrad applied to the update.",
)  # fmt: skip


# --------------------------------------------------------------------------------------------------
# SOAP family
# --------------------------------------------------------------------------------------------------


class SOAPBase(C.BaseOpt):
    use_precond_schedule: bool = False

    def _build_soap_defaults(self, locals_dict, fns):
        """Turns the constructor's arguments into group defaults and picks how often the eigenbases are refreshed:
        a fixed period (``precondition_frequency``) or the decaying schedule (``precond_scheduler``); the option that
        is not in use is dropped from the defaults."""
        params, defaults = C._build_defaults(locals_dict)
        period, scheduler = defaults.pop("precondition_frequency"), defaults.pop("precond_scheduler")
        if C.default(locals_dict["use_precond_schedule"], self.use_precond_schedule):
            self.precond_schedule = utils.get_soap_precond_schedule(scheduler)
        else:
            self.precond_schedule = 1 / period
        clips = (locals_dict["gradient_clipping"], locals_dict["update_clipping"])
        C.BaseOpt.__init__(self, params, defaults, *clips, locals_dict.get("palm", False), fns=fns)


def _soap_body(self, L):
    self._build_soap_defaults(L, fns=self._chain_fns)


def _soap_spec(betas, extra=""):
    return f"{_SOAP_HEAD.format(betas=betas)}, {extra}{_TAIL}"


SOAP = _define(
    "SOAP", _soap_spec("(0.9, 0.95)"), _soap_body,
    "SOAP (https://arxiv.org/abs/2409.11321): Adam in the slowly refreshed eigenbasis of Shampoo's Kronecker factors.",
    base=SOAPBase, _chain_fns=(C.scale_by_soap,),
)  # fmt: skip

KLShampoo = _define(
    "KLShampoo",
    f"{_SOAP_HEAD.format(betas='(0.9, 0.95)')}, {_TAIL}, init_factor=0.1, dampening=1e-9",
    _soap_body,
    "KL-Shampoo (https://arxiv.org/abs/2509.03378): Kronecker preconditioner with KL-corrected statistics applied to "
    "a momentum EMA; factors start at ``init_factor * I``.",
    base=SOAPBase, _chain_fns=(C.scale_by_kl_shampoo,),
)  # fmt: skip

SOAPNAdam = _define(
    "SOAPNAdam", _soap_spec("(0.9, 0.999)", "momentum_decay=4e-3, decoupled_weight_decay=False, "), _soap_body,
    "SOAP with NAdam in the eigenbasis.", base=SOAP, _chain_fns=(C.scale_by_soap_nadam,),
)  # fmt: skip

SOAPAdEMAMix = _define(
    "SOAPAdEMAMix", _soap_spec("(0.9, 0.95, 0.999)", "alpha=2.0, beta3_warmup=None, alpha_warmup=None, "), _soap_body,
    "SOAP with AdEMAMix in the eigenbasis.", base=SOAP, _chain_fns=(C.scale_by_soap_ademamix,),
)  # fmt: skip


def _variant(name, base, fn, doc):
    return type(name, (base,), {"_chain_fns": (fn,), "__doc__": doc, "__module__": __name__})


KLSOAP = _variant("KLSOAP", SOAP, C.scale_by_kl_soap, "SOAP with KL-Shampoo's two-sided factor statistics.")
SOLP = _variant("SOLP", SOAP, C.scale_by_soap_laprop, "SOAP with LaProp in the eigenbasis.")
HeavySOAP = _variant(
    "HeavySOAP", SOAP, C.scale_by_heavy_soap,
    "SOAP with post-orthogonalisation eigenvector sorting and Hadamard-square transport of the second moment.",
)  # fmt: skip
HeavyKLSOAP = _variant(
    "HeavyKLSOAP", KLSOAP, C.scale_by_heavy_kl_soap, "KLSOAP with HeavySOAP's refresh and pseudo-inverse KL weights."
)
HeavyKLShampoo = _variant(
    "HeavyKLShampoo", KLShampoo, C.scale_by_heavy_kl_shampoo, "KLShampoo with pseudo-inverse KL weights."
)
HeavySOAPNAdam = _variant("HeavySOAPNAdam", SOAPNAdam, C.scale_by_heavy_soap_nadam, "SOAPNAdam with HeavySOAP's refresh.")
HeavySOAPAdEMAMix = _variant(
    "HeavySOAPAdEMAMix", SOAPAdEMAMix, C.scale_by_heavy_soap_ademamix, "SOAPAdEMAMix with HeavySOAP's refresh."
)
HeavySOLP = _variant("HeavySOLP", SOLP, C.scale_by_heavy_soap_laprop, "SOLP with HeavySOAP's refresh.")


# --------------------------------------------------------------------------------------------------
# PSGD family
# --------------------------------------------------------------------------------------------------


class PSGDBase(C.BaseOpt):
    delayed: bool = False
    cached: bool = False
    exp_avg_input: bool = True
    sqrt: bool = False  # apply Q (a square root of P = Q^T Q) instead of P

    def _build_psgd_defaults(self, locals_dict, fns, *, default_update_clipping=utils.trust_region_clip_,
                             extra_defaults=None):  # fmt: skip
        """Group defaults of the PSGD family.  Class attributes supply what the caller left at ``use_default``
        (momentum in front of the preconditioner, trust-region clipping of the update); the fitting probability is
        taken out of the defaults and kept as the schedule."""
        resolved = dict(locals_dict)
        resolved["exp_avg_input"] = C.default(locals_dict.get("exp_avg_input", D), self.exp_avg_input)
        resolved["update_clipping"] = C.default(locals_dict["update_clipping"], default_update_clipping)
        params, defaults = C._build_defaults(resolved)
        probability = defaults.pop("preconditioner_update_probability")
        self.precond_schedule = C.default(probability, utils.precond_update_prob_schedule())
        defaults.update(extra_defaults or {})
        if self.sqrt:
            defaults["sqrt"] = True
        chain = ((C.exp_avg,) if resolved["exp_avg_input"] else ()) + tuple(fns)
        C.BaseOpt.__init__(self, params, defaults, resolved["gradient_clipping"], resolved["update_clipping"], False, fns=chain)


def _kron_body(self, L):
    delayed = C.default(L["delayed"], self.delayed)
    cached = C.default(L["cached"], self.cached)
    L = {**L, "delayed": delayed, "cached": cached}
    self._build_psgd_defaults(
        L, fns=(functools.partial(C.scale_by_delayed_psgd if delayed else C.scale_by_psgd, cached=cached),)
    )


PSGDKron = _define(
    "PSGDKron",
    f"{_KRON_HEAD.format(eps='', line='store_triu_as_line=True, ')}, delayed=D, cached=D, exp_avg_input=D, "
    f"{_KRON_MID}, {_PSGD_EXPERT}, {_HVP}, {_TAIL}",
    _kron_body,
    "PSGD with a Kronecker-factored, Lie-group-fitted preconditioner (https://arxiv.org/abs/1512.04202).",
    base=PSGDBase,
)


def _lather_body(self, L):
    self._build_psgd_defaults({**L, "exp_avg_input": False}, fns=(C.scale_by_lather,))


LATHER = _define(
    "LATHER",
    f"{_KRON_HEAD.format(eps='eps=1e-8, ', line='store_triu_as_line=True, ')}, {_KRON_MID}, {_PSGD_EXPERT}, {_HVP}, "
    f"{_TAIL}",
    _lather_body,
    "LATHER: Adam in the approximate eigenbasis of the PSGD-Kron preconditioner.",
    base=PSGDBase,
)


def _pro_body(self, L):
    cached = C.default(L["cached"], self.cached)
    L = {**L, "cached": cached}
    self._build_psgd_defaults(
        L, fns=(functools.partial(C.scale_by_psgd_pro, cached=cached),), default_update_clipping=None,
        extra_defaults={"store_triu_as_line": False},
    )  # fmt: skip


PSGDPRO = _define(
    "PSGDPRO",
    f"{_KRON_HEAD.format(eps='', line='')}, cached=D, exp_avg_input=D, {_KRON_MID}, {_PSGD_EXPERT}, {_TAIL}",
    _pro_body,
    "PSGD-Kron with the Q0.5EQ1.5 (Procrustes) update that keeps factors near-symmetric "
    "(https://arxiv.org/abs/2402.11858).",
    base=PSGDBase,
)

QSGD = type(
    "QSGD", (PSGDPRO,),
    {"sqrt": True, "__module__": __name__,
     "__doc__": "PSGDPRO applying the factor Q (about P^0.5) instead of P = Q^T Q when preconditioning."},
)  # fmt: skip


def _lra_body(self, L):
    delayed = C.default(L["delayed"], self.delayed)
    rank = L["rank"]
    params = L["params"]
    if rank is None:
        utils.warn_once(
            f"{rank=}. It will be set to log2(param_count). This requires `params` to be of type list. "
            f"Currently, {type(params)=}"
        )
        params = list(params)
        rank = max(1, round(math.log2(sum(p.numel() for p in params))))
        utils.warn_once(f"rank was set to {rank}")
    L = {**L, "delayed": delayed, "rank": rank, "params": params}
    self._build_psgd_defaults(L, fns=(C.scale_by_delayed_psgd_lra if delayed else C.scale_by_psgd_lra,))


PSGDLRA = _define(
    "PSGDLRA",
    "lr=0.001, beta=0.9, weight_decay=0.0, cautious_weight_decay=False, preconditioner_update_probability=D, "
    "momentum_into_precond_update=True, rank=None, warmup_steps=0, multi_tensor=True, q_dtype='float32', "
    "storage_dtype='float32', mars=False, caution=False, mars_gamma=0.0025, delayed=D, exp_avg_input=D, "
    f"gradient_clipping=D, update_clipping=D, eps=1e-8, precond_grad_accum=False, {_PSGD_EXPERT}, {_HVP}, {_TAIL}",
    _lra_body,
    "PSGD with a low-rank preconditioner.  ``multi_tensor=True`` fits one approximation across the whole group, "
    "``False`` one per parameter; these are different algorithms.",
    base=PSGDBase,
)


# --------------------------------------------------------------------------------------------------
# meta-optimizers
# --------------------------------------------------------------------------------------------------


class SplitOpt(utils.StatefulOptimizer):
    """Delegates parameter subsets to different optimizers::

        opt = SplitOpt([
            {'params': matrices, 'optimizer': Muon, 'lr': 0.02},
            {'params': vectors, 'optimizer': AdamW, 'lr': 0.001},
        ])

    Every spec is ``{"params": ..., "optimizer": class, **constructor arguments}``; specs without parameters are
    dropped.  The checkpoint is ``{"optimizers": [state_dict of each member, in order]}``.
    """

    def __init__(self, specs):
        members, covered = [], []
        for spec in specs:
            options = {k: v for k, v in spec.items() if k not in ("params", "optimizer")}
            own = list(spec["params"])
            if own:
                members.append(spec["optimizer"](own, **options))
                covered += own
        if not members:
            raise ValueError("No optimizers created")
        self.optimizers = members
        super().__init__(covered, {"multi_tensor": True})

    def _handle_closure(self, closure):
        # one evaluation serves every member: the first member owns closure handling (and curvature probes)
        return self.optimizers[0]._handle_closure(closure)

    @torch.no_grad()
    def step(self, closure=None):
        loss = None if closure is None else self._handle_closure(closure)
        for member in self.optimizers:
            member.step()
        return loss

    def zero_grad(self, set_to_none: bool = True):
        for member in self.optimizers:
            member.zero_grad(set_to_none=set_to_none)

    def state_dict(self):
        return {"optimizers": [member.state_dict() for member in self.optimizers]}

    def load_state_dict(self, state_dict):
        saved = state_dict["optimizers"]
        if len(saved) != len(self.optimizers):
            raise ValueError(f"checkpoint holds {len(saved)} optimizers, this SplitOpt has {len(self.optimizers)}")
        for member, part in zip(self.optimizers, saved):
            member.load_state_dict(part)


class SAMWrapper(torch.optim.Optimizer):
    """Adaptive SAM (https://arxiv.org/abs/2102.11600) around any optimizer of this package:
    ascent by ``ball * g * p^2``, gradient at the perturbed point, descent from the original point.
    ``step`` requires a closure."""

    def __init__(self, params, wrapped_optimizer: Union[utils.StatefulOptimizer, Type[utils.StatefulOptimizer]] = AdamW,
                 ball: float = 0.1):  # fmt: skip
        params = list(params)
        super().__init__(params, {"ball": ball})
        kind = wrapped_optimizer if isinstance(wrapped_optimizer, type) else type(wrapped_optimizer)
        if not issubclass(kind, utils.StatefulOptimizer):
            raise ValueError(f"{kind.__name__} is not a HeavyBall optimizer")
        self.wrapped_optimizer = wrapped_optimizer(params) if isinstance(wrapped_optimizer, type) else wrapped_optimizer

    @torch.no_grad()
    def step(self, closure=None):
        if closure is None:
            raise ValueError("SAM requires closure")
        with torch.enable_grad():
            closure()  # gradient at the current point, used for the ascent direction only
        originals = [(group["params"], utils.sam_step(group["params"], group["ball"])) for group in self.param_groups]
        inner = self.wrapped_optimizer
        evaluate = inner._handle_closure

        def at_ascent_point_then_restore(c):
            """The wrapped optimizer's closure evaluation happens at the perturbed parameters; they are put back before
            its update runs."""
            try:
                return evaluate(c)
            finally:
                for live, held in originals:
                    utils.copy_stochastic_list_(live, held)

        inner._handle_closure = at_ascent_point_then_restore
        try:
            return inner.step(closure)
        finally:
            inner._handle_closure = evaluate

    def zero_grad(self, set_to_none: bool = True):
        self.wrapped_optimizer.zero_grad(set_to_none=set_to_none)

    def state_dict(self):
        return {"wrapped": self.wrapped_optimizer.state_dict(), "ball": [group["ball"] for group in self.param_groups]}

    def load_state_dict(self, state_dict):
        self.wrapped_optimizer.load_state_dict(state_dict["wrapped"])
        for group, ball in zip(self.param_groups, state_dict["ball"]):
            group["ball"] = ball

    def train(self, mode: bool = True):
        self.wrapped_optimizer.train(mode)
        return self

    def eval(self):
        return self.train(False)


capture_param_shapes = utils.capture_param_shapes
_BASE_CLASSES = {SOAPBase, PSGDBase}
__all__ = ["capture_param_shapes"] + [
    k
    for k, v in list(globals().items())
    if isinstance(v, type) and issubclass(v, torch.optim.Optimizer) and v not in _BASE_CLASSES
]
